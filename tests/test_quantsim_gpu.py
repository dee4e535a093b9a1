"""Whole-model quantization simulation: placement of quantizers (CPU) and, on the GPU, that every quantizer of a
calibrated ResNet ends up with the encoding the CPU reference analyzers derive from the very tensors it saw."""
import numpy as np
import pytest
import torch
from torch import nn

from _data import assert_bits_equal


def _resnet(kind="resnet18"):
    import torchvision
    m = getattr(torchvision.models, kind)(weights=None)
    g = torch.Generator().manual_seed(0)
    for mod in m.modules():
        if isinstance(mod, nn.Conv2d):
            fan_out = mod.weight.shape[0] * mod.weight.shape[2] * mod.weight.shape[3]
            with torch.no_grad():
                mod.weight.copy_(torch.randn(mod.weight.shape, generator=g) * (2.0 / fan_out) ** 0.5)
        if isinstance(mod, nn.BatchNorm2d):   # non-trivial statistics so that folding is exercised
            with torch.no_grad():
                mod.running_mean.copy_(torch.randn(mod.running_mean.shape, generator=g) * 0.1)
                mod.running_var.copy_(torch.rand(mod.running_var.shape, generator=g) + 0.5)
                mod.weight.copy_(torch.rand(mod.weight.shape, generator=g) + 0.5)
                mod.bias.copy_(torch.randn(mod.bias.shape, generator=g) * 0.1)
    return m.eval()


def test_resnet50_placement_and_bn_folding():
    from aimet_b200.v2.quantsim import QuantizationSimModel
    m = _resnet("resnet50")
    sim = QuantizationSimModel(m)
    assert len(sim.layers) == 54                      # 53 convolutions + the classifier
    assert not any(isinstance(x, nn.BatchNorm2d) for x in sim.model.modules())
    names = set(sim.activation_quantizers)
    assert "act_q_x" in names and "act_q_fc" in names and "act_q_avgpool" in names
    assert "act_q_layer1_0_downsample_0" in names     # no ReLU follows: quantized at the convolution
    assert "act_q_layer1_0_conv1" not in names        # ReLU follows: quantized after the ReLU
    assert "act_q_layer1_0_relu" in names and "act_q_layer1_0_relu_2" in names   # the shared ReLU: one per call
    # folding keeps the function (float model, CPU)
    x = torch.randn(2, 3, 64, 64)
    import copy
    from torch import fx
    from aimet_b200.v2.quantsim import fold_batch_norms
    gm = fx.symbolic_trace(copy.deepcopy(m))
    assert fold_batch_norms(gm) == 53
    torch.testing.assert_close(gm(x), m(x), rtol=2e-3, atol=2e-3)


@pytest.mark.gpu
def test_resnet18_every_quantizer_matches_cpu_reference(cuda, oracle):
    from oracle import OracleTfeAnalyzer, v2_oracle as v2
    from aimet_b200.v2.quantsim import QuantizationSimModel
    m = _resnet("resnet18").to(cuda)
    g = torch.Generator().manual_seed(3)
    batches = [torch.randn(4, 3, 64, 64, generator=g).to(cuda) for _ in range(2)]
    sim = QuantizationSimModel(m, batches[0], quant_scheme="post_training_tf_enhanced_libpymo")
    seen = {name: [] for name in sim.activation_quantizers}
    hooks = [q.register_forward_pre_hook(lambda mod, args, n=name: seen[n].append(args[0].detach().float().cpu().numpy().reshape(-1)))
             for name, q in sim.activation_quantizers.items()]

    def run(model, data):
        for x in data:
            model(x)

    sim.compute_encodings(run, batches)
    for h in hooks:
        h.remove()
    # activations: TF-Enhanced over the tensors that reached each quantizer, in order
    for name, q in sim.activation_quantizers.items():
        assert len(seen[name]) == len(batches)
        ref = OracleTfeAnalyzer(oracle)
        for t in seen[name]:
            ref.update(t)
        want = ref.compute(8, False, False, False)
        assert q.is_initialized(), name
        assert float(q.min.detach()) == float(np.float32(want[0])) and float(q.max.detach()) == float(np.float32(want[1])), name
    # weights: per-output-channel symmetric min/max of the folded weights
    for name, layer in sim.layers.items():
        w = layer.layer.weight.detach().cpu().numpy()
        flat = w.reshape(w.shape[0], -1)
        shape = (w.shape[0],) + (1,) * (w.ndim - 1)
        emn, emx = v2.minmax_encodings(flat.min(axis=1).reshape(shape), flat.max(axis=1).reshape(shape), 255, True)
        wq = layer.param_quantizers["weight"]
        assert_bits_equal(wq.min.detach().cpu().numpy(), emn, name + " min")
        assert_bits_equal(wq.max.detach().cpu().numpy(), emx, name + " max")
    # the calibrated model runs forward and backward
    x = batches[0].clone().requires_grad_(True)
    y = sim.model(x)
    assert y.shape == (4, 1000) and torch.isfinite(y).all()
    y.square().mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
    first = sim.layers["conv1"]
    assert first.layer.weight.grad is not None and first.param_quantizers["weight"].min.grad is not None


@pytest.mark.gpu
def test_resnet50_full_size_every_quantizer_matches_cpu_reference(cuda, oracle):
    """Benchmark configuration 4 at its real size: ResNet-50, batches of 128 x 3 x 224 x 224 (two of them), W8 per
    channel symmetric / A8 TF-Enhanced.  Every activation quantizer must end with the encoding the CPU reference
    analyzer derives from the very tensors it saw (fed to the analyzer as they pass, batch by batch), every weight
    quantizer with the per-channel min/max encoding of the folded weights."""
    from oracle import OracleTfeAnalyzer, v2_oracle as v2
    from aimet_b200.v2.quantsim import QuantizationSimModel
    m = _resnet("resnet50").to(cuda)
    g = torch.Generator(device=cuda)
    batches = []
    for b in range(2):
        g.manual_seed(2000 + b)
        batches.append(torch.randn(128, 3, 224, 224, device=cuda, generator=g))
    sim = QuantizationSimModel(m, batches[0], quant_scheme="post_training_tf_enhanced_libpymo")
    assert len(sim.layers) == 54 and len(sim.activation_quantizers) == 73
    refs = {name: OracleTfeAnalyzer(oracle) for name in sim.activation_quantizers}
    fed = {name: 0 for name in sim.activation_quantizers}

    def feed(name, t):
        refs[name].update(t.detach().float().cpu().numpy().reshape(-1))
        fed[name] += 1

    hooks = [q.register_forward_pre_hook(lambda mod, args, n=name: feed(n, args[0]))
             for name, q in sim.activation_quantizers.items()]
    sim.compute_encodings(lambda model, data: [model(x) for x in data], batches)
    for h in hooks:
        h.remove()
    for name, q in sim.activation_quantizers.items():
        assert fed[name] == len(batches), name
        want = refs[name].compute(8, False, False, False)
        assert q.is_initialized(), name
        assert float(q.min.detach()) == float(np.float32(want[0])) and float(q.max.detach()) == float(np.float32(want[1])), name
    for name, layer in sim.layers.items():
        w = layer.layer.weight.detach().cpu().numpy()
        flat = w.reshape(w.shape[0], -1)
        shape = (w.shape[0],) + (1,) * (w.ndim - 1)
        emn, emx = v2.minmax_encodings(flat.min(axis=1).reshape(shape), flat.max(axis=1).reshape(shape), 255, True)
        wq = layer.param_quantizers["weight"]
        assert_bits_equal(wq.min.detach().cpu().numpy(), emn, name + " min")
        assert_bits_equal(wq.max.detach().cpu().numpy(), emx, name + " max")
    # one fake-quantized forward + backward step at full size
    x = batches[0].requires_grad_(True)
    y = sim.model(x)
    assert y.shape == (128, 1000) and torch.isfinite(y).all()
    y.square().mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()


@pytest.mark.gpu
def test_resnet18_v2_tf_enhanced_uses_sqnr_analyzers(cuda):
    """quant_scheme="post_training_tf_enhanced" is the reference's v2 mapping: SqnrEncodingAnalyzer for parameters
    (one histogram per output channel) and activations.  Every quantizer must end with what a stand-alone analyzer
    (pinned bit for bit to the reference's class in test_v2_sqnr_gpu.py) computes from the tensors it saw."""
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    from aimet_b200.v2.quantsim import QuantizationSimModel
    m = _resnet("resnet18").to(cuda)
    g = torch.Generator().manual_seed(3)
    batches = [torch.randn(4, 3, 64, 64, generator=g).to(cuda) for _ in range(2)]
    sim = QuantizationSimModel(m, batches[0], quant_scheme="post_training_tf_enhanced")
    assert all(isinstance(q.encoding_analyzer, SqnrEncodingAnalyzer) for q in sim.quantizers())
    refs = {name: SqnrEncodingAnalyzer(()) for name in sim.activation_quantizers}
    def feed(name, t):
        refs[name].update_stats(t.detach().clone())   # (a pre-hook's return value would replace the input)

    hooks = [q.register_forward_pre_hook(lambda mod, args, n=name: feed(n, args[0]))
             for name, q in sim.activation_quantizers.items()]
    sim.compute_encodings(lambda model, data: [model(x) for x in data], batches)
    for h in hooks:
        h.remove()
    for name, q in sim.activation_quantizers.items():
        mn, mx = refs[name].compute_encodings(255, False)
        assert q.is_initialized(), name
        assert torch.equal(q.min.detach(), mn) and torch.equal(q.max.detach(), mx), name
    for name, layer in list(sim.layers.items())[:6]:
        w = layer.layer.weight.detach()
        shape = (w.shape[0],) + (1,) * (w.dim() - 1)
        ref = SqnrEncodingAnalyzer(shape)
        ref.update_stats(w)
        mn, mx = ref.compute_encodings(255, True)
        wq = layer.param_quantizers["weight"]
        assert torch.equal(wq.min.detach(), mn) and torch.equal(wq.max.detach(), mx), name
    x = batches[0].clone().requires_grad_(True)
    y = sim.model(x)
    assert y.shape == (4, 1000) and torch.isfinite(y).all()
    y.square().mean().backward()
    assert x.grad is not None and torch.isfinite(x.grad).all()
