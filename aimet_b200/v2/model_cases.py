"""Whole-model measurements for the two model-level benchmark configurations (synthetic data, random weights):

* ``resnet50``: torchvision ResNet-50, He-initialised, batch norms folded; W8 per-channel symmetric, A8 TF-Enhanced
  asymmetric; ``compute_encodings`` over batches of 128 x 3 x 224 x 224 N(0,1) inputs, then one fake-quantized
  forward + backward step.
* ``llama_layer``: the seven weight matrices of a decoder layer (hidden 4096, MLP 11008), N(0, 0.02) in bf16,
  W4 symmetric in blocks of 64 along the input dimension (calibration + fake-quantization of each matrix), and A16
  per-tensor min/max on an [8, 2048, 4096] bf16 activation.

``python bench.py --model-case resnet50|llama_layer`` prints one JSON line with wall-clock numbers (CUDA events
around whole phases: these cases measure the orchestration, the kernels have their own cases).
"""
from __future__ import annotations

import math
from typing import Dict

import torch
from torch import nn

from .quantizer import QuantizeDequantize
from .quantsim import QuantizationSimModel


def _timed(fn, device) -> float:
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1) * 1e-3


def resnet50_case(device, batches: int = 32, batch_size: int = 128,
                  scheme: str = "post_training_tf_enhanced_libpymo") -> Dict:
    import torchvision
    model = torchvision.models.resnet50(weights=None)
    for m in model.modules():
        if isinstance(m, nn.Conv2d):
            nn.init.kaiming_normal_(m.weight, mode="fan_out", nonlinearity="relu")
    model = model.eval().to(device)
    g = torch.Generator(device=device)

    def batch(b):
        g.manual_seed(2000 + b)
        return torch.randn(batch_size, 3, 224, 224, device=device, generator=g)

    sim = QuantizationSimModel(model, batch(0), quant_scheme=scheme)

    def float_pass():
        with torch.no_grad():
            for b in range(batches):
                model(batch(b))

    def calibrate():
        sim.compute_encodings(lambda m, _: [m(batch(b)) for b in range(batches)], None)

    float_pass()                       # warm-up of cuDNN algorithm selection, untimed
    t_float = _timed(float_pass, device)
    calibrate()                        # warm-up (also the first use of every kernel flavour), untimed
    t_cal = _timed(calibrate, device)
    x = batch(0).requires_grad_(True)

    def step():
        sim.model.zero_grad(set_to_none=True)
        sim.model(x).square().mean().backward()

    step()
    t_step = _timed(step, device)
    n = batches * batch_size
    return {"model_case": "resnet50", "quant_scheme": scheme, "batches": batches, "batch_size": batch_size,
            "weight_quantizers": len(sim.layers), "activation_quantizers": len(sim.activation_quantizers),
            "compute_encodings_s": t_cal, "calibration_samples_per_s": n / t_cal,
            "float_forward_only_s": t_float, "float_forward_samples_per_s": n / t_float,
            "calibration_overhead_vs_float_forward": t_cal / t_float,
            "fake_quant_fwd_bwd_step_s": t_step}


def llama_layer_case(device) -> Dict:
    shapes = {"q_proj": (4096, 4096), "k_proj": (4096, 4096), "v_proj": (4096, 4096), "o_proj": (4096, 4096),
              "gate_proj": (11008, 4096), "up_proj": (11008, 4096), "down_proj": (4096, 11008)}
    g = torch.Generator(device=device).manual_seed(0)
    weights = {k: (torch.randn(*s, device=device, generator=g) * 0.02).to(torch.bfloat16) for k, s in shapes.items()}
    quantizers = {k: QuantizeDequantize((s[0], s[1] // 64), 4, True, block_size=(-1, 64)).to(device)
                  for k, s in shapes.items()}
    act = torch.randn(8, 2048, 4096, device=device, generator=g).to(torch.bfloat16)
    aq = QuantizeDequantize((), 16, False).to(device)

    def calibrate():
        with torch.no_grad():
            for k, q in quantizers.items():
                with q.compute_encodings():
                    q(weights[k])
            with aq.compute_encodings():
                aq(act)

    def fake_quant():
        with torch.no_grad():
            for k, q in quantizers.items():
                q(weights[k])
            aq(act)

    calibrate()
    t_cal = _timed(calibrate, device)
    fake_quant()
    t_fq = _timed(fake_quant, device)
    n_w = sum(math.prod(s) for s in shapes.values())
    bytes_fq = 4 * n_w + 8 * (n_w // 64) + 4 * act.numel()          # bf16 in + out, fp32 scale + offset per block
    bytes_cal = 2 * n_w + 2 * act.numel() + bytes_fq                # + one min/max pass (calibration also fake-quantizes)
    return {"model_case": "llama_layer", "weight_elements": n_w, "activation_elements": act.numel(),
            "calibrate_s": t_cal, "calibrate_GBps": bytes_cal / t_cal / 1e9,
            "fake_quant_s": t_fq, "fake_quant_GBps": bytes_fq / t_fq / 1e9,
            "algorithmic_bytes_fake_quant": bytes_fq, "algorithmic_bytes_calibrate": bytes_cal}


CASES = {"resnet50": resnet50_case, "llama_layer": llama_layer_case}
