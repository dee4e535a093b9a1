"""GPU tests of the v1 static-grid quantizer wrappers, the percentile scheme and the numpy-facing libpymo mirrors,
each against the CPU oracle (which is pinned to the reference's own code in test_oracle_pin.py)."""
import numpy as np
import pytest
import torch

from _data import assert_bits_equal, conv_weight, normal, relu_activations

pytestmark = pytest.mark.gpu


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def enc5(e):
    return np.array([e.min, e.max, e.delta, e.offset, e.bw], np.float64)


@pytest.mark.parametrize("scheme", ["tf", "tf_enhanced", "percentile"])
def test_per_tensor_quantizer_calibration_and_fake_quant(oracle, cuda, scheme):
    from oracle import OracleTfeAnalyzer
    from aimet_b200 import libpymo
    from aimet_b200.v1.tensor_quantizer import QuantScheme, StaticGridPerTensorQuantizer
    qs = {"tf": QuantScheme.post_training_tf, "tf_enhanced": QuantScheme.post_training_tf_enhanced,
          "percentile": QuantScheme.post_training_percentile}[scheme]
    q = StaticGridPerTensorQuantizer(8, libpymo.ROUND_NEAREST, qs, use_symmetric_encodings=False, enabled_by_default=True)
    if scheme == "percentile":
        q.set_percentile_value(99.9)
    batches = [relu_activations((4, 8, 20, 20), 70 + b) for b in range(3)]
    oa = OracleTfeAnalyzer(oracle)
    for b in batches:
        q.update_encoding_stats(dev(b, cuda))
        oa.update(b.reshape(-1))
    q.compute_encoding()
    if scheme == "tf":
        mn, mx = min(b.min() for b in batches), max(b.max() for b in batches)
        want = np.append(oracle.minmax_encoding(8, float(mn), float(mx)), 8)
    elif scheme == "tf_enhanced":
        want = oa.compute(8, False, False, False)
    else:
        want = oa.compute_percentile(99.9, 8, False, False, False)
    assert_bits_equal(enc5(q.encoding), want, scheme)
    # fake-quant forward + straight-through backward through the wrapper
    x = normal((4, 8, 20, 20), 5, 2.0, 1.0)
    g = normal((4, 8, 20, 20), 6)
    xd = dev(x, cuda).requires_grad_(True)
    y = q.quantize_dequantize(xd, libpymo.ROUND_NEAREST)
    y.backward(dev(g, cuda))
    e = q.encoding
    assert_bits_equal(y.detach().cpu().numpy(), oracle.qdq_per_tensor(x, e.min, e.max, 8), "qdq")
    assert_bits_equal(xd.grad.cpu().numpy().reshape(-1),
                      oracle.ste_bwd(x.reshape(-1), g.reshape(-1), np.float32(e.min), np.float32(e.max)), "dx")
    # half-precision input is upcast and cast back, as in the reference
    yh = q.quantize_dequantize(dev(x, cuda).half(), libpymo.ROUND_NEAREST)
    assert yh.dtype == torch.float16
    assert_bits_equal(yh.float().cpu().numpy(),
                      oracle.qdq_per_tensor(x.astype(np.float16).astype(np.float32), e.min, e.max, 8).astype(np.float16).astype(np.float32))
    # integer codes (signed by default in quantize-only mode)
    codes = q.quantize(dev(x, cuda), libpymo.ROUND_NEAREST).cpu().numpy()
    assert_bits_equal(codes, oracle.quantize_per_tensor(x, e.min, e.max, 8, True), "codes")
    if scheme == "tf_enhanced":
        hist = q.get_stats_histogram()
        assert len(hist) == 1 and len(hist[0]) == 512
    q.reset_encoding_stats()
    assert q.encoding is None


@pytest.mark.parametrize("axis,shape", [(0, (32, 16, 3, 3)), (1, (6, 10, 7, 5)), (0, (24, 40))])
@pytest.mark.parametrize("symmetric", [True, False])
def test_per_channel_quantizer_one_launch_calibration(oracle, cuda, axis, shape, symmetric):
    """Per-channel min/max calibration is one fused launch over the whole tensor; the encodings must be what the
    reference gets from one analyzer per channel slice."""
    from aimet_b200 import libpymo
    from aimet_b200.v1.tensor_quantizer import QuantScheme, StaticGridPerChannelQuantizer
    w1 = conv_weight(shape, 1) if len(shape) == 4 else normal(shape, 1, 0.1)
    w2 = (w1 * 1.5 + 0.01).astype(np.float32)
    C = shape[axis]
    q = StaticGridPerChannelQuantizer(8, libpymo.ROUND_NEAREST, QuantScheme.post_training_tf, symmetric, C, True, axis)
    for w in (w1, w2):
        q.update_encoding_stats(dev(w, cuda))
    q.compute_encoding()
    assert len(q.encoding) == C
    for c in range(C):
        a, b = np.take(w1, c, axis=axis), np.take(w2, c, axis=axis)
        mn, mx = min(a.min(), b.min()), max(a.max(), b.max())
        want = oracle.minmax_encoding(8, float(mn), float(mx), symmetric, False, True)
        assert_bits_equal(enc5(q.encoding[c])[:4], want, f"channel {c}")
    # forward: per-channel grid derived in the kernel from the encodings' min / max
    x = w1
    xd = dev(x, cuda).requires_grad_(True)
    y = q.quantize_dequantize(xd, libpymo.ROUND_NEAREST)
    mins = np.array([e.min for e in q.encoding], np.float64)
    maxs = np.array([e.max for e in q.encoding], np.float64)
    inner = int(np.prod(shape[axis + 1:]))
    grid = oracle.per_channel_grid(mins, maxs, 8)
    want = oracle.qdq_per_channel(x.reshape(-1), C, inner, *grid)
    assert_bits_equal(y.detach().cpu().numpy().reshape(-1), want, "per-channel qdq")
    g = normal(shape, 9)
    y.backward(dev(g, cuda))
    rows_x, rows_g = x.reshape(-1, inner), g.reshape(-1, inner)
    want_dx = np.stack([oracle.ste_bwd(rows_x[r], rows_g[r], np.float32(mins[r % C]), np.float32(maxs[r % C]))
                        for r in range(rows_x.shape[0])]).reshape(shape)
    assert_bits_equal(xd.grad.cpu().numpy(), want_dx, "per-channel dx")


def test_per_channel_tf_enhanced_uses_one_analyzer_per_channel(oracle, cuda):
    from oracle import OracleTfeAnalyzer
    from aimet_b200 import libpymo
    from aimet_b200.v1.tensor_quantizer import QuantScheme, StaticGridPerChannelQuantizer
    w = conv_weight((6, 16, 3, 3), 4)
    q = StaticGridPerChannelQuantizer(8, libpymo.ROUND_NEAREST, QuantScheme.post_training_tf_enhanced, True, 6, True, 0)
    q.update_encoding_stats(dev(w, cuda))
    q.compute_encoding()
    for c in range(6):
        oa = OracleTfeAnalyzer(oracle)
        oa.update(w[c].reshape(-1))
        assert_bits_equal(enc5(q.encoding[c]), oa.compute(8, True, False, True), f"channel {c}")


@pytest.mark.parametrize("kinds", [("relu",) * 3, ("zeros", "relu"), ("zeros",)])
@pytest.mark.parametrize("pct", [100.0, 99.99, 99.0, 50.0])
def test_percentile_scheme_matches_oracle(oracle, cuda, kinds, pct):
    from oracle import OracleTfeAnalyzer
    from aimet_b200 import libpymo
    gens = {"relu": lambda s: relu_activations(50001, s), "zeros": lambda s: np.zeros(3000, np.float32)}
    batches = [gens[k](11 + i) for i, k in enumerate(kinds)]
    q = libpymo.AimetTensorQuantizer(libpymo.QUANTIZATION_PERCENTILE)
    q.setPercentileValue(pct)
    oa = OracleTfeAnalyzer(oracle)
    for b in batches:
        q.updateStats(dev(b, cuda), True)
        oa.update(b)
    for bw, sym, strict, uns in ((8, False, False, False), (8, True, False, False), (4, True, True, False), (16, True, False, True)):
        enc, valid = q.getEncoding(bw, sym, strict, uns)
        assert valid
        assert_bits_equal(enc5(enc), oa.compute_percentile(pct, bw, sym, strict, uns), f"pct={pct} bw={bw} {sym}{strict}{uns}")


@pytest.mark.parametrize("kinds", [("relu",) * 3, ("normal",) * 2, ("zeros", "relu"), ("zeros",), ("neg", "neg")])
def test_mse_scheme_matches_oracle(oracle, cuda, kinds):
    """MseEncodingAnalyzer on the device against the C restatement (which test_oracle_pin.py pins to the reference)."""
    from oracle import OracleTfeAnalyzer
    from aimet_b200 import libpymo
    gens = {"relu": lambda s: relu_activations(50001, s), "zeros": lambda s: np.zeros(3000, np.float32),
            "normal": lambda s: normal(40000, s, 2.0, 1.0), "neg": lambda s: normal(40000, s, 1.0, -6.0)}
    batches = [gens[k](21 + i) for i, k in enumerate(kinds)]
    q = libpymo.AimetTensorQuantizer(libpymo.QUANTIZATION_MSE)
    oa = OracleTfeAnalyzer(oracle)
    for b in batches:
        q.updateStats(dev(b, cuda), True)
        oa.update(b)
    for bw, sym, strict, uns in ((8, False, False, False), (8, True, False, False), (4, False, False, False),
                                 (4, True, True, False), (16, True, False, True), (2, False, False, False)):
        enc, valid = q.getEncoding(bw, sym, strict, uns)
        assert valid
        assert_bits_equal(enc5(enc), oa.compute_mse(bw, sym, strict, uns), f"mse bw={bw} {sym}{strict}{uns}")


def test_numpy_facing_mirrors(oracle, cuda):
    from oracle import OracleTfeAnalyzer
    from aimet_b200 import libpymo
    x = relu_activations(40000, 3)
    an = libpymo.EncodingAnalyzerForPython(libpymo.QUANTIZATION_TF_ENHANCED)
    enc, valid = an.computeEncoding(8, False, False, False)
    assert not valid
    an.updateStats(x, True)
    enc, valid = an.computeEncoding(8, False, False, False)
    oa = OracleTfeAnalyzer(oracle)
    oa.update(x)
    assert valid
    assert_bits_equal(enc5(enc), oa.compute(8, False, False, False))
    sim = libpymo.TensorQuantizationSimForPython()
    y = sim.quantizeDequantize(x.reshape(200, 200), enc, libpymo.ROUND_NEAREST, True)
    assert y.shape == (200, 200)
    assert_bits_equal(y.reshape(-1), oracle.qdq_per_tensor(x, enc.min, enc.max, 8))
    y4 = sim.quantizeDequantize(x, enc, libpymo.ROUND_NEAREST, 4, True)
    assert_bits_equal(y4, oracle.qdq_per_tensor(x, enc.min, enc.max, 4))
    tq = libpymo.TensorQuantizer(libpymo.QUANTIZATION_PERCENTILE, libpymo.ROUND_NEAREST)
    tq.setPercentileValue(99.5)
    assert tq.getPercentileValue() == 99.5
    tq.updateStats(x, True)
    e = tq.computeEncoding(8, False)
    assert_bits_equal(enc5(e), oa.compute_percentile(99.5, 8, False, False, False))
    p = libpymo.TfEncoding(delta=0.5, offset=-10.0, bw=8)
    tq.computePartialEncoding(8, p, False, False, False)
    assert (p.min, p.max) == (-5.0, 122.5)


def test_fp16_fake_quant_is_the_double_cast(cuda):
    """aq_qdq_fp16 against float(half(x)) computed by torch on the CPU: ties, subnormals of half, overflow to inf."""
    from aimet_b200 import ops
    edge = np.array([0.0, -0.0, 1.0, 65504.0, 65519.9, 65520.0, -65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5,
                     1.0009765625, 1.00048828125, 1.000732421875, np.inf, -np.inf, np.nan, 3.1415927], np.float32)
    x = np.concatenate([normal(100_003, 9, 30.0, 0.0), normal(5000, 10, 1e-6, 0.0), edge])
    want = torch.from_numpy(x).half().float().numpy()
    got = ops.qdq_fp16(dev(x, cuda)).cpu().numpy()
    assert_bits_equal(got, want, "fp16 fake-quant")
    got1 = ops.qdq_fp16(dev(x, cuda)[1:]).cpu().numpy()   # unaligned view: scalar path
    assert_bits_equal(got1, want[1:], "fp16 fake-quant, unaligned")

