"""Bit parity at the full sizes of the five benchmark configurations (synthetic inputs with the shapes, dtypes and
value distributions of those configurations), CUDA path against the CPU oracle."""
import math

import numpy as np
import pytest
import torch

from _data import assert_bits_equal

pytestmark = pytest.mark.gpu
F32 = np.float32


def _scale_offset(mn, mx, qmin, qmax, symmetric):
    """MinMaxQuantizer.get_scale / get_offset in float32 (affine/quantizer.py:404-437)."""
    mn, mx = np.asarray(mn, np.float32), np.asarray(mx, np.float32)
    scale = ((mx - mn) / F32(qmax - qmin)).astype(np.float32)
    if symmetric:
        return scale, np.zeros_like(scale)
    with np.errstate(all="ignore"):
        return scale, (np.rint((mn / scale).astype(np.float32)) - F32(qmin)).astype(np.float32)


def test_config1_per_tensor_a8_forward_backward(cuda, oracle):
    """[32,64,56,56] fp32 N(0,1), 8-bit asymmetric, MinMax encoding: v2 semantics and libpymo semantics."""
    from oracle import v2_oracle as v2
    from aimet_b200 import libpymo
    from aimet_b200.v2.quantizer import QuantizeDequantize
    g = torch.Generator().manual_seed(0)
    x = torch.randn(32, 64, 56, 56, generator=g)
    gy = torch.randn(32, 64, 56, 56, generator=g)
    xn = x.numpy()
    # --- v2 ---
    q = QuantizeDequantize((), 8, False).to(cuda)
    xd = x.to(cuda).requires_grad_(True)
    with q.compute_encodings():
        q(xd.detach())
    emn, emx = v2.minmax_encodings(xn.min(), xn.max(), 255, False)
    assert_bits_equal(q.min.detach().cpu().numpy().reshape(()), np.asarray(emn, np.float32).reshape(()), "min")
    sc, of = _scale_offset(emn, emx, 0, 255, False)
    want, wmask = v2.quantize_dequantize(xn, sc, of, 0, 255, None, "float32")
    y = q(xd)
    assert_bits_equal(y.detach().cpu().numpy(), want, "qdq")
    y.backward(gy.to(cuda))
    assert_bits_equal(xd.grad.cpu().numpy(), (gy.numpy() * wmask).astype(np.float32), "dx")
    # --- libpymo: MinMax ("TF") analyzer, QDQ with half-away rounding, STE backward ---
    tq = libpymo.AimetTensorQuantizer(libpymo.QuantizationMode.QUANTIZATION_TF)
    tq.updateStats(x.to(cuda), True)
    enc, valid = tq.getEncoding(8, False, False, False)
    assert valid
    oenc = oracle.minmax_encoding(8, float(xn.min()), float(xn.max()), False, False, False)
    assert [enc.min, enc.max, enc.delta, enc.offset] == [float(v) for v in oenc]
    out = tq.quantizeDequantize(x.to(cuda), enc, libpymo.RoundingMode.ROUND_NEAREST, True)
    assert_bits_equal(out.cpu().numpy(), oracle.qdq_per_tensor(xn.reshape(-1), enc.min, enc.max, 8).reshape(xn.shape), "libpymo qdq")


def test_config2_per_channel_w8_symmetric(cuda, oracle):
    """[512,256,3,3] fp32 Kaiming-normal weights with the 1 % largest entries x8; per-output-channel symmetric."""
    from oracle import v2_oracle as v2
    from aimet_b200.v2.quantizer import QuantizeDequantize
    g = torch.Generator().manual_seed(0)
    w = torch.randn(512, 256, 3, 3, generator=g) * math.sqrt(2.0 / 2304)
    k = math.ceil(0.01 * w.numel())
    idx = torch.topk(w.abs().reshape(-1), k).indices
    w.view(-1)[idx] *= 8
    gy = torch.randn(512, 256, 3, 3, generator=g)
    wn = w.numpy()
    q = QuantizeDequantize((512, 1, 1, 1), 8, True).to(cuda)
    wd = w.to(cuda).requires_grad_(True)
    with q.compute_encodings():
        q(wd.detach())
    mn = wn.reshape(512, -1).min(axis=1).reshape(512, 1, 1, 1)
    mx = wn.reshape(512, -1).max(axis=1).reshape(512, 1, 1, 1)
    emn, emx = v2.minmax_encodings(mn, mx, 255, True)
    assert_bits_equal(q.min.detach().cpu().numpy(), emn, "min")
    assert_bits_equal(q.max.detach().cpu().numpy(), emx, "max")
    sc, of = _scale_offset(emn, emx, -128, 127, True)
    want, wmask = v2.quantize_dequantize(wn, sc, of, -128, 127, None, "float32")
    y = q(wd)
    assert_bits_equal(y.detach().cpu().numpy(), want, "qdq")
    y.backward(gy.to(cuda))
    assert_bits_equal(wd.grad.cpu().numpy(), (gy.numpy() * wmask).astype(np.float32), "dx")


def test_config3_tf_enhanced_256_batches(cuda, oracle):
    """256 batches of [64,256,28,28] ReLU(N(0,1)) with 0.1 % outliers x20: histogram rows, PDF and the chosen
    8-bit asymmetric encoding equal the sequential CPU analyzer's, bit for bit."""
    import bench
    from oracle import OracleTfeAnalyzer
    from aimet_b200.calibration import TfEnhancedCalibrator
    cal = TfEnhancedCalibrator(cuda)
    ref = OracleTfeAnalyzer(oracle)
    nb = 256
    for b in range(nb):
        x = bench.device_batch(b, cuda)
        cal.update(x)
        ref.update(x.reshape(-1).cpu().numpy())
    enc = cal.compute_encoding(8, False, False, False)
    want = ref.compute(8, False, False, False)
    assert [enc.min, enc.max, enc.delta, enc.offset] == [float(v) for v in want[:4]]
    pdf = cal.engine.state.pdf.cpu().numpy()
    assert_bits_equal(pdf, np.asarray(ref.pdf, np.float64), "pdf")
    total = cal.engine.state.hists[:nb].to(torch.int64).sum().item()
    assert 0 < total <= nb * 64 * 256 * 28 * 28


@pytest.mark.parametrize("shape", [(4096, 11008), (11008, 4096), (4096, 4096)])
def test_config5_blockwise_w4_bf16_weights(cuda, shape):
    """Decoder-layer weights, N(0, 0.02) in bf16, W4 symmetric, blocks of 64 along the input dimension."""
    from oracle import v2_oracle as v2
    from aimet_b200.v2.quantizer import QuantizeDequantize
    g = torch.Generator().manual_seed(shape[0] + shape[1])
    w = (torch.randn(*shape, generator=g) * 0.02).to(torch.bfloat16)
    enc_shape = (shape[0], shape[1] // 64)
    q = QuantizeDequantize(enc_shape, 4, True, block_size=(-1, 64)).to(cuda)
    wd = w.to(cuda)
    with torch.no_grad():
        with q.compute_encodings():
            q(wd)
        y = q(wd)
    wn = w.float().numpy()
    blocks = wn.reshape(shape[0], shape[1] // 64, 64)
    emn, emx = v2.minmax_encodings(blocks.min(axis=2), blocks.max(axis=2), 15, True, "bfloat16")
    assert_bits_equal(q.min.detach().cpu().numpy(), emn.astype(np.float32), "min")
    assert_bits_equal(q.max.detach().cpu().numpy(), emx.astype(np.float32), "max")
    sc, of = _scale_offset(emn, emx, -8, 7, True)
    want, _ = v2.quantize_dequantize(wn, sc, of, -8, 7, (-1, 64), "bfloat16")
    assert_bits_equal(y.float().cpu().numpy(), want, "qdq")


def test_config5_a16_per_tensor_bf16_activations(cuda):
    """Activations [8,2048,4096] bf16 N(0,1), 16-bit asymmetric per-tensor MinMax."""
    from oracle import v2_oracle as v2
    from aimet_b200.v2.quantizer import QuantizeDequantize
    g = torch.Generator().manual_seed(1)
    a = torch.randn(8, 2048, 4096, generator=g).to(torch.bfloat16)
    q = QuantizeDequantize((), 16, False).to(cuda)
    ad = a.to(cuda)
    with torch.no_grad():
        with q.compute_encodings():
            q(ad)
        y = q(ad)
    an = a.float().numpy()
    emn, emx = v2.minmax_encodings(an.min(), an.max(), 65535, False, "bfloat16")
    assert_bits_equal(q.min.detach().cpu().numpy().reshape(()), np.asarray(emn, np.float32).reshape(()), "min")
    assert_bits_equal(q.max.detach().cpu().numpy().reshape(()), np.asarray(emx, np.float32).reshape(()), "max")
    sc, of = _scale_offset(emn, emx, 0, 65535, False)
    want, _ = v2.quantize_dequantize(an, sc, of, 0, 65535, None, "bfloat16")
    assert_bits_equal(y.float().cpu().numpy(), want, "qdq")
