"""Integer codes in integer containers: the device kernels against the C restatement of quantizeToFxpPackedCpu /
dequantizeFromPackedFxpCpu (DlQuantization/src/trim_functions.cpp:220-605), which test_oracle_pin.py pins to the
reference's own build."""
import numpy as np
import pytest
import torch

from _data import assert_bits_equal, normal

pytestmark = pytest.mark.gpu

RANGES = ((-3.1, 4.2), (0.0, 5.0), (-2.0, 2.0), (-1e-3, 1e3))


def _values(n, seed):
    edge = np.array([0.0, -0.0, 1e-30, 4.2, -3.1, 4.19, -3.09, 100.0, -100.0, np.inf, -np.inf], np.float32)
    return np.concatenate([normal(n, seed, 2.0, 0.3), edge])


@pytest.mark.parametrize("bw", [1, 2, 4, 8, 16, 32])
@pytest.mark.parametrize("signed", [False, True])
def test_packed_round_trip_matches_oracle(oracle, bw, signed):
    from aimet_b200 import ops
    x = _values(100_003, 11 + bw)
    dx = torch.from_numpy(x).cuda()
    for mn, mx in RANGES:
        want = oracle.quantize_packed(x, mn, mx, bw, signed)
        got = ops.quantize_packed(dx, mn, mx, bw, signed)
        assert got.dtype == getattr(torch, np.dtype(oracle.packed_dtype(bw, signed)).name)
        np.testing.assert_array_equal(got.cpu().numpy(), want, err_msg=f"codes bw={bw} signed={signed} [{mn},{mx}]")
        back = ops.dequantize_packed(got, mn, mx, bw, signed)
        assert_bits_equal(back.cpu().numpy(), oracle.dequantize_packed(want, mn, mx, bw, signed),
                          f"dequantize bw={bw} signed={signed} [{mn},{mx}]")


def test_packed_codes_agree_with_float_container_path(oracle):
    """For 8 bits the integer container holds the same code the float-container quantize() yields plus offset."""
    from aimet_b200 import ops
    x = normal(1 << 20, 5, 1.5, 0.1)
    dx = torch.from_numpy(x).cuda()
    codes = ops.quantize_packed(dx, -4.0, 4.0, 8).cpu().numpy().astype(np.float64)
    enc = oracle.fill_encoding(8, -4.0, 4.0)
    back = ops.dequantize_packed(torch.from_numpy(codes.astype(np.uint8)).cuda(), -4.0, 4.0, 8).cpu().numpy()
    qdq = ops.qdq_per_tensor(dx, -4.0, 4.0, 8, 0).cpu().numpy()
    # the two paths round in different precisions (double here, float there): identical away from ties
    assert np.mean(np.abs(back - qdq) > 2 * np.spacing(np.abs(qdq))) < 1e-4
    assert np.all(np.abs(back - qdq) <= np.float32(enc[2]) * 1.0001)


def test_packed_empty_and_errors():
    from aimet_b200 import ops
    e = torch.empty(0, device="cuda")
    assert ops.quantize_packed(e, -1.0, 1.0, 8).numel() == 0
    with pytest.raises(RuntimeError):
        ops.quantize_packed(torch.ones(4, device="cuda"), -1.0, 1.0, 3)
    with pytest.raises(RuntimeError):
        ops.dequantize_packed(torch.ones(4, device="cuda", dtype=torch.int16), -1.0, 1.0, 8)


def test_libpymo_tensor_quantizer_packed(oracle):
    from aimet_b200 import libpymo
    tq = libpymo.TensorQuantizer(libpymo.QuantizationMode.QUANTIZATION_TF, libpymo.RoundingMode.ROUND_NEAREST)
    x = normal(10_000, 2, 1.0, 0.0)
    codes = tq.quantizeTensorPacked(x, -2.0, 2.0, 4, useStrictSymmetric=True)
    np.testing.assert_array_equal(codes, oracle.quantize_packed(x, -2.0, 2.0, 4, True))
    assert_bits_equal(tq.dequantize(codes, -2.0, 2.0, 4, True), oracle.dequantize_packed(codes, -2.0, 2.0, 4, True))
