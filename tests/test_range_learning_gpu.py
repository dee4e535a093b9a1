"""GPU parity of the learned-grid (range learning) forward / backward against fixtures produced by the reference's
``calculate_forward_pass`` / ``calculate_gradients`` (tests/golden/gen_golden.py:gen_range_learning)."""
import os
import types

import numpy as np
import pytest
import torch

from _data import assert_bits_equal

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def _names():
    g = np.load(os.path.join(GOLDEN, "v1_range_learning.npz"))
    return sorted({k.split("/")[0] for k in g.files})


@pytest.mark.gpu
@pytest.mark.parametrize("name", _names())
def test_forward_and_gradients_match_reference_fixture(cuda, name):
    from aimet_b200.range_learning import QuantizeDequantizeFunc
    g = np.load(os.path.join(GOLDEN, "v1_range_learning.npz"))
    dt = DT[str(g[f"{name}/dtype"])]
    bw, sym, strict, unsigned, axis = (int(v) for v in g[f"{name}/cfg"])
    q = types.SimpleNamespace(bitwidth=bw, use_symmetric_encodings=bool(sym), use_strict_symmetric=bool(strict),
                              is_unsigned_symmetric=bool(unsigned), channel_axis=axis)
    x = torch.from_numpy(g[f"{name}/x"]).to(cuda).to(dt).requires_grad_(True)
    emin = torch.from_numpy(g[f"{name}/min"]).to(cuda).to(dt).requires_grad_(True)
    emax = torch.from_numpy(g[f"{name}/max"]).to(cuda).to(dt).requires_grad_(True)
    y = QuantizeDequantizeFunc.apply(x, emin, emax, q)
    assert y.dtype == dt
    assert_bits_equal(y.detach().float().cpu().numpy(), g[f"{name}/y"], "output")
    y.backward(torch.from_numpy(g[f"{name}/gy"]).to(cuda).to(dt))
    assert_bits_equal(x.grad.float().cpu().numpy(), g[f"{name}/dx"], "dx")
    # sums over the tensor: the reduction order is not the reference's; 16-bit cases also differ in that the
    # reference accumulates in the 16-bit type
    want_min, want_max = g[f"{name}/dmin"], g[f"{name}/dmax"]
    if dt == torch.float32:
        scale = max(np.abs(want_min).max(), np.abs(want_max).max(), 1e-3)
        np.testing.assert_allclose(emin.grad.cpu().numpy(), want_min, rtol=3e-4, atol=3e-4 * scale)
        np.testing.assert_allclose(emax.grad.cpu().numpy(), want_max, rtol=3e-4, atol=3e-4 * scale)
    else:
        assert emin.grad.shape == emin.shape and torch.isfinite(emin.grad.float()).all()


@pytest.mark.gpu
def test_large_tensor_against_plain_tensor_expressions(cuda):
    """[32,64,56,56] fp32: the fused path equals the reference's expression sequence evaluated with tensor operations
    on the same device (outputs and dx bit for bit, min / max gradients to summation tolerance)."""
    from aimet_b200.range_learning import QuantizeDequantizeFunc, get_computed_encodings
    g = torch.Generator(device=cuda).manual_seed(5)
    x = torch.randn(32, 64, 56, 56, device=cuda, generator=g).requires_grad_(True)
    gy = torch.randn(32, 64, 56, 56, device=cuda, generator=g)
    emin = torch.tensor([-2.7], device=cuda, requires_grad=True)
    emax = torch.tensor([3.1], device=cuda, requires_grad=True)
    q = types.SimpleNamespace(bitwidth=8, use_symmetric_encodings=False, use_strict_symmetric=False,
                              is_unsigned_symmetric=False, channel_axis=0)
    y = QuantizeDequantizeFunc.apply(x, emin, emax, q)
    y.backward(gy)
    with torch.no_grad():
        delta, offset, steps = get_computed_encodings(8, emin, emax, False, False, False)
        xr = torch.round(x / delta) - offset
        xq = xr.clamp(torch.zeros_like(steps), steps)
        want = (xq + offset) * delta
        mask = xr.ge(0) * xr.le(steps)
        gs = ((xq + offset - x * mask / delta) * gy).sum()
        go = (delta * gy * (~mask)).sum()
        t1, t2 = gs / steps, steps / (emax - emin) ** 2 * go
    assert torch.equal(y, want)
    assert torch.equal(x.grad, gy * mask)
    torch.testing.assert_close(emin.grad, -t1 + emax.detach() * t2, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(emax.grad, t1 - emin.detach() * t2, rtol=2e-3, atol=2e-3)


def test_argument_errors():
    from aimet_b200.range_learning import QuantizeDequantizeFunc
    q = types.SimpleNamespace(bitwidth=8, use_symmetric_encodings=False, use_strict_symmetric=False,
                              is_unsigned_symmetric=False, channel_axis=0)
    x = torch.zeros(4)
    with pytest.raises(RuntimeError, match="Data type mismatch"):
        QuantizeDequantizeFunc.apply(x, torch.zeros(1, dtype=torch.float16), torch.ones(1), q)
    with pytest.raises(RuntimeError, match="Invalid input data type"):
        QuantizeDequantizeFunc.apply(x.double(), torch.zeros(1).double(), torch.ones(1).double(), q)
    with pytest.raises(RuntimeError, match="CUDA"):
        QuantizeDequantizeFunc.apply(x, torch.zeros(1), torch.ones(1), q)
    q32 = types.SimpleNamespace(bitwidth=32, use_symmetric_encodings=False, use_strict_symmetric=False,
                                is_unsigned_symmetric=False, channel_axis=0)
    assert QuantizeDequantizeFunc.apply(x, None, None, q32) is x or torch.equal(QuantizeDequantizeFunc.apply(x, None, None, q32), x)
