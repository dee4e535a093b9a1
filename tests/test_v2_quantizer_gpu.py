"""GPU parity of the affine quantizer modules against fixtures produced by the reference's own
``Quantize`` / ``QuantizeDequantize`` (tests/golden/gen_golden.py:gen_quantizer), plus the host-side behaviour that
the reference tests pin (TrainingExtensions/torch/test/python/v2/quantization/affine/test_affine_quantizer.py)."""
import os

import numpy as np
import pytest
import torch

from _data import assert_bits_equal

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def _cases():
    import sys
    sys.path.insert(0, GOLDEN)
    from gen_golden import quantizer_cases
    return [(c[0], c[1], c[2], c[3]) for c in quantizer_cases()]


@pytest.mark.gpu
@pytest.mark.parametrize("name,kind,args,kwargs", _cases(), ids=[c[0] for c in _cases()])
def test_module_matches_reference_fixture(cuda, name, kind, args, kwargs):
    from aimet_b200.v2.quantizer import GroupedBlockQuantizeDequantize, Quantize, QuantizeDequantize
    g = np.load(os.path.join(GOLDEN, "v2_quantizer.npz"))
    dt = DT[str(g[f"{name}/dtype"])]
    q = {"qdq": QuantizeDequantize, "q": Quantize, "gbq": GroupedBlockQuantizeDequantize}[kind](*args, **kwargs).to(cuda)
    assert not q.is_initialized() and q.get_scale() is None
    with pytest.raises(RuntimeError):
        q(torch.zeros(1, device=cuda))
    with torch.no_grad():
        with q.compute_encodings():
            b = 0
            while f"{name}/batch{b}" in g.files:
                x = torch.from_numpy(g[f"{name}/batch{b}"]).to(cuda).to(dt)
                assert_bits_equal(q(x).float().cpu().numpy(), g[f"{name}/dyn{b}"], f"dynamic output, batch {b}")
                b += 1
        assert q.is_initialized()
        assert_bits_equal(q.min.detach().cpu().numpy(), g[f"{name}/min"], "min")
        assert_bits_equal(q.max.detach().cpu().numpy(), g[f"{name}/max"], "max")
        assert_bits_equal(q.get_scale().cpu().numpy(), g[f"{name}/scale"], "scale")
        assert_bits_equal(q.get_offset().cpu().numpy(), g[f"{name}/offset"], "offset")
        probe = torch.from_numpy(g[f"{name}/probe"]).to(cuda).to(dt)
        for _ in range(2):   # the second call takes the cached scale / offset
            assert_bits_equal(q(probe).float().cpu().numpy(), g[f"{name}/out"], "output")
        if kind == "gbq":
            # grouped blocks: one scale per group, an integer multiple of it per block
            assert_bits_equal(q.get_per_channel_scale().cpu().numpy(), g[f"{name}/per_channel_scale"], "group scale")
            np.testing.assert_array_equal(q.get_per_block_integer_scale().cpu().numpy(), g[f"{name}/integer_scale"])
    enc = q.get_encoding()
    assert enc.qmin == q.qmin and enc.qmax == q.qmax and enc.symmetry == q.symmetric
    np.testing.assert_array_equal(enc.min.detach().cpu().numpy(), q.get_min().detach().cpu().numpy())


@pytest.mark.gpu
def test_gradients_reach_input_min_and_max(cuda):
    from aimet_b200.v2.quantizer import QuantizeDequantize
    q = QuantizeDequantize((4, 1), 8, False).to(cuda)
    x = torch.randn(4, 256, device=cuda)
    with q.compute_encodings():
        q(x)
    xr = (x * 1.5).requires_grad_(True)
    y = q(xr)
    y.sum().backward()
    assert xr.grad is not None and q.min.grad is not None and q.max.grad is not None
    assert q.min.grad.shape == q.min.shape and torch.isfinite(q.min.grad).all()
    # straight-through: gradient 1 inside the range, 0 where the input was clamped
    inside = (xr.detach() >= q.get_min()) & (xr.detach() <= q.get_max())
    assert torch.equal(xr.grad[inside], torch.ones_like(xr.grad[inside]))
    # training changed nothing yet: cached scale is refreshed after an optimiser step
    s0 = q.get_scale().clone()
    with torch.no_grad():
        q.max.mul_(2.0)
    assert not torch.equal(q.get_scale(), s0)


def test_constructor_forms_and_errors():
    from aimet_b200.v2.quantizer import Quantize, QuantizeDequantize, derive_qmin_qmax
    assert derive_qmin_qmax(8, False) == (0, 255) and derive_qmin_qmax(8, True) == (-128, 127)
    assert derive_qmin_qmax(4, True) == (-8, 7)
    a = QuantizeDequantize((3, 1), bitwidth=4, symmetric=True)
    b = QuantizeDequantize((3, 1), -8, 7, True)
    c = Quantize(shape=(3, 1), qmin=-8, qmax=7, symmetric=True)
    for q in (a, b, c):
        assert (q.qmin, q.qmax, q.symmetric, q.bitwidth, q.signed) == (-8, 7, True, 4, True)
        assert q.shape == (3, 1) and tuple(q.min.shape) == (3, 1)
    assert QuantizeDequantize(5, 8, False).shape == (5,)
    blk = QuantizeDequantize((12, 4), 4, True, block_size=(-1, 8))
    assert blk.encoding_analyzer.observer.shape == (12, 1, 4, 1)
    with pytest.raises(ValueError):
        QuantizeDequantize((), 5, 5, False)
    with pytest.raises(TypeError):
        QuantizeDequantize((), 8, False, bogus=1)
    with pytest.raises(TypeError):
        QuantizeDequantize(())
    from aimet_b200.v2.encoding_analyzer import MinMaxEncodingAnalyzer
    with pytest.raises(RuntimeError):
        QuantizeDequantize((3, 1), 8, False, MinMaxEncodingAnalyzer((4, 1)))


def test_initialisation_tracking_and_state_dict():
    from aimet_b200.v2.quantizer import QuantizeDequantize
    q = QuantizeDequantize((2,), 8, False)
    assert not q.is_initialized()
    q.set_range(torch.tensor([-1.0, -2.0]), torch.tensor([1.0, 3.0]))
    assert q.is_initialized()
    sd = q.state_dict()
    r = QuantizeDequantize((2,), 8, False)
    r.load_state_dict(sd)
    assert r.is_initialized() and torch.equal(r.min, q.min) and torch.equal(r.max, q.max)
    import copy
    c = copy.deepcopy(q)
    assert c.is_initialized() and torch.equal(c.min, q.min) and c.min is not q.min
    assert not copy.deepcopy(QuantizeDequantize((2,), 8, False)).is_initialized()
    fresh = QuantizeDequantize((2,), 8, False)
    r2 = QuantizeDequantize((2,), 8, False)
    r2.load_state_dict(fresh.state_dict())
    assert not r2.is_initialized()
    # a quantizer that may not be overwritten keeps its range through a calibration context
    q.allow_overwrite(False)
    before = q.min.clone()
    with q.compute_encodings():
        pass
    assert torch.equal(q.min, before)
    # calibration without data leaves the quantizer uninitialised
    e = QuantizeDequantize((), 8, False)
    with e.compute_encodings():
        pass
    assert not e.is_initialized()


def test_grouped_block_constructor_errors():
    from aimet_b200.v2.quantizer import GroupedBlockQuantizeDequantize as G
    with pytest.raises(RuntimeError, match="Length of block grouping"):
        G((4, 8), 4, True, 8, None, (1, 16), (2,))
    with pytest.raises(RuntimeError, match="divide evenly"):
        G((4, 8), 4, True, 8, None, (1, 16), (1, 3))
    with pytest.raises(RuntimeError, match="cannot be smaller"):
        G((4, 8), 8, True, 4, None, (1, 16), (1, 2))
    with pytest.raises(RuntimeError, match="only supports symmetric"):
        G((4, 8), 4, False, 8, None, (1, 16), (1, 2))
    assert G((4, 8), 4, True, 8, None, (1, 16), (1, -1)).get_expanded_scale_shape() == (4, 1, 1, 8)
    assert G((4, 8), 4, True, 8, None, (1, 16)).block_grouping == (1, 1)

