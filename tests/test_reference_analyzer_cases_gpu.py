"""The reference's own MinMaxEncodingAnalyzer test cases
(TrainingExtensions/torch/test/python/v2/quantization/test_encoding_analyzer.py:112-205), restated for CUDA tensors
and run against aimet_b200.v2.encoding_analyzer.MinMaxEncodingAnalyzer -- same inputs, same expectations."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _an(shape):
    from aimet_b200.v2.encoding_analyzer import MinMaxEncodingAnalyzer
    return MinMaxEncodingAnalyzer(shape)


def _full(an, v, cuda):
    return torch.full(tuple(an.observer.shape), v, device=cuda)


def test_compute_encodings_asymmetric(cuda):
    an = _an(())
    an.update_stats(torch.arange(start=0, end=26, step=0.5, dtype=torch.float, device=cuda))
    mn, mx = an.compute_encodings(num_steps=math.pow(2, 8) - 1, is_symmetric=False)
    assert torch.all(torch.isclose(mn, _full(an, 0.0, cuda))) and torch.all(torch.isclose(mx, _full(an, 25.5, cuda)))


def test_compute_encodings_strict_symmetric(cuda):
    an = _an(())
    an.update_stats(torch.arange(start=0, end=26, step=0.5, dtype=torch.float, device=cuda))
    mn, mx = an.compute_encodings(num_steps=math.pow(2, 8) - 2, is_symmetric=True)
    assert torch.all(torch.isclose(mn, _full(an, -25.5, cuda))) and torch.all(torch.isclose(mx, _full(an, 25.5, cuda)))


def test_compute_encodings_non_strict_symmetric(cuda):
    an = _an(())
    an.update_stats(torch.arange(start=-2, end=10, step=1, dtype=torch.float, device=cuda))
    mn, mx = an.compute_encodings(is_symmetric=True, num_steps=pow(2, 3) - 1)
    assert torch.all(torch.isclose(mn, _full(an, -12.0, cuda))) and torch.all(torch.isclose(mx, _full(an, 9.0, cuda)))


@pytest.mark.parametrize("min_max_size", [[3, 4], [2, 3, 1], [4], [1]])
def test_update_stats_with_different_dimensions(cuda, min_max_size):
    for _ in range(4):
        an = _an(min_max_size)
        an.update_stats(torch.randn(2, 3, 4, device=cuda))
        assert list(an.observer.stats.min.shape) == min_max_size
        assert list(an.observer.stats.max.shape) == min_max_size


def test_update_stats_incompatible_dimension(cuda):
    an = _an([3, 4])
    with pytest.raises(RuntimeError):
        an.update_stats(torch.randn(2, 3, 5, device=cuda))


def test_compute_encodings_with_same_nonzero_tensor(cuda):
    an = _an(())
    an.update_stats(torch.full((), 3.0, device=cuda))
    num_steps = pow(2, 8) - 1
    mn, mx = an.compute_encodings(num_steps=num_steps, is_symmetric=False)
    assert torch.allclose(mn, _full(an, 0.0, cuda)) and torch.allclose(mx, _full(an, 3.0, cuda))
    mn, mx = an.compute_encodings(num_steps=num_steps - 1, is_symmetric=True)
    assert torch.allclose(mn, _full(an, -3.0, cuda)) and torch.allclose(mx, _full(an, 3.0, cuda))


def test_compute_encodings_with_only_zero_tensor(cuda):
    an = _an(())
    an.update_stats(torch.zeros((), device=cuda))
    num_steps = pow(2, 8) - 1
    eps = torch.finfo(torch.float32).eps
    mn, mx = an.compute_encodings(num_steps=num_steps, is_symmetric=False)
    assert torch.all(torch.eq(mn, _full(an, 0.0, cuda))) and torch.all(torch.eq(mx, _full(an, eps * num_steps, cuda)))
    mn, mx = an.compute_encodings(num_steps=num_steps, is_symmetric=True)
    assert torch.all(torch.eq(mn, _full(an, -eps * math.ceil(num_steps / 2), cuda)))
    assert torch.all(torch.eq(mx, _full(an, eps * math.floor(num_steps / 2), cuda)))


@pytest.mark.parametrize("symmetric", [True, False])
def test_overflow(cuda, symmetric):
    an = _an(())
    an.update_stats((torch.arange(10) * torch.finfo(torch.float).eps).to(cuda))
    num_steps = pow(2, 8) - 2
    mn, mx = an.compute_encodings(num_steps=num_steps, is_symmetric=symmetric)
    scale = (mx - mn) / 255
    assert scale != 0
    assert torch.allclose(scale, torch.tensor(torch.finfo(scale.dtype).eps, device=cuda), rtol=0.01)
    an.update_stats((torch.arange(10) * torch.finfo(torch.float).max).to(cuda))
    mn1, mx1 = an.compute_encodings(num_steps=num_steps, is_symmetric=symmetric)
    assert torch.all(torch.isfinite(mn1)) and torch.all(torch.isfinite(mx1))


def _analyzers():
    """MinMax and SQNR analyzers of the reference's `encoding_analyzers` fixture (its percentile analyzer of the v2
    flavour is not part of this library)."""
    from aimet_b200.v2.encoding_analyzer import MinMaxEncodingAnalyzer, SqnrEncodingAnalyzer
    return [MinMaxEncodingAnalyzer(()), SqnrEncodingAnalyzer((1,))]


def test_compute_encodings_with_invalid_num_steps(cuda):
    for an in _analyzers():
        an.update_stats(torch.randn(3, 4, device=cuda))
        with pytest.raises(ValueError):
            an.compute_encodings(num_steps=0, is_symmetric=False)


def test_reset_stats(cuda):
    from aimet_b200.v2.encoding_analyzer import MinMaxEncodingAnalyzer
    for an in _analyzers():
        an.update_stats(torch.randn(3, 4, device=cuda))
        if isinstance(an, MinMaxEncodingAnalyzer):
            assert an.observer.stats.min and an.observer.stats.max
        else:
            assert all(x.min is not None for x in an.observer.stats)
            assert all(x.max is not None for x in an.observer.stats)
        an.reset_stats()
        if isinstance(an, MinMaxEncodingAnalyzer):
            assert not an.observer.stats.min and not an.observer.stats.max
        else:
            assert all(x.min is None for x in an.observer.stats)
            assert all(x.max is None for x in an.observer.stats)


def test_compute_encodings_with_no_stats():
    for an in _analyzers():
        with pytest.raises(RuntimeError):
            an.compute_encodings(num_steps=8, is_symmetric=False)


@pytest.mark.parametrize("dtype", [torch.float, torch.half])
@pytest.mark.parametrize("symmetric", [True, False])
def test_continuity(cuda, symmetric, dtype):
    """test_encoding_analyzer.py:89-110: a relative change of eps in the input moves the encodings monotonically and
    by no more than eps."""
    for an in _analyzers():
        normal_range = torch.arange(-128, 128).to(dtype).to(cuda) / 256
        eps = torch.finfo(dtype).eps
        num_steps = math.pow(2, 8) - 2
        min_1, max_1 = an.compute_dynamic_encodings(normal_range * (1 - eps), num_steps=num_steps, is_symmetric=symmetric)
        min_2, max_2 = an.compute_dynamic_encodings(normal_range, num_steps=num_steps, is_symmetric=symmetric)
        min_3, max_3 = an.compute_dynamic_encodings(normal_range * (1 + eps), num_steps=num_steps, is_symmetric=symmetric)
        assert min_3 <= min_2 <= min_1 <= max_1 <= max_2 <= max_3
        assert torch.allclose(max_1, max_2, atol=eps) and torch.allclose(min_1, min_2, atol=eps)
        assert torch.allclose(max_2, max_3, atol=eps) and torch.allclose(min_2, min_3, atol=eps)
