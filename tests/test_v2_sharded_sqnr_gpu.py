"""SQNR calibration on the v2 histograms with the batches spread over several workers: the statistics and encodings must
be those of one process feeding the batches in global order -- bit for bit.

The workers are emulated in one process (each runs its local steps; the two integer all-reduces become sums of the
workers' tables), and the result is compared with what the reference's own class produced for the same batches
(tests/golden/v2_sqnr.npz) and, at sizes where float32 counts round (bins beyond 2^24 elements), with this library's
sequential observer, which is pinned to the reference by tests/test_v2_sqnr_gpu.py.
"""
import os

import numpy as np
import pytest
import torch

from _data import assert_bits_equal

pytestmark = pytest.mark.gpu

S = np.load(os.path.join(os.path.dirname(__file__), "golden", "v2_sqnr.npz"))
GRIDS = [(float(s), bool(y)) for s, y in S["grids"]]


def steps_of(v):
    return int(v) if float(v).is_integer() and v != 256.0 else v


def emulate(world, shape, bins, batches, device, **kw):
    """``batches``: all batches in global order (None = absent).  Returns the workers' calibrators after calibration."""
    from aimet_b200.calibration import SqnrCalibrator
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    rounds = (len(batches) + world - 1) // world
    padded = list(batches) + [None] * (rounds * world - len(batches))
    workers = []
    for r in range(world):
        c = SqnrCalibrator(SqnrEncodingAnalyzer(shape, bins, **kw), device)
        c.rank, c.world = r, world
        workers.append(c)
    shares = [padded[r::world] for r in range(world)]
    ranges = sum(c.local_ranges(sh) for c, sh in zip(workers, shares))
    stage = [c.local_counts(sh, ranges) for c, sh in zip(workers, shares)]
    counts = sum(cn for _, cn in stage)
    for c, (plans, _) in zip(workers, stage):
        c.finish(ranges, plans, counts)
    return workers


@pytest.mark.parametrize("world", [1, 2, 3])
@pytest.mark.parametrize("name", [str(n) for n in S["names"]])
def test_sharded_statistics_match_reference_class(cuda, name, world):
    shape = tuple(int(v) for v in S[f"{name}/shape"])
    bins = int(S[f"{name}/bins"])
    nbat = int(S[f"{name}/num_batches"])
    batches = [torch.from_numpy(S[f"{name}/x{b}"]).to(cuda) for b in range(nbat)]
    nh = int(np.prod(shape)) if len(shape) else 1
    for c in emulate(world, shape, bins, batches, cuda, gamma=float(S[f"{name}/gamma"])):
        state = c.analyzer.observer.get_stats()
        for h in range(nh):
            key = f"{name}/b{nbat - 1}/state/{h}"
            assert_bits_equal(state[h].histogram.cpu().numpy(), S[f"{key}/hist"], f"{key} histogram")
            assert_bits_equal(state[h].bin_edges.cpu().numpy(), S[f"{key}/edges"], f"{key} bin edges")
            assert_bits_equal(np.array([state[h].min.item(), state[h].max.item()], np.float32), S[f"{key}/minmax"],
                              f"{key} min/max")
        for gi, (steps, sym) in enumerate(GRIDS):
            mn, mx = c.compute_encodings(steps_of(steps), sym)
            got = np.stack([mn.reshape(-1).cpu().numpy(), mx.reshape(-1).cpu().numpy()])
            assert_bits_equal(got, S[f"{name}/final/{gi}"], f"{name} final grid {gi}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sharded_equals_sequential_when_float_counts_round(cuda, dtype):
    """Post-ReLU batches of 12.8 M elements: the bin that holds the zeros passes 2^24 after three batches, so the order
    of the float32 additions matters; ranges grow twice, one batch is absent, one holds infinities."""
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    g = torch.Generator(device=cuda).manual_seed(5)
    n = 64 * 256 * 28 * 28
    batches = []
    for b, scale in enumerate((1.0, 0.8, 1.5, 1.0, 1.2, 2.5, 1.0)):
        x = torch.relu(torch.randn(n, device=cuda, generator=g)) * scale
        if b == 4:
            x[17] = float("inf")
            x[29] = float("-inf")
            x[31] = float("nan")
        batches.append(x.to(dtype))
    seq = SqnrEncodingAnalyzer((1,), 512)
    for x in batches:
        seq.update_stats(x)
    want = seq.observer.get_stats()[0]
    assert float(want.histogram.max()) > 2 ** 24
    with_gap = batches[:3] + [None] + batches[3:]
    for world in (2, 4):
        for c in emulate(world, (1,), 512, with_gap, cuda):
            got = c.analyzer.observer.get_stats()[0]
            assert_bits_equal(got.histogram.cpu().numpy(), want.histogram.cpu().numpy(), f"world {world} histogram")
            assert_bits_equal(got.bin_edges.cpu().numpy(), want.bin_edges.cpu().numpy(), f"world {world} edges")
            assert got.min.item() == want.min.item() and got.max.item() == want.max.item()
            for steps, sym in ((255, False), (255, True)):
                a, b_ = c.compute_encodings(steps, sym)
                p, q = seq.compute_encodings(steps, sym)
                assert a.dtype == p.dtype
                assert torch.equal(a, p) and torch.equal(b_, q)


def test_sharded_per_channel_and_errors(cuda):
    from aimet_b200.calibration import SqnrCalibrator
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    g = torch.Generator(device=cuda).manual_seed(9)
    batches = [torch.randn(8, 64, 5, 5, device=cuda, generator=g) * (1 + 0.3 * b) for b in range(5)]
    seq = SqnrEncodingAnalyzer((1, 64, 1, 1), 256)
    for x in batches:
        seq.update_stats(x)
    for c in emulate(2, (1, 64, 1, 1), 256, batches, cuda):
        for got, want in zip(c.analyzer.observer.get_stats(), seq.observer.get_stats()):
            assert torch.equal(got.histogram, want.histogram) and torch.equal(got.bin_edges, want.bin_edges)
        a, b_ = c.compute_encodings(255, False)
        p, q = seq.compute_encodings(255, False)
        assert a.shape == (1, 64, 1, 1) and torch.equal(a, p) and torch.equal(b_, q)
    # one process, no group: calibrate() is the whole job; a callable may stand for the batches
    solo = SqnrCalibrator(SqnrEncodingAnalyzer((1, 64, 1, 1), 256), cuda)
    solo.calibrate(lambda: iter(batches))
    assert torch.equal(solo.compute_encodings(255, False)[0], seq.compute_encodings(255, False)[0])
    # a batch without a finite value: the reference raises ValueError when it meets it
    bad = SqnrCalibrator(SqnrEncodingAnalyzer((1,), 64), cuda)
    bad.calibrate([torch.randn(100, device=cuda), torch.full((10,), float("nan"), device=cuda)])
    with pytest.raises(ValueError):
        bad.compute_encodings(255, False)
    with pytest.raises(RuntimeError):
        SqnrCalibrator(SqnrEncodingAnalyzer((1,), 64), cuda).compute_encodings(255, False)
    with pytest.raises(ValueError):
        SqnrCalibrator(SqnrEncodingAnalyzer((1,), 64), cuda).calibrate([])
