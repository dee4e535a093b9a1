"""GPU parity of the v2 histogram observer and SQNR analyzer with the reference's own classes.

tests/golden/v2_sqnr.npz was produced by the reference's ``SqnrEncodingAnalyzer`` / ``_HistogramObserver`` on CPU
(tests/golden/gen_golden.py): per-batch histograms, the merged statistics after every update, dynamic and final
encodings.  tests/golden/histc_rule.npz pins the bin rule of ``torch.histc`` (third-party code) on boundary values.
Histograms, bin edges, min / max and encodings must be bit-identical.
"""
import os

import numpy as np
import pytest
import torch

from _data import assert_bits_equal

pytestmark = pytest.mark.gpu

GOLD = os.path.join(os.path.dirname(__file__), "golden")
S = np.load(os.path.join(GOLD, "v2_sqnr.npz"))
H = np.load(os.path.join(GOLD, "histc_rule.npz"))
GRIDS = [(float(s), bool(y)) for s, y in S["grids"]]


def steps_of(v):
    return int(v) if float(v).is_integer() and v != 256.0 else v


@pytest.mark.parametrize("case", range(int(H["count"])))
def test_histc_rule(cuda, case):
    """The counting pass against the installed torch.histc on boundary values (collect over a forced range)."""
    from aimet_b200._lib import lib
    x = H[f"c{case}/x"]
    lo, hi = H[f"c{case}/range"]
    nb = int(H[f"c{case}/bins"])
    want = H[f"c{case}/counts"]
    # Drive the merge path, whose counting range is exactly [state.min, state.max] when the batch lies inside it:
    # keep only elements inside the range plus NaN (what histc looks at), so that the widened range stays [lo, hi].
    keep = ((x >= lo) & (x <= hi)) | np.isnan(x)
    xs = np.ascontiguousarray(x[keep])
    xd = torch.from_numpy(xs).to(cuda)
    words = (16 + (2 * nb + 1) * 4) // 4
    state = torch.zeros(words, dtype=torch.int32, device=cuda)
    state.view(torch.float32)[0] = float(lo)
    state.view(torch.float32)[1] = float(hi)
    state[2] = 1
    batch = torch.zeros(words, dtype=torch.int32, device=cuda)
    scratch = torch.empty(int(lib.aq_v2hist_scratch_bytes()), dtype=torch.uint8, device=cuda)
    upd = torch.empty(nb, dtype=torch.float32, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    # the merge takes the batch's finite min / max from the batch's own statistics
    assert lib.aq_v2hist_collect(xd.data_ptr(), 0, xd.numel(), nb, batch.data_ptr(), scratch.data_ptr(), st) == 0
    assert lib.aq_v2hist_merge(xd.data_ptr(), 0, xd.numel(), nb, state.data_ptr(), batch.data_ptr(), 1,
                               scratch.data_ptr(), upd.data_ptr(), st) == 0
    got = state.view(torch.float32)[4:4 + nb].cpu().numpy()
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("name", [str(n) for n in S["names"]])
def test_sqnr_analyzer_matches_reference(cuda, name):
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    shape = tuple(int(v) for v in S[f"{name}/shape"])
    bins = int(S[f"{name}/bins"])
    an = SqnrEncodingAnalyzer(shape, bins, gamma=float(S[f"{name}/gamma"]))
    nh = int(np.prod(shape)) if len(shape) else 1
    for b in range(int(S[f"{name}/num_batches"])):
        x = torch.from_numpy(S[f"{name}/x{b}"]).to(cuda)
        new = an.update_stats(x)
        state = an.observer.get_stats()
        assert len(new) == nh and len(state) == nh
        for h in range(nh):
            for kind, st in (("batch", new[h]), ("state", state[h])):
                key = f"{name}/b{b}/{kind}/{h}"
                assert_bits_equal(st.histogram.cpu().numpy(), S[f"{key}/hist"], f"{key} histogram")
                assert_bits_equal(st.bin_edges.cpu().numpy(), S[f"{key}/edges"], f"{key} bin edges")
                assert_bits_equal(np.array([st.min.item(), st.max.item()], np.float32), S[f"{key}/minmax"], f"{key} min/max")
        for gi, (steps, sym) in enumerate(GRIDS):
            mn, mx = an.compute_encodings_from_stats(new, steps_of(steps), sym)
            got = np.stack([mn.reshape(-1).cpu().numpy(), mx.reshape(-1).cpu().numpy()])
            assert_bits_equal(got, S[f"{name}/b{b}/dynamic/{gi}"], f"{name} batch {b} dynamic grid {gi}")
    for gi, (steps, sym) in enumerate(GRIDS):
        mn, mx = an.compute_encodings(steps_of(steps), sym)
        assert mn.shape == shape and mx.shape == shape
        got = np.stack([mn.reshape(-1).cpu().numpy(), mx.reshape(-1).cpu().numpy()])
        assert_bits_equal(got, S[f"{name}/final/{gi}"], f"{name} final grid {gi}")


def test_sqnr_analyzer_protocol(cuda):
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer, StatisticsNotFoundError
    with pytest.raises(ValueError):
        SqnrEncodingAnalyzer((1,), 0)
    an = SqnrEncodingAnalyzer((1,), 512)
    with pytest.raises(StatisticsNotFoundError):
        an.compute_encodings(255, False)
    x = torch.randn(1000, device=cuda)
    an.update_stats(x)
    with pytest.raises(ValueError):
        an.compute_encodings(0, False)
    mn, mx = an.compute_encodings(255, False)
    assert mn.shape == (1,) and mn.device.type == "cuda"
    an.reset_stats()
    with pytest.raises(StatisticsNotFoundError):
        an.compute_encodings(255, False)
    with pytest.raises(RuntimeError):
        an.update_stats(torch.randn(10))          # CPU tensor: there is no CPU path
    with pytest.raises(RuntimeError):
        SqnrEncodingAnalyzer((3,), 64).update_stats(torch.randn(5, 4, device=cuda))   # shape not expandable
    # 16-bit input: statistics in float32, encodings come back in the input dtype
    h = SqnrEncodingAnalyzer((), 256)
    h.update_stats(torch.randn(4000, device=cuda).to(torch.bfloat16))
    mn, mx = h.compute_encodings(255, True)
    assert mn.dtype == torch.bfloat16 and mn.shape == ()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,steps,sym", [((), 255, False), ((6, 1), 255, True), ((6, 1), 15, False)])
def test_fused_calibration_step_matches_separate_calls(cuda, dtype, shape, steps, sym):
    """fused_update (statistics update with one counting pass + search + scale / offset in the search launch) against
    collect_stats / merge_stats / compute_encodings_from_stats followed by the quantizer's expressions."""
    from aimet_b200.v2.encoding_analyzer import SqnrEncodingAnalyzer
    torch.manual_seed(7)
    qmin = -(steps + 1) // 2 if sym else 0
    fused, plain = SqnrEncodingAnalyzer(shape), SqnrEncodingAnalyzer(shape)
    for b in range(3):
        x = (torch.randn(6, 4000, device=cuda) * (1.0 + b) + (0.0 if sym else 0.3)).to(dtype)
        scale, offset = fused.fused_update(x, steps, sym, qmin)
        stats = plain.observer.collect_stats(x)
        plain.observer.merge_stats(stats, x)
        dmin, dmax = plain.compute_encodings_from_stats(stats, steps, sym)
        want_scale = (dmax.float() - dmin.float()) / torch.tensor(float(steps), device=cuda)
        want_offset = torch.zeros_like(want_scale) if sym else torch.round(dmin.float() / want_scale) - qmin
        np.testing.assert_array_equal(scale.cpu().numpy(), want_scale.cpu().numpy())
        np.testing.assert_array_equal(offset.cpu().numpy(), want_offset.cpu().numpy())
    for a, b in zip(fused.observer.get_stats(), plain.observer.get_stats()):
        np.testing.assert_array_equal(a.histogram.cpu().numpy(), b.histogram.cpu().numpy())
        np.testing.assert_array_equal(a.bin_edges.cpu().numpy(), b.bin_edges.cpu().numpy())
    got, want = fused.compute_encodings(steps, sym), plain.compute_encodings(steps, sym)
    np.testing.assert_array_equal(got[0].float().cpu().numpy(), want[0].float().cpu().numpy())
    np.testing.assert_array_equal(got[1].float().cpu().numpy(), want[1].float().cpu().numpy())



@pytest.mark.parametrize("bins", [512, 2048])
@pytest.mark.parametrize("edge_share", [1.0, 2e-3, 0.0])
def test_counting_pass_with_values_on_bin_edges(cuda, bins, edge_share):
    """Values that sit exactly on bin edges take the counting kernel's exact path: a few per CTA go through its queue,
    many make it recount its share; either way the counts are those of torch.histc (on the CPU) over the same range."""
    from aimet_b200.v2.encoding_analyzer import _HistogramObserver
    g = torch.Generator().manual_seed(bins)
    n = 3_000_000
    x = torch.rand(n, generator=g) * bins
    on_edge = torch.rand(n, generator=g) < edge_share
    x = torch.where(on_edge, torch.floor(x), x)
    x[0], x[1] = 0.0, float(bins)            # the range is [0, bins]: every integer is an edge
    x[2], x[3], x[4] = float("inf"), float("-inf"), float("nan")
    obs = _HistogramObserver((1,), bins)
    got = obs.collect_stats(x.to(cuda))[0]
    want = torch.histc(x, bins=bins, min=0.0, max=float(bins))
    want[0] += 1       # -inf
    want[-1] += 1      # +inf
    assert got.min.item() == 0.0 and got.max.item() == float(bins)
    assert_bits_equal(got.histogram.cpu().numpy(), want.numpy(), "histogram")
    # the same batch merged into statistics with a wider range (the fused update counts it over both ranges at once)
    obs.update_stats(torch.tensor([-1.0, float(bins) + 3.0], device=cuda))
    obs.update_stats(x.to(cuda))
    wide = torch.histc(x, bins=bins, min=-1.0, max=float(bins) + 3.0)
    first = torch.histc(torch.tensor([-1.0, float(bins) + 3.0]), bins=bins, min=-1.0, max=float(bins) + 3.0)
    wide[0] += 1
    wide[-1] += 1
    assert_bits_equal(obs.get_stats()[0].histogram.cpu().numpy(), (wide + first).numpy(), "merged histogram")


@pytest.mark.parametrize("shape,enc", [((5, 77), (5, 1)), ((3, 1001), (3, 1)), ((1, 4099), (1,))])
@pytest.mark.parametrize("shift", [0, 1, 3])
def test_observer_on_odd_row_lengths_and_unaligned_starts(cuda, shape, enc, shift):
    """Rows whose length is no multiple of the packet width, and tensors that start off a 16-byte boundary, take the
    element-wise forms of the two passes; statistics must equal the CPU restatement of the reference observer (which
    tests/test_oracle_pin.py pins to the reference class) after every update."""
    from oracle import v2_hist_oracle as vh
    from aimet_b200.v2.encoding_analyzer import _HistogramObserver
    bins = 64
    n = int(np.prod(shape))
    rng = np.random.default_rng(shift + n)
    obs = _HistogramObserver(enc, bins)
    state = [None] * shape[0]
    for b in range(3):
        base = (rng.standard_normal(n + 4) * (1.0 + b)).astype(np.float32)
        base[5] = 0.0
        x = base[shift:shift + n].reshape(shape)
        xd = torch.from_numpy(base).to(cuda)[shift:shift + n].view(shape)
        obs.update_stats(xd)
        got = obs.get_stats()
        for r in range(shape[0]):
            state[r] = vh.merge(state[r], x[r], bins)
            assert_bits_equal(got[r].histogram.cpu().numpy(), state[r].hist, f"batch {b} row {r} histogram")
            assert_bits_equal(got[r].bin_edges.cpu().numpy(), state[r].edges, f"batch {b} row {r} edges")
            assert got[r].min.item() == float(state[r].min) and got[r].max.item() == float(state[r].max)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("edge_share", [0.5, 1e-3, 0.0])
def test_16bit_inputs_count_like_their_float32_values(cuda, dtype, edge_share):
    """The reference upcasts the input before torch.histc, so a 16-bit batch must give the statistics of the same
    values held in float32 (whose path the reference fixtures pin) -- through the 8-elements-per-packet forms of both
    passes, with values on bin edges, infinities and a NaN."""
    from aimet_b200.v2.encoding_analyzer import _HistogramObserver
    g = torch.Generator().manual_seed(11)
    bins, n = 128, 1_000_003
    o16, o32 = _HistogramObserver((1,), bins), _HistogramObserver((1,), bins)
    for b in range(3):
        x = torch.rand(n, generator=g) * bins * (1 + b)
        x = torch.where(torch.rand(n, generator=g) < edge_share, torch.floor(x), x)
        x[0], x[1] = 0.0, float(bins * (1 + b))
        x[7], x[9], x[11] = float("inf"), float("-inf"), float("nan")
        x16 = x.to(dtype).to(cuda)
        o16.update_stats(x16)
        o32.update_stats(x16.float())
        a, c = o16.get_stats()[0], o32.get_stats()[0]
        assert_bits_equal(a.histogram.cpu().numpy(), c.histogram.cpu().numpy(), f"batch {b} histogram")
        assert_bits_equal(a.bin_edges.cpu().numpy(), c.bin_edges.cpu().numpy(), f"batch {b} edges")
        assert float(a.min) == float(c.min) and float(a.max) == float(c.max)
