"""GPU parity of the TF-Enhanced calibration path (512-bucket histogram, PDF replay, SQNR search)."""
import numpy as np
import pytest
import torch

from _data import assert_bits_equal, normal, relu_activations

pytestmark = pytest.mark.gpu


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def gen(kind, seed, n):
    if kind == "relu":
        return relu_activations(n, seed)
    if kind == "normal":
        return normal(n, seed, 2.0, 1.0)
    if kind == "neg":
        return normal(n, seed, 1.0, -2.0)
    if kind == "zeros":
        return np.zeros(n, np.float32)
    if kind == "const":
        return np.full(n, 4.0, np.float32)
    if kind == "specials":
        x = normal(n, seed, 3.0)
        x[:8] = [np.nan, np.inf, -np.inf, 3e38, -3e38, 0.0, -0.0, 1e-40]
        return x
    raise ValueError(kind)


def run_gpu(batches, cuda):
    from aimet_b200 import ops
    st = ops.TfeDeviceState(cuda, capacity=2)
    for b in batches:
        xd = dev(b, cuda)
        if not st.is_initialized():
            st.init_grid_from(ops.minmax(xd).reshape(-1))
        st.add_batch(xd)
    st.replay()
    return st


SCENARIOS = [
    (["relu"] * 5, 60000),
    (["normal"] * 3, 60001),
    (["zeros", "zeros", "relu", "relu"], 4099),
    (["neg", "neg"], 60000),
    (["const"], 6000),
    (["zeros"], 6000),
    (["specials", "normal"], 10007),
    (["relu"] * 3, 1 << 21),
]


@pytest.mark.parametrize("kinds,n", SCENARIOS)
def test_tfe_matches_oracle(oracle, cuda, kinds, n):
    from oracle import OracleTfeAnalyzer
    batches = [gen(k, 100 + i, n) for i, k in enumerate(kinds)]
    oa = OracleTfeAnalyzer(oracle)
    for b in batches:
        oa.update(b)
    st = run_gpu(batches, cuda)

    counts = st.counts[:st.num_batches].cpu().numpy()
    used = [i for i in range(len(batches)) if counts[i] != 0]
    assert len(used) == len(oa.batch_hists)
    hists = st.hists[:st.num_batches].cpu().numpy().view(np.uint32)
    for j, i in enumerate(used):
        assert counts[i] == batches[i].size
        np.testing.assert_array_equal(hists[i], oa.batch_hists[j], err_msg=f"batch {i} histogram")
        # conservation: every sample is either counted once or lies outside the 512 buckets
        assert hists[i].sum() <= batches[i].size
    if oa.initialized.value:
        assert st.is_initialized()
        assert_bits_equal(st.x_left().cpu().numpy(), oa.x_left, "bucket grid")
        assert_bits_equal(st.pdf.cpu().numpy(), oa.pdf, "running PDF")
        assert int(st.iterations.item()) == oa.iterations.value
    else:
        assert not st.is_initialized()

    for bw in (8, 4, 16):
        for sym, strict, uns in [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]:
            want = oa.compute(bw, sym, strict, uns)
            got = st.search(True, bw, sym, strict, uns).cpu().numpy()
            assert_bits_equal(got, want, f"encoding bw={bw} sym={sym} strict={strict} unsigned={uns}")


def test_tfe_no_stats_gives_zero_encoding(oracle, cuda):
    from aimet_b200 import ops
    st = ops.TfeDeviceState(cuda)
    st.replay()
    got = st.search(False, 8, 0, 0, 0).cpu().numpy()
    np.testing.assert_array_equal(got, np.zeros(5))


def test_tfe_misaligned_input(oracle, cuda):
    from aimet_b200 import ops
    x = relu_activations(50001, 5)
    xl = oracle.pdf_init(*oracle.min_max(x[1:]))
    bs, po = oracle.pdf_geometry(xl)
    want = oracle.hist512(x[1:], bs, po)
    xd = dev(x, cuda)[1:]
    st = ops.TfeDeviceState(cuda)
    st.init_grid_from(ops.minmax(xd).reshape(-1))
    st.add_batch(xd)
    np.testing.assert_array_equal(st.hists[0].cpu().numpy().view(np.uint32), want)


# ---- fused range + grid setup, gated / many-batch histogram, cross-rank grid selection ------------------------------
def _rows(st):
    n = st.num_batches
    return st.hists[:n].cpu().numpy().view(np.uint32), st.counts[:n].cpu().numpy()


@pytest.mark.parametrize("kinds,n", SCENARIOS)
def test_offer_grid_equals_minmax_plus_init(oracle, cuda, kinds, n):
    """One launch (min/max pass + grid setup, a no-op once a grid exists) against the two-step form."""
    from aimet_b200 import ops
    batches = [gen(k, 100 + i, n) for i, k in enumerate(kinds)]
    ref = run_gpu(batches, cuda)
    st = ops.TfeDeviceState(cuda, capacity=len(batches))
    for b in batches:
        xd = dev(b, cuda)
        st.offer_grid(xd)      # always offered: the device ignores it once the grid exists
        st.add_batch(xd)
    st.replay()
    h0, c0 = _rows(ref)
    h1, c1 = _rows(st)
    np.testing.assert_array_equal(c1, c0)
    np.testing.assert_array_equal(h1, h0)
    np.testing.assert_array_equal(st.state.cpu().numpy(), ref.state.cpu().numpy(), err_msg="state record")
    assert_bits_equal(st.pdf.cpu().numpy(), ref.pdf.cpu().numpy(), "pdf")


def test_offer_grid_reports_range(oracle, cuda):
    from aimet_b200 import ops
    for n, off in ((100003, 0), (4097, 1), (3, 0), (70001, 3)):
        x = normal(n + off, 7 + n, 3.0, 0.5)
        xd = dev(x, cuda)[off:]
        st = ops.TfeDeviceState(cuda)
        r = st.batch_range(xd).cpu().numpy()
        want = oracle.min_max(x[off:])
        assert_bits_equal(r[:2], want, f"range n={n} off={off}")
        assert r[2] == 1.0 and not st.is_initialized()
        st.offer_grid(xd)
        assert st.is_initialized()
        assert_bits_equal(st.x_left().cpu().numpy(), oracle.pdf_init(*want), "grid")
        # a second offer is skipped and reports (0, 0, 1)
        r = st.batch_range(dev(normal(1000, 1, 50.0), cuda)).cpu().numpy()
        np.testing.assert_array_equal(r, [0.0, 0.0, 1.0])
    assert st.batch_range(None).cpu().tolist() == [0.0, 0.0, 0.0]


@pytest.mark.parametrize("m,stride", [(1, 1), (3, 1), (16, 1), (19, 1), (5, 4)])
def test_histogram_many_equals_single(oracle, cuda, m, stride):
    """m resident batches in one launch (ragged sizes, one of them not 16-byte aligned) against one launch each."""
    from aimet_b200 import ops
    sizes = [50000 + 4099 * (i % 5) + i for i in range(m)]
    xs = [dev(relu_activations(s + 1, 300 + i), cuda) for i, s in enumerate(sizes)]
    xs = [x[1:] if i % 4 == 2 else x[:-1] for i, x in enumerate(xs)]
    rows = (m - 1) * stride + 1
    one, many = ops.TfeDeviceState(cuda, rows), ops.TfeDeviceState(cuda, rows)
    for st in (one, many):
        st.offer_grid(xs[0])
    for i, x in enumerate(xs):
        one.add_batch(x, i * stride)
    many.add_batches(xs, 0, stride)
    h0, c0 = _rows(one)
    h1, c1 = _rows(many)
    np.testing.assert_array_equal(c1, c0)
    np.testing.assert_array_equal(h1, h0)
    assert (c0[::stride] == [x.numel() for x in xs]).all() and c0.sum() == sum(x.numel() for x in xs)
    bs, po = oracle.pdf_geometry(one.x_left().cpu().numpy())
    for i, x in enumerate(xs):
        np.testing.assert_array_equal(h0[i * stride], oracle.hist512(x.cpu().numpy(), bs, po))


@pytest.mark.parametrize("seed", range(6))
def test_histogram_many_mixed_sizes(oracle, cuda, seed):
    """Launches of 1..16 batches whose sizes range from empty to millions of samples (so that every way of splitting
    the batches over the CTAs is taken: fewer CTAs than batches, a grid cut to a multiple of the batch count, the full
    grid with several (batch, slice) pairs per CTA), some starting off a 16-byte boundary, against the oracle row by row."""
    from aimet_b200 import ops
    rng = np.random.default_rng(900 + seed)
    m = int(rng.integers(1, 17))
    big = [int(rng.integers(200_000, 3_000_000)) for _ in range(m)] if seed % 2 else \
          [int(rng.choice([0, 1, 3, 5, 17, 4096, 70_001, 900_000])) for _ in range(m)]
    xs = []
    for i, n in enumerate(big):
        off = int(rng.integers(0, 4))
        base = dev(relu_activations(n + off, 40 * seed + i) if i % 3 else normal(n + off, 40 * seed + i, 2.0, 0.5), cuda)
        xs.append(base[off:])
    st = ops.TfeDeviceState(cuda, m)
    st.init_grid_from(torch.tensor([-1.5, 9.0], device=cuda))
    st.add_batches(xs, 0, 1)
    h, c = _rows(st)
    np.testing.assert_array_equal(c[:m], [x.numel() for x in xs])
    bs, po = oracle.pdf_geometry(st.x_left().cpu().numpy())
    for i, x in enumerate(xs):
        np.testing.assert_array_equal(h[i], oracle.hist512(x.cpu().numpy(), bs, po), err_msg=f"batch {i} of {m}, n={x.numel()}")


def test_histogram_many_before_grid_counts_nothing(cuda):
    from aimet_b200 import ops
    st = ops.TfeDeviceState(cuda, 4)
    st.add_batches([dev(normal(5000, i), cuda) for i in range(3)], 0, 1)
    h, c = _rows(st)
    assert not h.any() and not c.any()


@pytest.mark.parametrize("table,rank,want_gate,want_range", [
    ([[0, 0, 1], [-1, 2, 1], [5, 6, 1]], 0, 0, (-1, 2)),     # all-zero batch ahead of the defining one: dropped
    ([[0, 0, 1], [-1, 2, 1], [5, 6, 1]], 1, 1, (-1, 2)),
    ([[0, 0, 1], [-1, 2, 1], [5, 6, 1]], 2, 1, (-1, 2)),
    ([[3, 4, 0], [0, 0, 1], [0.5, 0.5, 1]], 1, 0, (0.5, 0.5)),   # absent ranks are skipped
    ([[0, 0, 1], [0, 0, 1]], 1, 0, None),                        # nobody can define the grid this round
])
def test_select_grid(oracle, cuda, table, rank, want_gate, want_range):
    from aimet_b200 import ops
    st = ops.TfeDeviceState(cuda)
    t = torch.tensor(table, dtype=torch.float32, device=cuda).reshape(-1)
    st.select_grid(t, len(table), rank)
    assert int(st.gate.item()) == want_gate
    x = dev(np.zeros(1000, np.float32), cuda)
    st.add_batch(x, 0, gated=True)
    assert int(st.counts[0].item()) == (1000 if want_gate else 0)
    if want_range is None:
        assert not st.is_initialized()
        return
    assert_bits_equal(st.x_left().cpu().numpy(), oracle.pdf_init(np.float32(want_range[0]), np.float32(want_range[1])), "grid")
    # once a grid exists the selection is a no-op that opens the gate
    st.select_grid(torch.tensor([[9.0, 10.0, 1.0]], device=cuda).reshape(-1), 1, 0)
    assert int(st.gate.item()) == 1
    assert_bits_equal(st.x_left().cpu().numpy(), oracle.pdf_init(np.float32(want_range[0]), np.float32(want_range[1])), "grid kept")


def test_compute_encoding_equals_replay_plus_search(oracle, cuda):
    from aimet_b200 import ops
    st = run_gpu([gen("relu", 100 + i, 60000) for i in range(5)], cuda)
    for bw, sym in ((8, 0), (4, 1)):
        want = st.search(True, bw, sym, 0, 0).cpu().numpy().copy()
        got = st.compute_encoding(True, bw, sym, 0, 0).cpu().numpy()
        assert_bits_equal(got, want, "encoding")
    # the "any batch offered" flag taken from the device instead of the host
    empty = ops.TfeDeviceState(cuda)
    np.testing.assert_array_equal(empty.compute_encoding(None, 8, 0, 0, 0).cpu().numpy(), np.zeros(5))
    empty.flags[0:1].fill_(2)
    assert_bits_equal(empty.compute_encoding(None, 8, 0, 0, 0).cpu().numpy(),
                      empty.compute_encoding(True, 8, 0, 0, 0).cpu().numpy().copy(), "all-zero-data encoding")


def test_calibrator_update_many_equals_updates(oracle, cuda):
    from aimet_b200.calibration import TfEnhancedCalibrator
    batches = [np.zeros(3000, np.float32)] * 2 + [relu_activations(30000 + 7 * i, 40 + i) for i in range(21)]
    xs = [dev(b, cuda) for b in batches]
    a, b = TfEnhancedCalibrator(cuda), TfEnhancedCalibrator(cuda, num_batches=len(xs))
    for x in xs:
        a.update(x)
    b.update_many(xs[:5])
    b.update_many(xs[5:])
    ea, eb = a.compute_encoding(8), b.compute_encoding(8)
    assert [ea.min, ea.max, ea.delta, ea.offset] == [eb.min, eb.max, eb.delta, eb.offset]
    ha, ca = _rows(a.engine.state)
    hb, cb = _rows(b.engine.state)
    np.testing.assert_array_equal(ca, cb)
    np.testing.assert_array_equal(ha, hb)
    from oracle import OracleTfeAnalyzer
    oa = OracleTfeAnalyzer(oracle)
    for x in batches:
        oa.update(x)
    assert_bits_equal(np.array([ea.min, ea.max, ea.delta, ea.offset, ea.bw]), oa.compute(8, 0, 0, 0), "encoding")
