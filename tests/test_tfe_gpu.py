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
