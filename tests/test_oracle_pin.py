"""Pins the CPU oracles (test infrastructure) to the reference:

1. the reference's own known-answer vectors (tests/golden/reference_kats.json, taken from its unit tests);
2. golden fixtures produced by running the reference itself (tests/golden/*.npz, see gen_golden.py);
3. where oracle/_ref was built, the unmodified reference code on fresh seeded inputs, bit for bit.
"""
import json
import os

import numpy as np
import pytest

from _data import SPECIALS, assert_bits_equal, conv_weight, normal, relu_activations

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
KATS = json.load(open(os.path.join(GOLDEN, "reference_kats.json")))


def ulp_close(a, b, ulps=4):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    return np.all(np.abs(a - b) <= ulps * np.spacing(np.maximum(np.abs(a), np.abs(b))))


# ---- 1. known-answer vectors -------------------------------------------------------------------------------------
@pytest.mark.parametrize("k", KATS["qdq_per_tensor"])
def test_kat_qdq(oracle, k):
    got = oracle.qdq_per_tensor(np.array(k["input"], np.float32), k["min"], k["max"], k["bw"])
    assert ulp_close(got, k["expected"])   # the reference asserts EXPECT_FLOAT_EQ (4 ulp)


@pytest.mark.parametrize("k", KATS["quantize_per_tensor"])
def test_kat_codes(oracle, k):
    got = oracle.quantize_per_tensor(np.array(k["input"], np.float32), k["min"], k["max"], k["bw"], k["shift"])
    np.testing.assert_array_equal(got, np.array(k["expected"], np.float32))


@pytest.mark.parametrize("k", KATS["fill_encoding"])
def test_kat_fill_encoding(oracle, k):
    e = oracle.fill_encoding(k["bw"], k["min"], k["max"])
    assert abs(e[0] - k["expected_min"]) <= 4 * np.spacing(abs(k["expected_min"]))
    assert abs(e[1] - k["expected_max"]) <= 4 * np.spacing(abs(k["expected_max"]))


@pytest.mark.parametrize("k", KATS["broadcast"])
def test_kat_broadcast(oracle, k):
    enc = [np.array(k[n], np.float32) for n in ("enc_min", "enc_max", "enc_delta", "enc_offset")]
    got = oracle.qdq_broadcast(np.array(k["input"], np.float32), k["in_strides"], k["enc_strides"], *enc)
    assert_bits_equal(got, np.array(k["expected"], np.float32))


def test_kat_tfe_all_zero(oracle):
    from oracle import OracleTfeAnalyzer
    k = KATS["tfe_all_zero"]
    a = OracleTfeAnalyzer(oracle)
    a.update(np.zeros(k["count"], np.float32))
    e = a.compute(k["bw"])
    assert abs(e[0] - k["min"]) < k["tol"] and abs(e[1] - k["max"]) < k["tol"] and e[3] == k["offset"] and e[4] == 8


def test_tfe_statistical_properties(oracle):
    """Shape of the reference's typed tests (TestTfEnhancedEncodingAnalyzer.cpp:199-296): symmetric offsets."""
    from oracle import OracleTfeAnalyzer
    a = OracleTfeAnalyzer(oracle)
    a.update(normal(6000, 1, 1.0, -2.0))
    e = a.compute(8, True, False, False)
    assert e[3] == -128 and e[4] == 8
    e = a.compute(8, True, True, False)
    assert e[3] == -127 and e[0] == -e[1]


# ---- 2. golden fixtures generated from the reference -------------------------------------------------------------
@pytest.fixture(scope="module")
def libpymo_golden():
    return np.load(os.path.join(GOLDEN, "libpymo.npz"))


def test_golden_libpymo_qdq(oracle, libpymo_golden):
    g = libpymo_golden
    x = g["qdq/x"]
    for i in range(5):
        mn, mx, bw = g[f"qdq/{i}/enc"]
        assert_bits_equal(oracle.qdq_per_tensor(x, mn, mx, int(bw)), g[f"qdq/{i}/y"], f"qdq {i}")
        assert_bits_equal(oracle.quantize_per_tensor(x, mn, mx, int(bw), False), g[f"qdq/{i}/codes"])
        assert_bits_equal(oracle.quantize_per_tensor(x, mn, mx, int(bw), True), g[f"qdq/{i}/codes_signed"])


@pytest.mark.parametrize("name", ["relu", "normal", "zeros_then_relu", "negative"])
def test_golden_libpymo_calibration(oracle, libpymo_golden, name):
    from oracle import OracleTfeAnalyzer
    g = libpymo_golden
    batches = []
    while f"cal/{name}/batch{len(batches)}" in g:
        batches.append(g[f"cal/{name}/batch{len(batches)}"])
    a = OracleTfeAnalyzer(oracle)
    mn, mx = np.inf, -np.inf
    used = []
    for b, xb in enumerate(batches):
        if a.update(xb):
            used.append(b)
        mm = oracle.min_max(xb)
        mn, mx = min(mn, float(mm[0])), max(mx, float(mm[1]))
    assert_bits_equal(a.x_left, g[f"cal/{name}/x_left"])
    assert_bits_equal(a.pdf, g[f"cal/{name}/pdf"])
    for j, b in enumerate(used):
        np.testing.assert_array_equal(a.batch_hists[j], g[f"cal/{name}/hist{b}"])
    for bw in (8, 4):
        for sym, strict, uns in ((0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)):
            assert_bits_equal(a.compute(bw, sym, strict, uns), g[f"cal/{name}/tfe_b{bw}_{sym}{strict}{uns}"])
            want = g[f"cal/{name}/tf_b{bw}_{sym}{strict}{uns}"]
            assert_bits_equal(oracle.minmax_encoding(bw, mn, mx, sym, strict, uns), want[:4])


def _v2_cases():
    g = np.load(os.path.join(GOLDEN, "v2_backend.npz"))
    names = sorted({k.split("/")[0] for k in g.files})
    return g, names


@pytest.mark.parametrize("name", _v2_cases()[1])
def test_golden_v2_backend(name):
    from oracle import v2_oracle as v2
    g, _ = _v2_cases()
    x, scale, offset = g[f"{name}/x"], g[f"{name}/scale"], g[f"{name}/offset"]
    qmin, qmax = (int(v) for v in g[f"{name}/q"])
    block = tuple(int(b) for b in g[f"{name}/block"]) or None
    dtype = str(g[f"{name}/dtype"]).replace("torch.", "")
    y, mask = v2.quantize_dequantize(x, scale, offset, qmin, qmax, block, dtype)
    assert_bits_equal(y, g[f"{name}/qdq"], "qdq")
    np.testing.assert_array_equal(mask, g[f"{name}/mask"])
    if f"{name}/codes" in g.files:
        q, _ = v2.quantize_dequantize(x, scale, offset, qmin, qmax, block, dtype, codes_only=True, arithmetic=dtype)
        assert_bits_equal(q, g[f"{name}/codes"], "codes")
        assert_bits_equal(v2.dequantize(g[f"{name}/codes"], scale, offset, block, dtype), g[f"{name}/deq"], "deq")
    if v2.internal_dtype(dtype, qmin, qmax) == "float32":
        dx, ds, do, axes, s_shape = v2.backward(x, g[f"{name}/gy"], scale, offset, qmin, qmax, block, dtype)
        assert_bits_equal(dx, g[f"{name}/dx"], "dx")
        # the summed encoding gradients depend on torch's reduction order: compare to float32 accuracy
        ds_sum = ds.sum(axis=axes, keepdims=True, dtype=np.float64).reshape(g[f"{name}/dscale"].shape)
        do_sum = do.sum(axis=axes, keepdims=True, dtype=np.float64).reshape(g[f"{name}/doffset"].shape)
        np.testing.assert_allclose(ds_sum, g[f"{name}/dscale"], rtol=2e-4, atol=1e-4)
        np.testing.assert_allclose(do_sum, g[f"{name}/doffset"], rtol=2e-4, atol=1e-4)


def _ste_cases():
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "v1_ste.npz"))
    names = sorted({k.split("/")[0] for k in g.files})
    return g, names


def ste_geometry(shape, axis, num_enc):
    """(num_ch, inner) of the flat buffer for encodings broadcast on `axis` (one encoding: per tensor)."""
    if num_enc == 1:
        return 1, int(np.prod(shape))
    return shape[axis], int(np.prod(shape[axis + 1:]))


def test_golden_v1_ste_backward(oracle):
    """orc_ste_bwd against compute_dloss_by_dx of the reference (fixture generated by the reference's own file):
    per tensor, and per channel on axis 0 / 1 through the (num_ch, inner) geometry the kernels use."""
    g, names = _ste_cases()
    assert len(names) >= 5
    for name in names:
        x, grad, want = g[f"{name}/x"], g[f"{name}/grad"], g[f"{name}/dx"]
        mins, maxs = g[f"{name}/min"].reshape(-1), g[f"{name}/max"].reshape(-1)
        num_ch, inner = ste_geometry(x.shape, int(g[f"{name}/axis"]), mins.size)
        rows = x.reshape(-1, inner)
        grows = grad.reshape(-1, inner)
        got = np.stack([oracle.ste_bwd(rows[r], grows[r], mins[r % num_ch], maxs[r % num_ch])
                        for r in range(rows.shape[0])]).reshape(x.shape)
        from _data import assert_bits_equal
        assert_bits_equal(got, want, name)


def test_golden_v2_minmax():
    from oracle import v2_oracle as v2
    g = np.load(os.path.join(GOLDEN, "v2_minmax.npz"))
    k = 0
    while f"c{k}/x" in g.files:
        dt, enc_shape, steps, sym = g[f"c{k}/meta"]
        dtype = dt.replace("torch.", "")
        enc_shape = tuple(json.loads(enc_shape))
        x = g[f"c{k}/x"]
        x2 = v2.to_storage(v2.to_storage(x * np.float32(0.5), dtype) + np.float32(0.1), dtype)
        if enc_shape == (1,):
            red = lambda a: (a.min(keepdims=True).reshape(1), a.max(keepdims=True).reshape(1))
        elif enc_shape == (8, 1, 1, 1):
            red = lambda a: (a.min(axis=(1, 2, 3), keepdims=True), a.max(axis=(1, 2, 3), keepdims=True))
        else:
            red = lambda a: (a.reshape(6, 2, 8).min(axis=2), a.reshape(6, 2, 8).max(axis=2))
        (mn1, mx1), (mn2, mx2) = red(x), red(x2)
        mn, mx = v2.minmax_encodings(np.minimum(mn1, mn2), np.maximum(mx1, mx2), int(steps), bool(int(sym)), dtype)
        assert_bits_equal(mn.reshape(g[f"c{k}/min"].shape), g[f"c{k}/min"], f"case {k} min")
        assert_bits_equal(mx.reshape(g[f"c{k}/max"].shape), g[f"c{k}/max"], f"case {k} max")
        k += 1
    assert k == 24


# ---- 3. live comparison with the compiled reference ---------------------------------------------------------------
def test_ref_fill_encoding(oracle, reference):
    for mn, mx, bw in [(-0.46, 0.72, 8), (0.5, 1.0, 8), (0.5, 0.5, 8), (-0.5, -0.1, 8), (-5, 10, 3), (-5, 5, 3),
                       (-1.3, 2.7, 4), (-3, 3, 16), (0, 0, 8), (-1e-7, 1e-7, 8)]:
        assert_bits_equal(oracle.fill_encoding(bw, mn, mx), reference.fill_encoding(bw, mn, mx))


def test_ref_qdq(oracle, reference):
    x = np.concatenate([normal(200000, 0, 2.0), SPECIALS])
    for mn, mx, bw in [(-0.46, 0.72, 8), (-3.1, 4.2, 8), (-2, 2, 8), (0, 5, 4), (-7, 3, 16), (-1, 1, 2)]:
        assert_bits_equal(oracle.qdq_per_tensor(x, mn, mx, bw), reference.qdq_per_tensor(x, mn, mx, bw))
        for s in (False, True):
            assert_bits_equal(oracle.quantize_per_tensor(x, mn, mx, bw, s), reference.quantize_per_tensor(x, mn, mx, bw, s))
    assert_bits_equal(oracle.min_max(x), reference.min_max(x))


def test_ref_per_channel_and_broadcast(oracle, reference):
    w = conv_weight((32, 16, 3, 3), 3)
    flat = w.reshape(32, -1)
    for mins, maxs in [(-np.abs(flat).max(1), np.abs(flat).max(1)), (flat.min(1), flat.max(1))]:
        g = oracle.per_channel_grid(mins.astype(np.float64), maxs.astype(np.float64), 8)
        assert_bits_equal(oracle.qdq_per_channel(w, 32, 144, *g), reference.qdq_per_channel(w, 32, 144, *g))
    x = normal((4, 6, 8), 4)
    enc = [normal(24, 5, 0.1) - 1, normal(24, 6, 0.1) + 1, np.full(24, 0.01, np.float32), np.full(24, -100, np.float32)]
    for ins, ens in [([48, 8, 1], [6, 1, 0]), ([48, 8, 1], [0, 0, 1][:3])]:
        assert_bits_equal(oracle.qdq_broadcast(x, ins, ens, *enc), reference.qdq_broadcast(x, ins, ens, *enc))


def test_ref_computed_encodings(oracle, reference):
    for bw in (4, 8, 16):
        for mn, mx in [(-1.5, 3.2), (0, 4.4), (-3, 0), (-2, 2), (-1e-3, 1e-3), (-np.inf, 5), (0, 0.01)]:
            for sym, strict, uns in [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]:
                assert_bits_equal(oracle.computed_encodings(bw, mn, mx, sym, strict, uns),
                                  reference.computed_encodings(bw, mn, mx, sym, strict, uns))


@pytest.mark.parametrize("kinds", [["relu"] * 5, ["normal"] * 3, ["zeros", "zeros", "relu", "relu"], ["neg"] * 2,
                                   ["const"], ["zeros"], ["specials", "normal"]])
def test_ref_tf_enhanced(oracle, reference, kinds):
    from oracle import OracleTfeAnalyzer, RefAnalyzer

    def gen(kind, seed, n=40000):
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
        x = normal(n, seed, 3.0)
        x[:8] = [np.nan, np.inf, -np.inf, 3e38, -3e38, 0.0, -0.0, 1e-40]
        return x
    oa, ra = OracleTfeAnalyzer(oracle), RefAnalyzer(reference, "tfe")
    for i, k in enumerate(kinds):
        b = gen(k, 100 + i)
        oa.update(b)
        ra.update(b)
    xl, pdf = ra.histogram()
    if xl is not None:
        assert_bits_equal(oa.x_left, xl)
        assert_bits_equal(oa.pdf, pdf)
    for bw in (4, 8, 16):
        for sym, strict, uns in [(0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1)]:
            assert_bits_equal(oa.compute(bw, sym, strict, uns), ra.compute(bw, sym, strict, uns), f"{bw} {sym}{strict}{uns}")


@pytest.mark.parametrize("kinds", [("relu",) * 4, ("normal",) * 3, ("zeros", "zeros", "relu"), ("neg", "neg"), ("zeros",)])
def test_ref_percentile(oracle, reference, kinds):
    """The percentile restatement against the reference's PercentileEncodingAnalyzer on the same batches."""
    from oracle import OracleTfeAnalyzer, RefAnalyzer
    gens = {"relu": lambda s: relu_activations(7001, s), "normal": lambda s: normal(7001, s, 2.0, 1.0),
            "neg": lambda s: normal(7001, s, 1.0, -2.0), "zeros": lambda s: np.zeros(500, np.float32)}
    batches = [gens[k](31 + i) for i, k in enumerate(kinds)]
    oa = OracleTfeAnalyzer(oracle)
    for b in batches:
        oa.update(b)
    for pct in (100.0, 99.99, 99.9, 99.0, 90.0, 50.0):
        ra = RefAnalyzer(reference, "pct")
        ra.set_percentile(pct)
        for b in batches:
            ra.update(b)
        for bw, sym, strict, uns in ((8, 0, 0, 0), (8, 1, 0, 0), (4, 1, 1, 0), (16, 1, 0, 1)):
            want = ra.compute(bw, sym, strict, uns)
            got = oa.compute_percentile(pct, bw, sym, strict, uns)
            assert_bits_equal(got[:4], want[:4], f"percentile {pct} bw={bw} sym={sym}{strict}{uns}")


@pytest.mark.parametrize("kinds", [("relu",) * 4, ("normal",) * 3, ("zeros", "zeros", "relu"), ("neg", "neg"), ("zeros",),
                                   ("pos",) * 2])
def test_ref_mse(oracle, reference, kinds):
    """The MSE restatement against the reference's MseEncodingAnalyzer on the same batches."""
    from oracle import OracleTfeAnalyzer, RefAnalyzer
    gens = {"relu": lambda s: relu_activations(7001, s), "normal": lambda s: normal(7001, s, 2.0, 1.0),
            "neg": lambda s: normal(7001, s, 1.0, -6.0), "pos": lambda s: normal(7001, s, 0.5, 4.0),
            "zeros": lambda s: np.zeros(500, np.float32)}
    batches = [gens[k](41 + i) for i, k in enumerate(kinds)]
    oa = OracleTfeAnalyzer(oracle)
    ra = RefAnalyzer(reference, "mse")
    for b in batches:
        oa.update(b)
        ra.update(b)
    for bw, sym, strict, uns in ((8, 0, 0, 0), (8, 1, 0, 0), (4, 0, 0, 0), (4, 1, 1, 0), (16, 1, 0, 1), (2, 0, 0, 0)):
        want = ra.compute(bw, sym, strict, uns)
        got = oa.compute_mse(bw, sym, strict, uns)
        assert_bits_equal(got[:4], want[:4], f"mse bw={bw} sym={sym}{strict}{uns}")


def test_ref_partial_encoding(reference):
    """compute_partial_encoding (host arithmetic of the libpymo mirror) against the reference's two helper functions."""
    import ctypes as C
    from aimet_b200.libpymo import TfEncoding, compute_partial_encoding
    cases = [(8, dict(delta=0.5, offset=-10.0, bw=8)), (8, dict(delta=0.0123, offset=-128.0, bw=8)),
             (4, dict(delta=0.25, offset=0.0, bw=4)), (8, dict(min=-1.0, max=2.0, bw=8)), (8, dict(min=0.0, max=3.3, bw=8)),
             (16, dict(min=-7.5, max=7.5, bw=16)), (8, dict(min=-2.0, max=-0.5, bw=8))]
    for bw, fields in cases:
        for sym, uns, strict in ((0, 0, 0), (1, 0, 0), (1, 1, 0), (1, 0, 1), (1, 1, 1)):
            e = TfEncoding(**fields)
            enc5 = np.array([e.min, e.max, e.delta, e.offset, e.bw], np.float64)
            rc = reference.lib.ref_partial_encoding(bw, enc5.ctypes.data_as(C.POINTER(C.c_double)), sym, uns, strict)
            assert rc == 0
            compute_partial_encoding(bw, e, bool(sym), bool(uns), bool(strict))
            assert_bits_equal(np.array([e.min, e.max, e.delta, e.offset]), enc5[:4], f"{fields} {sym}{uns}{strict}")


@pytest.mark.parametrize("bw", [1, 2, 4, 8, 16, 32])
@pytest.mark.parametrize("signed", [False, True])
def test_ref_packed_codes(oracle, reference, bw, signed):
    """Integer containers: the restatement against quantizeTensorPacked / dequantizeTensor of the reference."""
    import ctypes as C
    x = np.concatenate([normal(5000, 3 + bw, 2.0, 0.3), np.array([0.0, -0.0, 1e-30, 4.0, -4.0, 3.99, -3.99, 100.0, -100.0], np.float32)])
    for mn, mx in ((-3.1, 4.2), (0.0, 5.0), (-2.0, 2.0)):
        dt = oracle.packed_dtype(bw, signed)
        want = np.zeros(x.shape, dt)
        reference.lib.ref_quantize_packed(x.ctypes.data_as(C.POINTER(C.c_float)), x.size, want.ctypes.data_as(C.c_void_p),
                                          mn, mx, bw, int(signed))
        got = oracle.quantize_packed(x, mn, mx, bw, signed)
        np.testing.assert_array_equal(got, want, err_msg=f"codes bw={bw} signed={signed} [{mn},{mx}]")
        back_want = np.zeros(x.shape, np.float32)
        reference.lib.ref_dequantize_packed(want.ctypes.data_as(C.c_void_p), x.size,
                                            back_want.ctypes.data_as(C.POINTER(C.c_float)), mn, mx, bw, int(signed))
        assert_bits_equal(oracle.dequantize_packed(want, mn, mx, bw, signed), back_want, f"dequantize bw={bw}")



# ---- v2 histogram observer: the sequential restatement and its cut into the steps of sharded calibration -----------
SQNR_GOLD = np.load(os.path.join(GOLDEN, "v2_sqnr.npz"))


def _sqnr_rows(name):
    """Per histogram, the list of its batches (the encoding axes of these scenarios lead)."""
    nh = max(1, int(np.prod(SQNR_GOLD[f"{name}/shape"])))
    nbat = int(SQNR_GOLD[f"{name}/num_batches"])
    return [[SQNR_GOLD[f"{name}/x{b}"].reshape(nh, -1)[h] for b in range(nbat)] for h in range(nh)]


@pytest.mark.parametrize("name", [str(n) for n in SQNR_GOLD["names"]])
def test_v2_histogram_oracle_matches_reference_class(name):
    from oracle import v2_hist_oracle as vh
    bins = int(SQNR_GOLD[f"{name}/bins"])
    for h, batches in enumerate(_sqnr_rows(name)):
        for b, st in enumerate(vh.sequential(batches, bins)):
            own = vh.collect(batches[b], bins)
            assert_bits_equal(own.hist, SQNR_GOLD[f"{name}/b{b}/batch/{h}/hist"], f"{name} batch {b} own hist")
            assert_bits_equal(own.edges, SQNR_GOLD[f"{name}/b{b}/batch/{h}/edges"], f"{name} batch {b} own edges")
            assert_bits_equal(st.hist, SQNR_GOLD[f"{name}/b{b}/state/{h}/hist"], f"{name} batch {b} hist")
            assert_bits_equal(st.edges, SQNR_GOLD[f"{name}/b{b}/state/{h}/edges"], f"{name} batch {b} edges")
            assert_bits_equal(np.array([st.min, st.max], np.float32), SQNR_GOLD[f"{name}/b{b}/state/{h}/minmax"],
                              f"{name} batch {b} min/max")


@pytest.mark.parametrize("name", [str(n) for n in SQNR_GOLD["names"]])
def test_v2_histogram_oracle_steps_give_the_sequential_statistics(name):
    """range records -> plans -> counts -> replay == feeding the batches one by one (also with absent batches)."""
    from oracle import v2_hist_oracle as vh
    bins = int(SQNR_GOLD[f"{name}/bins"])
    for h, batches in enumerate(_sqnr_rows(name)):
        padded = [batches[0], None] + list(batches[1:]) + [None]
        ranges = np.stack([vh.range_record(x) if x is not None else np.zeros(4, np.int32) for x in padded])
        plans = vh.plan_batches(ranges, bins)
        counts = np.stack([vh.count(x, bins, plans[i]) if x is not None else np.zeros(bins + 2, np.int32)
                           for i, x in enumerate(padded)])
        st = vh.replay(counts, plans, bins)
        last = len(batches) - 1
        assert_bits_equal(st.hist, SQNR_GOLD[f"{name}/b{last}/state/{h}/hist"], f"{name} hist")
        assert_bits_equal(st.edges, SQNR_GOLD[f"{name}/b{last}/state/{h}/edges"], f"{name} edges")
        assert_bits_equal(np.array([st.min, st.max], np.float32), SQNR_GOLD[f"{name}/b{last}/state/{h}/minmax"],
                          f"{name} min/max")
