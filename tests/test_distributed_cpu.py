"""Multi-rank calibration protocol on CPU ranks (gloo, world_size 2 and 3).

The exchange logic of aimet_b200.calibration (grid agreement decided per round from the gathered ranges, rows kept
at global batch indices, one all-reduce of the dense row buffer, ordered replay on every rank) runs unchanged; only
the per-GPU arithmetic is replaced by a stand-in engine built on the CPU oracle, so that the protocol is covered
without a GPU.  The result must equal the sequential single-process oracle run bit for bit on every rank.
"""
import ctypes as C
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from _data import normal, relu_activations


class OracleEngine:
    """Stand-in for CudaTfeEngine (same interface, same buffer layout) on CPU tensors, for protocol tests only."""

    def __init__(self):
        from oracle import Oracle
        self.o = Oracle()
        self.x_left = None
        self.gate = 1
        self._alloc(4)

    def _alloc(self, cap, keep=False):
        buf = torch.zeros(cap * 514 + 2, dtype=torch.int32)
        h = buf[:cap * 512].view(cap, 512)
        c = buf[cap * 512:cap * 514].view(torch.int64)
        if keep:
            old = min(self.h.shape[0], cap)
            h[:old], c[:old] = self.h[:old], self.c[:old]
            buf[-2:] = self.flags
        self.buffer, self.h, self.c, self.flags = buf, h, c, buf[-2:]

    def reserve(self, rows):
        if rows > self.h.shape[0]:
            self._alloc(max(rows, 2 * self.h.shape[0]), keep=True)

    def mark_updated(self):
        self.flags[0] = 1

    def _init(self, mn, mx):
        if self.x_left is None and not (mn == 0.0 and mx == 0.0):
            self.x_left = self.o.pdf_init(np.float32(mn), np.float32(mx))

    def offer_grid(self, x):
        if self.x_left is None:
            self._init(*self.o.min_max(x.numpy()).tolist())

    def grid_known(self, wait=False):
        return self.x_left is not None

    def batch_range(self, x):
        if x is None:
            return torch.zeros(3)
        if self.x_left is not None:
            return torch.tensor([0.0, 0.0, 1.0])
        mn, mx = self.o.min_max(x.numpy()).tolist()
        return torch.tensor([mn, mx, 1.0], dtype=torch.float32)

    def select_grid(self, ranges, num_ranks, rank):
        if self.x_left is not None:
            self.gate = 1
            return
        t = ranges.view(num_ranks, 3).tolist()
        chosen = next((r for r, (mn, mx, present) in enumerate(t) if present and not (mn == 0.0 and mx == 0.0)), -1)
        self.gate = 1 if (chosen >= 0 and rank >= chosen) else 0
        if chosen >= 0:
            self._init(t[chosen][0], t[chosen][1])

    def add_batch(self, x, row, gated=False):
        self.reserve(row + 1)
        if self.x_left is None or (gated and not self.gate):
            return
        bs, po = self.o.pdf_geometry(self.x_left)
        self.h[row] += torch.from_numpy(self.o.hist512(x.numpy(), bs, po).astype(np.int32))
        self.c[row] = x.numel()

    def add_batches(self, xs, row0, row_stride):
        for i, x in enumerate(xs):
            self.add_batch(x, row0 + i * row_stride)

    def exchange_buffer(self, n_total):
        if n_total != self.h.shape[0]:
            self._alloc(n_total, keep=True)
        return self.buffer

    def encoding(self, stats_updated, bw, symmetric, strict, unsigned_sym, num_rows=None):
        from oracle import OracleTfeAnalyzer
        a = OracleTfeAnalyzer(self.o)
        a.stats_updated = bool(self.flags[0].item()) if stats_updated is None else bool(stats_updated)
        n = self.h.shape[0] if num_rows is None else num_rows
        if self.x_left is not None:
            a.x_left[:] = self.x_left
            a.initialized = C.c_int(1)
            for h, c in zip(self.h[:n].numpy(), self.c[:n].tolist()):
                if c:
                    hh = np.ascontiguousarray(h, np.uint32)
                    self.o.lib.orc_pdf_accumulate(hh.ctypes.data_as(C.POINTER(C.c_uint32)), int(c),
                                                  a.pdf.ctypes.data_as(C.POINTER(C.c_double)), C.byref(a.iterations))
        return torch.from_numpy(a.compute(bw, symmetric, strict, unsigned_sym))


def make_batches(scenario):
    if scenario == "relu":
        return [relu_activations(3000 + 17 * b, 1000 + b) for b in range(7)]
    if scenario == "zeros_first":
        return [np.zeros(2000, np.float32)] * 3 + [normal(2000, 5 + b, 2.0, 0.5) for b in range(4)]
    if scenario == "all_zero":
        return [np.zeros(1000, np.float32)] * 4
    raise ValueError(scenario)


def sequential(batches, bw, flags):
    from oracle import Oracle, OracleTfeAnalyzer
    a = OracleTfeAnalyzer(Oracle())
    for b in batches:
        a.update(b)
    return a.compute(bw, *flags)


def _worker(rank, world, port, scenario, out, feed="single"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from aimet_b200.calibration import TfEnhancedCalibrator
        batches = make_batches(scenario)
        cal = TfEnhancedCalibrator("cpu", engine=OracleEngine(), num_batches=len(batches) if feed == "many" else None)
        rounds = (len(batches) + world - 1) // world
        mine = [torch.from_numpy(batches[k * world + rank]) if k * world + rank < len(batches) else None
                for k in range(rounds)]
        if feed == "many" and mine[-1] is not None:
            cal.update_many(mine)
        elif feed == "many":
            # update_many takes whole rounds only; a rank without a batch in the last round feeds that one singly
            cal.update_many(mine[:-1])
            cal.update(None)
        else:
            for x in mine:
                cal.update(x)
        res = []
        for bw, flags in ((8, (False, False, False)), (8, (True, False, False)), (4, (True, True, False))):
            e = cal.compute_encoding(bw, *flags)
            res.append([e.min, e.max, e.delta, e.offset, e.bw])
        out[rank] = res
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("feed", ["single", "many"])
@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("scenario", ["relu", "zeros_first", "all_zero"])
def test_sharded_tf_enhanced_equals_sequential(world, scenario, feed):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), scenario, out, feed), nprocs=world, join=True)
    batches = make_batches(scenario)
    want = [sequential(batches, bw, flags) for bw, flags in
            ((8, (False, False, False)), (8, (True, False, False)), (4, (True, True, False)))]
    for rank in range(world):
        for got, w in zip(out[rank], want):
            assert np.array(got, np.float64).tobytes() == np.asarray(w, np.float64).tobytes() or \
                np.array_equal(np.array(got), np.asarray(w)), (rank, got, w)


def test_single_process_protocol_matches_sequential():
    from aimet_b200.calibration import TfEnhancedCalibrator
    batches = make_batches("zeros_first")
    w = sequential(batches, 8, (False, False, False))
    for feed in ("single", "many"):
        cal = TfEnhancedCalibrator("cpu", engine=OracleEngine())
        if feed == "many":
            cal.update_many([torch.from_numpy(b) for b in batches])
        else:
            for b in batches:
                cal.update(torch.from_numpy(b))
        e = cal.compute_encoding(8)
        assert [e.min, e.max, e.delta, e.offset, e.bw] == list(w), feed


# ---- SQNR on the v2 histograms: two passes, two all-reduces --------------------------------------------------------
class OracleHistogramObserver:
    """Stand-in for the four sharded-calibration steps of _HistogramObserver on CPU tensors (one histogram), built on
    the CPU oracle; ``state`` holds the replayed statistics."""

    num_histograms = 1

    def __init__(self, num_bins):
        self.num_bins = num_bins
        self.state = None

    def batch_range(self, x, out):
        from oracle import v2_hist_oracle as vh
        out[0] = torch.from_numpy(vh.range_record(x.numpy()))

    def plan_batches(self, ranges):
        from oracle import v2_hist_oracle as vh
        return torch.from_numpy(vh.plan_batches(ranges[:, 0].numpy(), self.num_bins)).unsqueeze(1).contiguous()

    def count_batch(self, x, plan, out):
        from oracle import v2_hist_oracle as vh
        out[0] = torch.from_numpy(vh.count(x.numpy(), self.num_bins, plan[0].numpy()))

    def replay_batches(self, counts, plans, dtype):
        from oracle import v2_hist_oracle as vh
        self.state = vh.replay(counts[:, 0].numpy(), plans[:, 0].numpy(), self.num_bins)


class _OracleAnalyzer:
    def __init__(self, num_bins):
        self.observer = OracleHistogramObserver(num_bins)


def make_v2_batches(scenario):
    if scenario == "growing":
        return [normal(4000 + 13 * b, 40 + b, 1.0 + 0.5 * b, 0.2 * b) for b in range(7)]
    if scenario == "relu_inf":
        out = [relu_activations(5000, 2000 + b) for b in range(5)]
        out[2] = np.concatenate([out[2], np.array([np.inf, -np.inf, np.nan], np.float32)])
        return out
    if scenario == "shrinking":
        return [normal(3000, 60 + b, s) for b, s in enumerate((4.0, 1.0, 0.25, 2.0))]
    raise ValueError(scenario)


def _v2_worker(rank, world, port, scenario, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from aimet_b200.calibration import SqnrCalibrator
        batches = make_v2_batches(scenario)
        rounds = (len(batches) + world - 1) // world
        mine = [torch.from_numpy(batches[k * world + rank]) if k * world + rank < len(batches) else None
                for k in range(rounds)]
        cal = SqnrCalibrator(_OracleAnalyzer(128), "cpu")
        cal.calibrate(mine)
        st = cal.analyzer.observer.state
        out[rank] = (st.hist.tobytes(), st.edges.tobytes(), float(st.min), float(st.max))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("scenario", ["growing", "relu_inf", "shrinking"])
def test_sharded_v2_histograms_equal_sequential(world, scenario):
    from oracle import v2_hist_oracle as vh
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_v2_worker, args=(world, _free_port(), scenario, out), nprocs=world, join=True)
    want = vh.sequential(make_v2_batches(scenario), 128)[-1]
    for rank in range(world):
        hist, edges, mn, mx = out[rank]
        assert hist == want.hist.tobytes() and edges == want.edges.tobytes(), (rank, scenario)
        assert (mn, mx) == (float(want.min), float(want.max))
