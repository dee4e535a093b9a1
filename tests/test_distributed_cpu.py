"""Multi-rank calibration protocol on CPU ranks (gloo, world_size 2 and 3).

The exchange logic of aimet_b200.calibration (grid agreement, per-batch rows, all-reduce, ordered replay,
broadcast) runs unchanged; only the per-GPU arithmetic is replaced by a stand-in engine built on the CPU oracle,
because this machine has no GPU.  The result must equal the sequential single-process oracle run bit for bit.
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
    """Stand-in for CudaTfeEngine (same interface) on CPU tensors, for protocol tests only."""

    def __init__(self):
        from oracle import Oracle
        self.o = Oracle()
        self.x_left = None
        self.h, self.c = [], []

    def minmax(self, x):
        return torch.from_numpy(self.o.min_max(x.numpy()))

    def init_grid(self, minmax):
        mn, mx = (np.float32(v) for v in minmax.tolist())
        self.x_left = self.o.pdf_init(mn, mx)

    def is_initialized(self):
        return self.x_left is not None

    def add_batch(self, x, row):
        assert row == len(self.h)
        if self.x_left is None:
            return self.add_empty_row(row)
        bs, po = self.o.pdf_geometry(self.x_left)
        self.h.append(self.o.hist512(x.numpy(), bs, po).astype(np.int64))
        self.c.append(x.numel())

    def add_empty_row(self, row):
        assert row == len(self.h)
        self.h.append(np.zeros(512, np.int64))
        self.c.append(0)

    def num_rows(self):
        return len(self.h)

    def rows(self):
        return torch.from_numpy(np.stack(self.h)).to(torch.int32), torch.tensor(self.c, dtype=torch.int64)

    def load_rows(self, hists, counts):
        self.h = [r.numpy().astype(np.int64) for r in hists]
        self.c = counts.tolist()

    def encoding(self, stats_updated, bw, symmetric, strict, unsigned_sym):
        from oracle import OracleTfeAnalyzer
        a = OracleTfeAnalyzer(self.o)
        a.stats_updated = bool(stats_updated)
        if self.x_left is not None:
            a.x_left[:] = self.x_left
            a.initialized = C.c_int(1)
            for h, c in zip(self.h, self.c):
                if c:
                    hh = np.ascontiguousarray(h, np.uint32)
                    self.o.lib.orc_pdf_accumulate(hh.ctypes.data_as(C.POINTER(C.c_uint32)), int(c),
                                                  a.pdf.ctypes.data_as(C.POINTER(C.c_double)), C.byref(a.iterations))
        return torch.from_numpy(a.compute(bw, symmetric, strict, unsigned_sym))


class GlobalRowsOracleEngine(OracleEngine):
    """Same stand-in, but keeping its rows at their global indices in one dense table, like the CUDA engine does:
    exercises the exchange that all-reduces the table in place."""
    global_rows = True

    def __init__(self):
        super().__init__()
        self.table = torch.zeros((0, 512), dtype=torch.int32)
        self.counts = torch.zeros(0, dtype=torch.int64)

    def _reserve(self, n):
        if n > self.table.shape[0]:
            t, c = torch.zeros((n, 512), dtype=torch.int32), torch.zeros(n, dtype=torch.int64)
            t[:self.table.shape[0]], c[:self.counts.shape[0]] = self.table, self.counts
            self.table, self.counts = t, c

    def add_batch(self, x, row):
        self._reserve(row + 1)
        if self.x_left is None:
            return
        bs, po = self.o.pdf_geometry(self.x_left)
        self.table[row] = torch.from_numpy(self.o.hist512(x.numpy(), bs, po).astype(np.int32))
        self.counts[row] = x.numel()

    def add_empty_row(self, row):
        self._reserve(row + 1)

    def num_rows(self):
        return self.table.shape[0]

    def exchange_views(self, n_total):
        self._reserve(n_total)
        return self.table[:n_total], self.counts[:n_total]

    def encoding(self, stats_updated, bw, symmetric, strict, unsigned_sym):
        self.h = [r.numpy().astype(np.int64) for r in self.table]
        self.c = self.counts.tolist()
        return super().encoding(stats_updated, bw, symmetric, strict, unsigned_sym)


ENGINES = {"packed": OracleEngine, "in_place": GlobalRowsOracleEngine}


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


def _worker(rank, world, port, scenario, out, engine="packed"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from aimet_b200.calibration import TfEnhancedCalibrator
        batches = make_batches(scenario)
        cal = TfEnhancedCalibrator("cpu", engine=ENGINES[engine]())
        rounds = (len(batches) + world - 1) // world
        for k in range(rounds):
            g = k * world + rank
            cal.update(torch.from_numpy(batches[g]) if g < len(batches) else None)
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


@pytest.mark.parametrize("engine", ["packed", "in_place"])
@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("scenario", ["relu", "zeros_first", "all_zero"])
def test_sharded_tf_enhanced_equals_sequential(world, scenario, engine):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), scenario, out, engine), nprocs=world, join=True)
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
    cal = TfEnhancedCalibrator("cpu", engine=OracleEngine())
    for b in batches:
        cal.update(torch.from_numpy(b))
    e = cal.compute_encoding(8)
    w = sequential(batches, 8, (False, False, False))
    assert [e.min, e.max, e.delta, e.offset, e.bw] == list(w)
