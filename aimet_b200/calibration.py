"""Data-parallel calibration of one quantizer over the GPUs of a node.

The reference calibrates in a single process: ``compute_encodings`` feeds batches to ``updateStats`` one after
the other (aimet_torch/v1/quantsim.py:381-448, aimet_torch/v2/quantsim/quantsim.py:205-224).  Here batch ``b``
of the calibration set is handled by rank ``b % world_size``; the ranks exchange only small statistics, and the
result is bit-identical to the sequential reference run:

* MinMax: every rank keeps a running min/max, one all-reduce(MIN) and one all-reduce(MAX) combine them (exact,
  order independent).
* TF-Enhanced: the bucket grid is defined by the first batch, in global order, whose (min, max) is not (0, 0)
  (DlQuantization/src/math_functions.cpp:248-262).  The ranks all-gather the (min, max) of their first batches
  until such a batch is found.  Each rank then histograms its own batches into per-batch rows; at the end one
  all-reduce(SUM) over the zero-padded [num_batches, 512] integer table gives every rank every batch's exact
  histogram, and the reference's floating-point running mean (math_functions.cpp:278-287) is replayed in global
  batch order before the SQNR search.  (Summing histograms first would not reproduce the running mean bit for
  bit.)  The encoding is finally broadcast from rank 0.

The arithmetic lives behind a small engine interface so that the exchange protocol can be tested on CPU ranks
(gloo) with a stand-in engine; the product engine is ``CudaTfeEngine`` and runs everything on the device.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .libpymo import TfEncoding


class CudaTfeEngine:
    """TF-Enhanced statistics of one quantizer on one GPU (kernels through the C ABI)."""

    #: rows are addressed by GLOBAL batch index: a rank's rows sit where the merged table wants them (the rows of
    #: other ranks stay zero), so the exchange is an all-reduce of the table itself, with nothing to pack or unpack
    global_rows = True

    def __init__(self, device):
        from . import ops   # needs the CUDA library; imported here so that CPU-only protocol tests can run
        self._ops = ops
        self.device = torch.device(device)
        self.state = ops.TfeDeviceState(self.device)
        self._mm: Optional[torch.Tensor] = None

    def minmax(self, x: torch.Tensor) -> torch.Tensor:
        self._mm = self._ops.minmax(x, 1, None, propagate_nan=False, out=self._mm)
        return self._mm.reshape(-1)

    def init_grid(self, minmax: torch.Tensor) -> None:
        self.state.init_grid_from(minmax.to(self.device, torch.float32).contiguous())

    def is_initialized(self) -> bool:
        return self.state.is_initialized()

    def offer_grid(self, x: torch.Tensor) -> bool:
        """Single-process shortcut: the batch's (min, max) goes straight to the device-side grid setup, which
        ignores it when the grid exists or the batch is all zeros; nothing waits for the device.  Returns True once
        the host has learned that the grid exists."""
        if self.state.poll_initialized():
            return True
        self.state.init_grid_from(self.minmax(x))
        self.state.start_probe()
        return False

    def add_batch(self, x: torch.Tensor, row: int) -> None:
        self.state.add_batch(x, row)

    def add_empty_row(self, row: int) -> None:
        self.state.reserve(row + 1)   # rows are zero-filled; count 0 marks the batch as dropped
        self.state.num_batches = max(self.state.num_batches, row + 1)

    def num_rows(self) -> int:
        return self.state.num_batches

    def rows(self) -> Tuple[torch.Tensor, torch.Tensor]:
        n = self.state.num_batches
        return self.state.hists[:n], self.state.counts[:n]

    def exchange_views(self, n_total: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """The first n_total rows of the histogram table and of the counts, as the tensors to all-reduce in place."""
        self.state.reserve(n_total)
        self.state.num_batches = n_total
        return self.state.hists[:n_total], self.state.counts[:n_total]

    def load_rows(self, hists: torch.Tensor, counts: torch.Tensor) -> None:
        n = hists.shape[0]
        self.state.reserve(n)
        self.state.hists[:n].copy_(hists)
        self.state.counts[:n].copy_(counts)
        self.state.num_batches = n

    def encoding(self, stats_updated: bool, bw: int, symmetric: bool, strict: bool, unsigned_sym: bool) -> torch.Tensor:
        self.state.replay()
        return self.state.search(stats_updated, bw, symmetric, strict, unsigned_sym)


class TfEnhancedCalibrator:
    """TF-Enhanced calibration of one quantizer, sharded by batch over the ranks of ``group``.

    Every rank calls ``update(x)`` once per calibration round, in the same order (round k holds global batches
    k * world_size ... k * world_size + world_size - 1; rank r feeds batch k * world_size + r).  A rank that has no
    batch left in the last round passes ``None``.
    """

    def __init__(self, device, group=None, engine=None):
        self.device = torch.device(device)
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        self.engine = engine if engine is not None else CudaTfeEngine(self.device)
        self.round = 0
        self.updated = False
        self.grid_known = False
        self.local_global_index: List[int] = []   # global batch index of each local row

    def update(self, x: Optional[torch.Tensor]) -> None:
        g = self.round * self.world + self.rank
        self.round += 1
        if x is not None:
            self.updated = True
        defining_rank = None
        if not self.grid_known:
            if not self.distributed and x is not None and hasattr(self.engine, "offer_grid"):
                # no exchange needed: the device decides whether this batch defines the grid (a batch seen while no
                # grid exists keeps count 0 and is skipped by the replay, exactly like the reference drops it)
                self.grid_known = self.engine.offer_grid(x)
            else:
                defining_rank = self._agree_on_grid(x)
        if x is None:
            return
        row = g if getattr(self.engine, "global_rows", False) else len(self.local_global_index)
        self.local_global_index.append(g)
        if defining_rank is not None and self.rank < defining_rank:
            # an all-zero batch that precedes, in global order, the batch that defines the grid: the sequential
            # reference dropped it before the grid existed, so it must not be counted now either
            self.engine.add_empty_row(row)
        else:
            # (a batch seen while no grid exists at all keeps count 0 and is skipped by the replay)
            self.engine.add_batch(x, row)

    def _agree_on_grid(self, x: Optional[torch.Tensor]) -> Optional[int]:
        """Returns the rank whose batch of this round defines the grid, or None if no batch of the round can."""
        bufs = getattr(self, "_grid_bufs", None)
        if bufs is None:
            # (min, max, present) of this rank, and the gathered table; allocated once
            bufs = (torch.zeros(3, dtype=torch.float32, device=self.device),
                    torch.empty(self.world * 3, dtype=torch.float32, device=self.device))
            self._grid_bufs = bufs
        mine, flat = bufs
        if x is not None:
            mine[:2].copy_(self.engine.minmax(x).reshape(2))
            mine[2:].fill_(1.0)
        else:
            mine.zero_()
        if self.distributed:
            dist.all_gather_into_tensor(flat, mine, group=self.group)
            table = flat.view(self.world, 3)
        else:
            table = mine.reshape(1, 3)
        t = table.cpu()
        if not hasattr(self, "_any_present"):
            self._any_present = bool(t[:, 2].any())   # first round: a rank without data now never gets any
        for r in range(self.world):   # global order inside the round == rank order
            mn, mx, present = t[r].tolist()
            if present and not (mn == 0.0 and mx == 0.0):
                self.engine.init_grid(table[r, :2].contiguous())
                self.grid_known = True
                return r
        return None

    def compute_encoding(self, bw: int, symmetric: bool = False, strict: bool = False,
                         unsigned_sym: bool = False) -> TfEncoding:
        eng = self.engine
        if self.distributed and getattr(self, "_merged", None) is not None:
            # the tables were exchanged by an earlier call; every rank already holds all rows
            enc = eng.encoding(self._merged, bw, symmetric, strict, unsigned_sym)
        elif self.distributed and getattr(eng, "global_rows", False):
            # The engine keeps its rows at their global indices, zero elsewhere: the merged table is the element-wise
            # sum over ranks of the tables themselves.  All ranks have called update() the same number of times, so
            # the row count needs no agreement; whether any rank saw data is known from the first round's exchange.
            n_total = self.round * self.world
            if n_total:
                h, c = eng.exchange_views(n_total)
                dist.all_reduce(h, op=dist.ReduceOp.SUM, group=self.group)
                dist.all_reduce(c, op=dist.ReduceOp.SUM, group=self.group)
            any_updated = bool(getattr(self, "_any_present", False) or self.updated)
            self._merged = any_updated
            enc = eng.encoding(any_updated, bw, symmetric, strict, unsigned_sym).clone()
            dist.broadcast(enc, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                           group=self.group)
        elif self.distributed:
            # One exchange: a zero-padded int32 buffer holding [n_total, 512] histogram rows, then the n_total int64
            # counts (as int32 pairs), then the number of ranks that saw data.  Every row is non-zero on exactly one
            # rank, so the element-wise integer sum reproduces each row and each 64-bit count exactly.  n_total needs
            # no agreement step: all ranks have called update() the same number of times.
            dev = self.device
            n_local = eng.num_rows()
            n_total = self.round * self.world
            buf = torch.zeros(n_total * 514 + 2, dtype=torch.int32, device=dev)
            hists = buf[:n_total * 512].view(n_total, 512)
            counts = buf[n_total * 512:n_total * 514].view(torch.int64)
            if n_local:
                idx = torch.tensor(self.local_global_index, dtype=torch.int64, device=dev)
                h, c = eng.rows()
                hists.index_copy_(0, idx, h)
                counts.index_copy_(0, idx, c)
            if self.updated:
                buf[-2:].fill_(1)
            dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group)
            eng.load_rows(hists, counts)
            any_updated = bool(buf[-1].item())
            self._merged = any_updated   # statistics are final from here on (further update() calls are not merged)
            enc = eng.encoding(any_updated, bw, symmetric, strict, unsigned_sym).clone()
            dist.broadcast(enc, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                           group=self.group)
        else:
            enc = eng.encoding(self.updated, bw, symmetric, strict, unsigned_sym)
        e = enc.tolist()
        return TfEncoding(e[0], e[1], e[2], e[3], int(e[4]))


class MinMaxCalibrator:
    """MinMax ("TF") calibration of one quantizer, sharded by batch over the ranks of ``group``."""

    def __init__(self, device, group=None):
        from . import ops
        self._ops = ops
        self.device = torch.device(device)
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.acc = torch.tensor([[float("inf")], [float("-inf")]], dtype=torch.float32, device=self.device)

    def update(self, x: Optional[torch.Tensor]) -> None:
        if x is not None:
            self._ops.minmax(x, 1, None, propagate_nan=False, out=self.acc, accumulate=True)

    def compute_encoding(self, bw: int, symmetric: bool = False, strict: bool = False,
                         unsigned_sym: bool = False) -> TfEncoding:
        mn, mx = self.acc[0].clone(), self.acc[1].clone()
        if self.distributed:
            dist.all_reduce(mn, op=dist.ReduceOp.MIN, group=self.group)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX, group=self.group)
        return TfEncoding._from_c(self._ops.minmax_encoding(bw, float(mn), float(mx), symmetric, strict, unsigned_sym))
