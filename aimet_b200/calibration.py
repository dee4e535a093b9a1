"""Data-parallel calibration of one quantizer over the GPUs of a node.

The reference calibrates in a single process: ``compute_encodings`` feeds batches to ``updateStats`` one after
the other (aimet_torch/v1/quantsim.py:381-448, aimet_torch/v2/quantsim/quantsim.py:205-224).  Here batch ``b``
of the calibration set is handled by rank ``b % world_size``; the ranks exchange only small statistics, and the
result is bit-identical to the sequential reference run:

* MinMax: every rank keeps a running min/max, one all-reduce(MIN) and one all-reduce(MAX) combine them (exact,
  order independent).
* TF-Enhanced: the bucket grid is defined by the first batch, in global order, whose (min, max) is not (0, 0)
  (DlQuantization/src/math_functions.cpp:248-262).  Per round the ranks all-gather the (min, max, present) triple of
  their batch and every rank's device picks the defining batch from the gathered table (no host read); the rounds
  with an exchange end as soon as the host has learned, from an asynchronous read, that the grid exists.  Each rank
  histograms its own batches into rows at their GLOBAL batch indices; at the end ONE all-reduce(SUM) over the
  ``[num_batches, 512]`` integer table, the 64-bit counts and a flag word gives every rank every batch's exact
  histogram, and the reference's floating-point running mean (math_functions.cpp:278-287) is replayed in global
  batch order before the SQNR search.  (Summing histograms first would not reproduce the running mean bit for
  bit.)  All ranks hold identical rows and run identical arithmetic, so every rank ends with the same encoding and
  nothing is broadcast.

* SQNR on the aimet_torch v2 histograms (``SqnrCalibrator``): the observer's merge is sequential -- a batch is counted
  over the range that it and all earlier batches cover, and old counts are re-binned with rounding when that range grows
  (aimet_torch/v2/quantization/encoding_analyzer.py:212-262).  Two passes over each rank's batches and two all-reduces:
  finite (min, max) per batch -> every batch's counting range (a scan in global batch order, on every rank) -> integer
  counts per batch -> the merges replayed in global batch order on every rank.

The arithmetic lives behind a small engine interface so that the exchange protocol can be tested on CPU ranks
(gloo) with a stand-in engine; the product engine is ``CudaTfeEngine`` and runs everything on the device.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .libpymo import TfEncoding


class CudaTfeEngine:
    """TF-Enhanced statistics of one quantizer on one GPU (kernels through the C ABI).

    Engine interface (what ``TfEnhancedCalibrator`` needs; the CPU stand-in of the protocol tests has the same):
    ``reserve``, ``mark_updated``, ``offer_grid``, ``grid_known``, ``batch_range``, ``select_grid``, ``add_batch``,
    ``add_batches``, ``exchange_buffer``, ``encoding``.
    """

    def __init__(self, device, capacity: int = 256):
        from . import ops   # needs the CUDA library; imported here so that CPU-only protocol tests can run
        self._ops = ops
        self.device = torch.device(device)
        self.state = ops.TfeDeviceState(self.device, capacity)
        self._marked = False

    def reserve(self, rows: int) -> None:
        self.state.reserve(rows)

    def mark_updated(self) -> None:
        """Sets the device-side "this rank offered a batch" flag (summed over ranks by the exchange)."""
        if not self._marked:
            self.state.flags[0:1].fill_(1)
            self._marked = True

    def offer_grid(self, x: torch.Tensor) -> None:
        """The batch's (min, max) goes straight to the device-side grid setup, which ignores it when the grid exists
        or the batch is all zeros; nothing waits for the device."""
        self.state.offer_grid(x)
        self.state.start_probe()

    def grid_known(self, wait: bool = False) -> bool:
        """Whether the HOST has learned that the grid exists (never waits for the device unless ``wait``)."""
        return self.state.poll_initialized(wait)

    def batch_range(self, x: Optional[torch.Tensor]) -> torch.Tensor:
        return self.state.batch_range(x)

    def select_grid(self, ranges: torch.Tensor, num_ranks: int, rank: int) -> None:
        self.state.select_grid(ranges, num_ranks, rank)
        self.state.start_probe()

    def add_batch(self, x: torch.Tensor, row: int, gated: bool = False) -> None:
        self.state.add_batch(x, row, gated)

    def add_batches(self, xs: Sequence[torch.Tensor], row0: int, row_stride: int) -> None:
        self.state.add_batches(xs, row0, row_stride)

    def exchange_buffer(self, n_total: int) -> torch.Tensor:
        """The dense int32 buffer to all-reduce in place: n_total rows, their counts, the flag words."""
        self.state.resize_exact(n_total)
        return self.state.buffer

    def encoding(self, stats_updated, bw: int, symmetric: bool, strict: bool, unsigned_sym: bool,
                 num_rows: Optional[int] = None) -> torch.Tensor:
        return self.state.compute_encoding(stats_updated, bw, symmetric, strict, unsigned_sym, num_rows)


class TfEnhancedCalibrator:
    """TF-Enhanced calibration of one quantizer, sharded by batch over the ranks of ``group``.

    Every rank calls ``update(x)`` once per calibration round, in the same order (round k holds global batches
    k * world_size ... k * world_size + world_size - 1; rank r feeds batch k * world_size + r).  A rank that has no
    batch left in the last round passes ``None``.  ``update_many(xs)`` feeds several rounds at once when the batches
    are resident already; every rank must pass the same number of rounds.  ``num_batches`` (the job's total over all
    ranks, when known) sizes the row table once instead of growing it during the job.
    """

    def __init__(self, device, group=None, engine=None, num_batches: Optional[int] = None):
        self.device = torch.device(device)
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        cap = int(num_batches) if num_batches else 256
        self.engine = engine if engine is not None else CudaTfeEngine(self.device, cap)
        if engine is not None and num_batches:
            self.engine.reserve(int(num_batches))
        self.round = 0
        self.updated = False
        self._merged = False
        self._known = False       # host knowledge that the grid exists (same on every rank in every round)
        self._gathered = None     # [world, 3] table of the grid agreement, allocated once
        self._host_table = None
        self._table_read = None   # (pinned copy of the table, event) of the previous round, not yet looked at

    # ---- statistics ---------------------------------------------------------------------------------------------
    def _grid_known(self, wait: bool = False) -> bool:
        """Whether this rank's HOST knows that the grid exists.  With several ranks the answer must be the same on
        every rank in every round (it decides whether the round has a collective), so it is derived from the gathered
        table of the previous round -- identical everywhere -- whose copy to pinned memory was queued before that
        round's histogram: by the time it is waited for, the device is busy with that histogram."""
        if self._known:
            return True
        if not self.distributed:
            self._known = self.engine.grid_known(wait)
            return self._known
        pending = self._table_read
        if pending is None:
            return False
        host, event = pending
        if event is not None:
            event.synchronize()
        self._table_read = None
        for r in range(self.world):   # global order inside the round == rank order
            mn, mx, present = host[3 * r:3 * r + 3].tolist()
            if present and not (mn == 0.0 and mx == 0.0):
                self._known = True
                break
        return self._known

    def _exchange_round(self, x: Optional[torch.Tensor], row: int) -> None:
        """One round with grid agreement: the device decides (no host read in between) which batch of the round
        defines the grid and whether this rank's batch counts."""
        eng = self.engine
        mine = eng.batch_range(x)
        if self._gathered is None:
            cuda = self.device.type == "cuda"
            self._gathered = torch.empty(self.world * 3, dtype=torch.float32, device=self.device)
            self._host_table = torch.empty(self.world * 3, dtype=torch.float32, pin_memory=cuda)
        dist.all_gather_into_tensor(self._gathered, mine, group=self.group)
        eng.select_grid(self._gathered, self.world, self.rank)
        self._host_table.copy_(self._gathered, non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(self.device))
        self._table_read = (self._host_table, event)
        if x is not None:
            eng.add_batch(x, row, gated=True)

    def update(self, x: Optional[torch.Tensor]) -> None:
        eng = self.engine
        row = self.round * self.world + self.rank
        self.round += 1
        if x is not None and not self.updated:
            self.updated = True
            eng.mark_updated()
        if self._grid_known():
            if x is not None:
                eng.add_batch(x, row)
        elif self.distributed:
            self._exchange_round(x, row)
        elif x is not None:
            # no exchange needed: the device decides whether this batch defines the grid (a batch seen while no
            # grid exists keeps count 0 and is skipped by the replay, exactly like the reference drops it)
            eng.offer_grid(x)
            eng.add_batch(x, row)

    def update_many(self, xs: Sequence[torch.Tensor]) -> None:
        """``len(xs)`` consecutive rounds.  Until the host knows that the grid exists the batches go one by one
        (each launch must see the state its predecessors left); after that, many per launch."""
        i = 0
        while i < len(xs) and not self._grid_known():
            self.update(xs[i])
            i += 1
            # wait for the read queued behind the grid setup -- the device meanwhile works on the histogram that was
            # queued behind it, so this costs the host a few microseconds and the device nothing
            self._grid_known(wait=True)
        rest = xs[i:]
        if not len(rest):
            return
        if not self.updated:
            self.updated = True
            self.engine.mark_updated()
        row0 = self.round * self.world + self.rank
        self.round += len(rest)
        self.engine.add_batches(rest, row0, self.world)

    # ---- encoding -----------------------------------------------------------------------------------------------
    def compute_encoding(self, bw: int, symmetric: bool = False, strict: bool = False,
                         unsigned_sym: bool = False) -> TfEncoding:
        eng = self.engine
        if self.distributed:
            # All ranks have called update() the same number of times, so the row count needs no agreement.  Every
            # row is non-zero on exactly one rank, so the element-wise integer sum reproduces each batch's exact
            # histogram and 64-bit count on every rank; the flag word sums to the number of ranks that saw data.
            n_total = self.round * self.world
            if not self._merged:
                dist.all_reduce(eng.exchange_buffer(n_total), op=dist.ReduceOp.SUM, group=self.group)
                self._merged = True   # statistics are final from here on (further update() calls are not merged)
            enc = eng.encoding(None, bw, symmetric, strict, unsigned_sym, n_total)
        else:
            enc = eng.encoding(self.updated, bw, symmetric, strict, unsigned_sym, self.round)
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


class SqnrCalibrator:
    """SQNR calibration of one quantizer on the aimet_torch v2 histogram statistics, sharded by batch over the ranks of
    ``group``; the statistics (and so the encodings) are those of one process feeding all batches in global order to
    ``SqnrEncodingAnalyzer.update_stats``.

    ``analyzer``: an ``aimet_b200.v2.encoding_analyzer.SqnrEncodingAnalyzer`` (any analyzer whose ``observer`` offers
    ``batch_range`` / ``plan_batches`` / ``count_batch`` / ``replay_batches``).  ``calibrate(batches)`` takes this
    rank's batches -- entry ``k`` is global batch ``k * world_size + rank``, ``None`` where the rank has none -- as a
    sequence or as a callable that returns a fresh iterator (the batches are read twice).  Every rank passes the same
    number of entries.
    """

    def __init__(self, analyzer, device, group=None):
        self.analyzer = analyzer
        self.device = torch.device(device)
        self.group = group
        self.distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.rank = dist.get_rank(group) if self.distributed else 0
        self.world = dist.get_world_size(group) if self.distributed else 1
        self._ranges = None
        self._dtype = torch.float32
        self._rounds = 0

    def _exchange(self, table: torch.Tensor) -> None:
        # every row is non-zero on exactly one rank: the integer sum hands every rank every row, bit for bit
        if self.distributed:
            dist.all_reduce(table, op=dist.ReduceOp.SUM, group=self.group)

    @staticmethod
    def _walker(batches):
        return batches if callable(batches) else (lambda: iter(batches))

    # The three local steps; calibrate() runs them with an exchange after the first two.
    def local_ranges(self, batches) -> torch.Tensor:
        """First pass: int32 ``[rounds * world, histograms, 4]`` with this rank's rows filled, the others zero."""
        obs = self.analyzer.observer
        if not callable(batches) and hasattr(batches, "__len__"):
            # the number of rounds is known: the records go straight into their rows of the table
            self._rounds = len(batches)
            if self._rounds == 0:
                raise ValueError("aimet_b200: no batches to calibrate with")
            ranges = torch.zeros((self._rounds * self.world, obs.num_histograms, 4), dtype=torch.int32,
                                 device=self.device)
            many = getattr(obs, "batch_range_many", None)
            if many is not None and many(batches, ranges, self.rank, self.world):
                self._dtype = next((x.dtype for x in batches if x is not None), self._dtype)
                return ranges
            for k, x in enumerate(batches):
                if x is not None:
                    obs.batch_range(x, ranges[k * self.world + self.rank])
                    self._dtype = x.dtype
            return ranges
        records: List[torch.Tensor] = []
        for x in self._walker(batches)():
            rec = torch.zeros((obs.num_histograms, 4), dtype=torch.int32, device=self.device)
            if x is not None:
                obs.batch_range(x, rec)
                self._dtype = x.dtype
            records.append(rec)
        self._rounds = len(records)
        if not records:
            raise ValueError("aimet_b200: no batches to calibrate with")
        ranges = torch.zeros((self._rounds * self.world, obs.num_histograms, 4), dtype=torch.int32, device=self.device)
        ranges[self.rank::self.world] = torch.stack(records)
        return ranges

    def local_counts(self, batches, ranges: torch.Tensor):
        """Second pass, from every rank's range records: the plans of all batches and int32 ``[rounds * world,
        histograms, bins + 2]`` counts with this rank's rows filled."""
        obs = self.analyzer.observer
        plans = obs.plan_batches(ranges)
        counts = torch.zeros((ranges.shape[0], obs.num_histograms, obs.num_bins + 2), dtype=torch.int32,
                             device=self.device)
        many = getattr(obs, "count_many", None)
        if many is not None and not callable(batches) and hasattr(batches, "__len__") and \
                len(batches) == self._rounds and many(batches, plans, counts, self.rank, self.world):
            return plans, counts
        seen = 0
        for k, x in enumerate(self._walker(batches)()):
            seen += 1
            if x is not None:
                g = k * self.world + self.rank
                obs.count_batch(x, plans[g], counts[g])
        if seen != self._rounds:
            raise RuntimeError("aimet_b200: the batches changed between the two passes")
        return plans, counts

    def finish(self, ranges: torch.Tensor, plans: torch.Tensor, counts: torch.Tensor) -> None:
        self.analyzer.observer.replay_batches(counts, plans, self._dtype)
        self._ranges = ranges

    def calibrate(self, batches) -> None:
        ranges = self.local_ranges(batches)
        self._exchange(ranges)
        plans, counts = self.local_counts(batches, ranges)
        self._exchange(counts)
        self.finish(ranges, plans, counts)

    def compute_encodings(self, num_steps: int, is_symmetric: bool):
        """(min, max) like ``SqnrEncodingAnalyzer.compute_encodings``; identical on every rank."""
        if self._ranges is None:
            raise RuntimeError("aimet_b200: calibrate() has not run")
        present, finite = self._ranges[..., 3] != 0, self._ranges[..., 2] != 0
        if bool((present & ~finite).any()):
            raise ValueError("Input tensor cannot contain only infinite or only NaN values")
        if not bool((present & finite).any()):
            raise ValueError("aimet_b200: no batch was offered on any rank")
        return self.analyzer.compute_encodings(num_steps, is_symmetric)
