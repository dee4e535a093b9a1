"""Encoding analyzers with the interface of ``aimet_torch.v2.quantization.encoding_analyzer``.

``MinMaxEncodingAnalyzer`` mirrors the reference class of the same name
(TrainingExtensions/torch/src/python/aimet_torch/v2/quantization/encoding_analyzer.py:272-386): same constructor,
``update_stats`` / ``reset_stats`` / ``compute_encodings`` / ``compute_dynamic_encodings`` /
``compute_encodings_from_stats``, same exceptions, ``.observer.shape``.  The per-batch reduction to the encoding
shape is ONE fused min+max kernel on the B200 (the reference permutes, reshapes and reduces twice).

``TfEnhancedEncodingAnalyzer`` exposes the libpymo TF-Enhanced calibration (512-bucket PDF + SQNR search,
DlQuantization/src/TfEnhancedEncodingAnalyzer.cpp) through the same analyzer interface, per tensor.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .. import ops
from ..libpymo import _TfEnhancedStats
from .backend import resolve_geometry

_MINIMUM_SCALE = torch.finfo(torch.float32).eps


_SCALARS = {}


def device_scalar(value: float, dtype: torch.dtype, device) -> torch.Tensor:
    """A 0-dim device tensor holding ``value``, made once per (value, dtype, device): creating one per call costs a
    host-to-device copy each time, and the encoding arithmetic needs three or four of them per quantizer."""
    key = (float(value), dtype, str(device))
    t = _SCALARS.get(key)
    if t is None:
        t = _SCALARS[key] = torch.tensor(float(value), dtype=dtype, device=device)
    return t


class StatisticsNotFoundError(RuntimeError):
    """No statistics were collected before encodings were requested (aimet_torch/v2/utils.py)."""


@dataclass
class _MinMaxRange:
    min: Optional[torch.Tensor] = None
    max: Optional[torch.Tensor] = None


class _MinMaxObserver:
    """Running min / max per encoding (reference: _MinMaxObserver, encoding_analyzer.py:92-128).

    The running range lives in one float32 device tensor ``[2, count]`` (mins, then maxs, in the encoding's own
    flattened order) whatever the dtype of the observed tensors -- float32 holds float16 / bfloat16 values exactly --
    so that the fused calibration step (:meth:`MinMaxEncodingAnalyzer.fused_update`) can update it in place; the
    ``_MinMaxRange`` the reference exposes is built from it on request, in the dtype of the observed tensors."""

    def __init__(self, shape):
        if isinstance(shape, int):
            shape = (shape,)
        self.shape = tuple(shape)
        self._running: Optional[torch.Tensor] = None
        self._valid = False
        self._dtype = torch.float32

    def _geometry(self, input_tensor: torch.Tensor):
        if not input_tensor.is_cuda:
            raise RuntimeError("aimet_b200: statistics are collected on the GPU only (no CPU path exists)")
        x = input_tensor.detach()
        if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise RuntimeError(f"aimet_b200: unsupported dtype {x.dtype}")
        enc_shape = self.shape
        if len(enc_shape) > x.dim() or any(s not in (1, t) for s, t in zip(enc_shape[::-1], tuple(x.shape)[::-1])):
            raise RuntimeError(f"Shape {self.shape} is incompatible with input of shape {tuple(x.shape)}")
        return x, resolve_geometry(x, enc_shape, None)

    @torch.no_grad()
    def collect_stats(self, input_tensor: torch.Tensor) -> _MinMaxRange:
        x, g = self._geometry(input_tensor)
        enc_shape = self.shape
        mm = ops.minmax(g.x_work, g.num_ch, g.inner, propagate_nan=True)   # [2, num_ch] float32, channel order
        # channel order -> the encoding's own layout
        view = [s for s in g.enc_view]
        if g.enc_perm != list(range(len(view))):
            perm_shape = [view[d] for d in g.enc_perm]
            inv = [g.enc_perm.index(d) for d in range(len(view))]
            mn = mm[0].reshape(perm_shape).permute(inv)
            mx = mm[1].reshape(perm_shape).permute(inv)
        else:
            mn, mx = mm[0], mm[1]
        mn = mn.reshape(enc_shape).to(x.dtype)
        mx = mx.reshape(enc_shape).to(x.dtype)
        return _MinMaxRange(mn, mx)

    @torch.no_grad()
    def merge_stats(self, stats: _MinMaxRange):
        if stats.min is None or stats.max is None:
            return
        new = torch.stack([stats.min.detach().float().reshape(-1), stats.max.detach().float().reshape(-1)])
        if not self._valid or self._running is None or self._running.shape != new.shape \
                or self._running.device != new.device:
            self._running, self._dtype = new, stats.min.dtype
        else:
            self._running[0] = torch.minimum(self._running[0], new[0])
            self._running[1] = torch.maximum(self._running[1], new[1])
        self._valid = True

    def reset_stats(self):
        self._valid = False

    def get_stats(self) -> _MinMaxRange:
        if not self._valid:
            return _MinMaxRange()
        return _MinMaxRange(self._running[0].view(self.shape).to(self._dtype),
                            self._running[1].view(self.shape).to(self._dtype))

    @property
    def stats(self) -> _MinMaxRange:
        return self.get_stats()


class EncodingAnalyzer:
    """Base class (reference: EncodingAnalyzer, encoding_analyzer.py:272-319)."""

    def __init__(self, observer):
        self.observer = observer

    @torch.no_grad()
    def update_stats(self, input_tensor: torch.Tensor):
        new_stats = self.observer.collect_stats(input_tensor)
        self.observer.merge_stats(new_stats)
        return new_stats

    def reset_stats(self):
        self.observer.reset_stats()

    def compute_encodings(self, num_steps: int, is_symmetric: bool):
        return self.compute_encodings_from_stats(self.observer.get_stats(), num_steps, is_symmetric)

    def compute_dynamic_encodings(self, input_tensor: torch.Tensor, num_steps: int, is_symmetric: bool):
        return self.compute_encodings_from_stats(self.observer.collect_stats(input_tensor), num_steps, is_symmetric)

    def compute_encodings_from_stats(self, stats, num_steps: int, is_symmetric: bool):
        raise NotImplementedError


class MinMaxEncodingAnalyzer(EncodingAnalyzer):
    """Min-max calibration: encodings [min(input), max(input)] widened to contain zero
    (reference: MinMaxEncodingAnalyzer, encoding_analyzer.py:325-386)."""

    def __init__(self, shape: tuple):
        super().__init__(_MinMaxObserver(shape))

    @torch.no_grad()
    def fused_update(self, input_tensor: torch.Tensor, num_steps: int, is_symmetric: bool, qmin: int):
        """One calibration step in two launches: the min/max reduction, then -- for all encodings at once -- the merge
        into the running range, the encodings of THIS batch and the scale / offset to quantize it with (the
        reference: update_stats + compute_encodings_from_stats + the quantizer's scale / offset arithmetic, about 25
        small tensor operations).  Returns float32 ``(scale, offset)`` shaped like the observer, or None when the
        encoding's layout is a permutation of the reduction's channel order (the general path handles that)."""
        if num_steps <= 0:
            raise ValueError('The number of quantization bins cannot be less than or equal to 0.')
        obs = self.observer
        x, g = obs._geometry(input_tensor)
        if g.enc_perm != list(range(len(g.enc_view))):
            return None
        count = g.num_ch
        mm = ops.minmax(g.x_work, count, g.inner, propagate_nan=True)
        if obs._running is None or obs._running.shape != mm.shape or obs._running.device != mm.device:
            obs._running, obs._valid = torch.empty_like(mm), False
        out = torch.empty((4, count), dtype=torch.float32, device=mm.device)
        with ops._on(mm):
            check(lib.aq_v2_minmax_encoding(mm.data_ptr(), obs._running.data_ptr(), int(obs._valid), _DT[x.dtype], count,
                                            float(num_steps), int(bool(is_symmetric)), float(qmin), out.data_ptr(),
                                            ops._stream(mm)), "aq_v2_minmax_encoding")
        if not obs._valid:
            obs._dtype = x.dtype
        obs._valid = True
        return out[2].view(obs.shape), out[3].view(obs.shape)

    @torch.no_grad()
    def compute_encodings(self, num_steps: int, is_symmetric: bool):
        obs = self.observer
        if num_steps <= 0:
            raise ValueError('The number of quantization bins cannot be less than or equal to 0.')
        if not obs._valid:
            raise StatisticsNotFoundError('No statistics present to compute encodings.')
        count = obs._running.shape[1]
        out = torch.empty((4, count), dtype=torch.float32, device=obs._running.device)
        with ops._on(out):
            check(lib.aq_v2_minmax_encoding(None, obs._running.data_ptr(), 1, _DT[obs._dtype], count, float(num_steps),
                                            int(bool(is_symmetric)), 0.0, out.data_ptr(), ops._stream(out)),
                  "aq_v2_minmax_encoding")
        return out[0].view(obs.shape).to(obs._dtype), out[1].view(obs.shape).to(obs._dtype)

    @torch.no_grad()
    def compute_encodings_from_stats(self, stats: _MinMaxRange, num_steps: int, is_symmetric: bool) \
            -> Tuple[torch.Tensor, torch.Tensor]:
        # The statistics are at most a few thousand values; this mirrors the reference expression for expression
        # (including its type promotion: the adjustment term is a float32 tensor) on the device.
        if num_steps <= 0:
            raise ValueError('The number of quantization bins cannot be less than or equal to 0.')
        if stats.min is None or stats.max is None:
            raise StatisticsNotFoundError('No statistics present to compute encodings.')
        # Divisors are 0-dim device tensors, not Python scalars: dividing a CUDA tensor by a host scalar is
        # evaluated as a multiplication by the reciprocal, which is not the IEEE quotient the CPU reference gets.
        def divisor(v):
            return device_scalar(v, torch.float32, stats.min.device)

        min_with_zero = torch.clamp(stats.min, max=0)
        max_with_zero = torch.clamp(stats.max, min=0)
        tensor_diff = (max_with_zero - min_with_zero) / divisor(num_steps)
        adjustment_step = _MINIMUM_SCALE * (tensor_diff < _MINIMUM_SCALE)
        if is_symmetric:
            updated_max = max_with_zero + math.floor(num_steps / 2) * adjustment_step
            updated_min = min_with_zero - math.ceil(num_steps / 2) * adjustment_step
            num_pos_steps = math.floor(num_steps / 2)
            num_neg_steps = math.ceil(num_steps / 2)
            delta = torch.maximum(updated_max / divisor(num_pos_steps), -updated_min / divisor(num_neg_steps))
            offset = -1 * num_neg_steps
            updated_min = offset * delta
            updated_max = num_pos_steps * delta
        else:
            updated_max = max_with_zero + num_steps * adjustment_step
            updated_min = min_with_zero
        updated_max = torch.clamp(updated_max, max=torch.finfo(stats.min.dtype).max).to(stats.min.dtype)
        updated_min = torch.clamp(updated_min, min=torch.finfo(stats.max.dtype).min).to(stats.max.dtype)
        return updated_min, updated_max


class TfEnhancedEncodingAnalyzer(EncodingAnalyzer):
    """Per-tensor TF-Enhanced (512-bucket PDF + SQNR grid search) behind the analyzer interface.

    Statistics live on the device: one histogram row per batch, replayed in batch order into the reference's
    running-mean PDF when encodings are requested, so the result equals what the reference's sequential
    ``updateStats`` / ``computeEncoding`` calls produce (DlQuantization/src/TfEnhancedEncodingAnalyzer.cpp:60-113).
    ``num_steps`` must be ``2**bw - 1``.
    """

    class _Observer:
        def __init__(self, shape):
            self.shape = tuple(shape)

    #: Inside a quantizer's calibration context the input passes through unquantized while statistics are taken
    #: (the analysis mode of the libpymo flow, aimet_torch/v1/qc_quantize_op.py): no per-batch encoding exists for
    #: these statistics, whose bucket grid is fixed by the first batch.
    calibration_passthrough = True

    def __init__(self, shape: tuple = (1,)):
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        if math.prod(shape) != 1:
            raise RuntimeError("aimet_b200: TfEnhancedEncodingAnalyzer computes one encoding per tensor")
        super().__init__(self._Observer(shape))
        self._stats = _TfEnhancedStats()

    @torch.no_grad()
    def update_stats(self, input_tensor: torch.Tensor):
        if not input_tensor.is_cuda:
            raise RuntimeError("aimet_b200: statistics are collected on the GPU only (no CPU path exists)")
        x = input_tensor.detach()
        if x.dtype != torch.float32:
            x = x.float()   # the reference's callers upcast before the native call
        if not x.is_contiguous():
            x = x.contiguous()
        self._stats.update(x)
        return None

    def reset_stats(self):
        self._stats = _TfEnhancedStats()

    def compute_encodings(self, num_steps: int, is_symmetric: bool, strict_symmetric: bool = False,
                          unsigned_symmetric: bool = False):
        if num_steps <= 0:
            raise ValueError('The number of quantization bins cannot be less than or equal to 0.')
        if not self._stats.updated:
            raise StatisticsNotFoundError('No statistics present to compute encodings.')
        bw = int(round(math.log2(num_steps + 1)))
        if 2 ** bw - 1 != num_steps:
            raise ValueError("TF-Enhanced encodings are defined for num_steps = 2**bw - 1")
        e = self._stats.compute(bw, is_symmetric, strict_symmetric, unsigned_symmetric)
        dev = self._stats.dev.device
        mn = torch.tensor(e.min, dtype=torch.float32, device=dev).view(self.observer.shape)
        mx = torch.tensor(e.max, dtype=torch.float32, device=dev).view(self.observer.shape)
        return mn, mx

    def compute_dynamic_encodings(self, input_tensor, num_steps, is_symmetric):
        a = TfEnhancedEncodingAnalyzer(self.observer.shape)
        a.update_stats(input_tensor)
        return a.compute_encodings(num_steps, is_symmetric)

    def compute_encodings_from_stats(self, stats, num_steps, is_symmetric):
        raise RuntimeError("aimet_b200: TF-Enhanced statistics are device-resident; use compute_encodings()")


# ---------------------------------------------------------------------------------------------------
# v2 histogram statistics + SQNR search
# ---------------------------------------------------------------------------------------------------
from .. import _lib   # noqa: E402
from .._lib import check, lib   # noqa: E402

_DT = {torch.float32: _lib.AQ_F32, torch.float16: _lib.AQ_F16, torch.bfloat16: _lib.AQ_BF16}


class _Histogram:
    """Host view of one histogram (reference: _Histogram, encoding_analyzer.py:57-62): ``histogram``, ``bin_edges``,
    ``min``, ``max``.  When it describes device-resident statistics the four tensors are views of one row of the
    statistics tensor, made on first access (a per-channel observer hands out thousands of these); reading their
    values synchronises like any device tensor."""

    def __init__(self, histogram=None, bin_edges=None, min=None, max=None):   # pylint: disable=redefined-builtin
        self._fields = {"histogram": histogram, "bin_edges": bin_edges, "min": min, "max": max}
        self._blocks = None    # [rows, words] int32 statistics tensor
        self._row = 0
        self._num_bins = 0
        self._dtype = torch.float32
        self._rows = None      # the batch these statistics were collected from, until it has been merged

    @staticmethod
    def of_block(blocks: torch.Tensor, row: int, num_bins: int, dtype: torch.dtype) -> "_Histogram":
        h = _Histogram()
        h._blocks, h._row, h._num_bins, h._dtype = blocks, row, num_bins, dtype
        return h

    @property
    def _block(self) -> Optional[torch.Tensor]:
        return None if self._blocks is None else self._blocks[self._row]

    def _get(self, name):
        if self._fields[name] is None and self._blocks is not None:
            f, nb = self._blocks[self._row].view(torch.float32), self._num_bins
            self._fields["histogram"] = f[4:4 + nb]
            self._fields["bin_edges"] = f[4 + nb:4 + 2 * nb + 1]
            self._fields["min"] = f[0].to(self._dtype)
            self._fields["max"] = f[1].to(self._dtype)
        return self._fields[name]

    histogram = property(lambda self: self._get("histogram"))
    bin_edges = property(lambda self: self._get("bin_edges"))
    min = property(lambda self: self._get("min"))
    max = property(lambda self: self._get("max"))

    def __repr__(self):
        return f"_Histogram(min={self.min}, max={self.max}, bins={self._num_bins})"


class _HistogramRows:
    """The list of ``_Histogram`` views of a statistics tensor, one per row, made when an entry is asked for (a
    per-channel observer has thousands of rows and most callers hand the list straight back to the analyzer)."""

    def __init__(self, blocks: torch.Tensor, count: int, num_bins: int, dtype: torch.dtype):
        self.blocks, self.count, self.num_bins, self.dtype = blocks, count, num_bins, dtype
        self._made = {}

    def __len__(self):
        return self.count

    def __getitem__(self, i):
        if isinstance(i, slice):
            return [self[j] for j in range(*i.indices(self.count))]
        if i < 0:
            i += self.count
        if not 0 <= i < self.count:
            raise IndexError(i)
        h = self._made.get(i)
        if h is None:
            h = self._made[i] = _Histogram.of_block(self.blocks, i, self.num_bins, self.dtype)
        return h

    def __iter__(self):
        return (self[i] for i in range(self.count))


def _joint_blocks(stats) -> torch.Tensor:
    """The statistics tensor whose rows the given histograms are, in order (a copy only if they are not)."""
    if isinstance(stats, _HistogramRows) and stats.blocks.shape[0] == stats.count:
        return stats.blocks
    blocks = stats[0]._blocks
    if blocks is not None and blocks.shape[0] == len(stats) and all(h._blocks is blocks and h._row == i
                                                                     for i, h in enumerate(stats)):
        return blocks
    return torch.stack([h._block for h in stats])


def _block_words(num_bins: int) -> int:
    """int32 words of one statistics block (header + histogram + edges), rounded up to 16 bytes."""
    return ((_lib.V2HIST_HEAD_BYTES + (2 * num_bins + 1) * 4 + 15) // 16) * 4


def _new_blocks(count: int, num_bins: int, device) -> torch.Tensor:
    """Statistics blocks for the kernels to fill (every field of a block is written by the launch that produces it)."""
    return torch.empty((count, _block_words(num_bins)), dtype=torch.int32, device=device)


class _HistogramObserver:
    """Per-encoding histograms of everything seen so far (reference: _HistogramObserver, encoding_analyzer.py:131-270).

    ``collect_stats`` gives the batch's own histograms (finite min / max, ``torch.histc`` counts over that range,
    infinities folded into the end bins); ``merge_stats`` widens the running histograms' range when needed, re-bins
    the old counts with the reference's split-and-round rule and counts the batch again at the widened range.  All of
    it runs on the device, no host synchronisation.  With several histograms (per-channel observers) the reference
    loops over the channels in Python; here all channels go through the same few launches (one grid row each), and
    their statistics blocks are the rows of one tensor.
    """

    def __init__(self, shape: tuple, num_bins: int):
        if isinstance(shape, int):
            shape = (shape,)
        self.shape = tuple(shape)
        self.num_bins = int(num_bins)
        if self.num_bins > _lib.AQ_V2HIST_MAX_BINS:
            raise ValueError(f"aimet_b200: at most {_lib.AQ_V2HIST_MAX_BINS} histogram bins are supported")
        self.num_histograms = int(math.prod(self.shape))
        if self.num_histograms > 65535:
            raise ValueError("aimet_b200: at most 65535 histograms per observer")
        self._state = None          # [num_histograms, words] int32 device tensor once statistics exist
        self._dtype = torch.float32
        self._scratch = None
        self._updates = None

    # ---- helpers ---------------------------------------------------------------------------------------------
    def _buffers(self, device):
        if self._scratch is None or self._scratch.device != device:
            self._scratch = torch.empty(self.num_histograms * int(lib.aq_v2hist_scratch_bytes()), dtype=torch.uint8,
                                        device=device)
            self._updates = torch.empty(self.num_histograms * self.num_bins, dtype=torch.float32, device=device)
        return self._scratch, self._updates

    def _rows(self, input_tensor: torch.Tensor) -> torch.Tensor:
        """The input as a dense [num_histograms, elements per histogram] matrix, in histogram order (no copy when the
        encoding axes already lead, e.g. a weight observed per output channel)."""
        x = input_tensor.detach()
        if not x.is_cuda:
            raise RuntimeError("aimet_b200: statistics are collected on the GPU only (no CPU path exists)")
        if x.dtype not in _DT:
            raise RuntimeError(f"aimet_b200: unsupported dtype {x.dtype}")
        enc_shape = self.shape
        if len(enc_shape) > x.dim() or any(s not in (1, t) for s, t in zip(enc_shape[::-1], tuple(x.shape)[::-1])):
            raise RuntimeError(f"Shape {self.shape} is incompatible with input of shape {tuple(x.shape)}")
        if self.num_histograms == 1:
            return x.reshape(1, -1).contiguous()
        padded = (1,) * (x.dim() - len(enc_shape)) + tuple(enc_shape)
        axes = [a for a, d in enumerate(padded) if d != 1]
        rest = [a for a in range(x.dim()) if a not in axes]
        return x.permute(axes + rest).reshape(self.num_histograms, -1).contiguous()

    def _views(self, blocks: torch.Tensor, dtype: torch.dtype):
        return _HistogramRows(blocks, self.num_histograms, self.num_bins, dtype)

    # ---- observer interface ----------------------------------------------------------------------------------
    @torch.no_grad()
    def collect_stats(self, input_tensor: torch.Tensor):
        rows = self._rows(input_tensor)
        scratch, _ = self._buffers(input_tensor.device)
        stream = torch.cuda.current_stream(input_tensor.device).cuda_stream
        blocks = _new_blocks(self.num_histograms, self.num_bins, rows.device)
        with ops._on(input_tensor):
            check(lib.aq_v2hist_collect_rows(rows.data_ptr(), _DT[rows.dtype], rows.shape[1], self.num_histograms,
                                             self.num_bins, blocks.data_ptr(), blocks.stride(0) * 4, scratch.data_ptr(),
                                             stream), "aq_v2hist_collect_rows")
        out = self._views(blocks, input_tensor.dtype)
        out[0]._rows = rows   # kept for the merge that usually follows
        return out

    @torch.no_grad()
    def merge_stats(self, new_stats_list, input_tensor: torch.Tensor):
        scratch, updates = self._buffers(input_tensor.device)
        stream = torch.cuda.current_stream(input_tensor.device).cuda_stream
        first = self._state is None
        if first:
            self._state = _new_blocks(self.num_histograms, self.num_bins, input_tensor.device)
            self._dtype = input_tensor.dtype
        rows = new_stats_list[0]._rows
        if rows is None:
            rows = self._rows(input_tensor)
        blocks = _joint_blocks(new_stats_list)
        with ops._on(input_tensor):
            check(lib.aq_v2hist_merge_rows(rows.data_ptr(), _DT[rows.dtype], rows.shape[1], self.num_histograms,
                                           self.num_bins, self._state.data_ptr(), blocks.data_ptr(),
                                           blocks.stride(0) * 4, 0 if first else 1, scratch.data_ptr(),
                                           updates.data_ptr(), stream), "aq_v2hist_merge_rows")
        new_stats_list[0]._rows = None   # the batch need not outlive the update

    @torch.no_grad()
    def update_stats(self, input_tensor: torch.Tensor):
        """collect_stats + merge_stats of one batch with a single counting pass (two passes over the data, not three)."""
        rows = self._rows(input_tensor)
        scratch, updates = self._buffers(input_tensor.device)
        stream = torch.cuda.current_stream(input_tensor.device).cuda_stream
        first = self._state is None
        if first:
            self._state = _new_blocks(self.num_histograms, self.num_bins, input_tensor.device)
            self._dtype = input_tensor.dtype
        blocks = _new_blocks(self.num_histograms, self.num_bins, rows.device)
        with ops._on(input_tensor):
            check(lib.aq_v2hist_update_rows(rows.data_ptr(), _DT[rows.dtype], rows.shape[1], self.num_histograms,
                                            self.num_bins, self._state.data_ptr(), blocks.data_ptr(),
                                            blocks.stride(0) * 4, 0 if first else 1, scratch.data_ptr(),
                                            updates.data_ptr(), stream), "aq_v2hist_update_rows")
        return self._views(blocks, input_tensor.dtype)

    # ---- the same statistics from batches that are spread over several workers (aimet_b200.calibration) -------------
    # merge_stats is sequential (the range a batch is counted over depends on every earlier batch), so the work is cut
    # into: the batches' finite ranges -> [exchange] -> every batch's counting range -> counts -> [exchange] -> replay.
    @torch.no_grad()
    def batch_range(self, input_tensor: torch.Tensor, out: torch.Tensor) -> None:
        """Writes the batch's range records (int32 ``[num_histograms, 4]``: min bits, max bits, any finite, 1)."""
        rows = self._rows(input_tensor)
        scratch, _ = self._buffers(input_tensor.device)
        with ops._on(input_tensor):
            check(lib.aq_v2hist_range_rows(rows.data_ptr(), _DT[rows.dtype], rows.shape[1], self.num_histograms,
                                           out.data_ptr(), scratch.data_ptr(),
                                           torch.cuda.current_stream(input_tensor.device).cuda_stream),
                  "aq_v2hist_range_rows")

    @torch.no_grad()
    def plan_batches(self, ranges: torch.Tensor) -> torch.Tensor:
        """``ranges``: int32 ``[n_batches, num_histograms, 4]`` in batch order -> float32 ``[n_batches, num_histograms,
        8]``: the range every batch is counted over."""
        plans = torch.empty(ranges.shape[:2] + (8,), dtype=torch.float32, device=ranges.device)
        with ops._on(ranges):
            check(lib.aq_v2hist_plan_batches(ranges.data_ptr(), ranges.shape[0], self.num_histograms, self.num_bins,
                                             plans.data_ptr(), torch.cuda.current_stream(ranges.device).cuda_stream),
                  "aq_v2hist_plan_batches")
        return plans

    @torch.no_grad()
    def count_batch(self, input_tensor: torch.Tensor, plan: torch.Tensor, out: torch.Tensor) -> None:
        """Counts the batch over ``plan`` (one batch's rows of ``plan_batches``) and adds the counts to ``out``, int32
        ``[num_histograms, num_bins + 2]`` (zero-filled by the caller)."""
        rows = self._rows(input_tensor)
        with ops._on(input_tensor):
            check(lib.aq_v2hist_count_rows(rows.data_ptr(), _DT[rows.dtype], rows.shape[1], self.num_histograms,
                                           self.num_bins, plan.data_ptr(), out.data_ptr(),
                                           torch.cuda.current_stream(input_tensor.device).cuda_stream),
                  "aq_v2hist_count_rows")

    def _uniform_rows(self, batches):
        """For a list of batches (``None`` = absent): their row matrices, when all present ones have one shape and dtype
        and need no copy to become row matrices -- otherwise ``None`` (the caller then goes batch by batch)."""
        rows, like = [], None
        for x in batches:
            if x is None:
                rows.append(None)
                continue
            if not x.is_cuda or x.dtype not in _DT:
                return None
            r = self._rows(x)
            if r.data_ptr() != x.data_ptr() or (like is not None and (r.shape != like.shape or r.dtype != like.dtype)):
                return None
            like = r
            rows.append(r)
        return None if like is None else (rows, like)

    @torch.no_grad()
    def batch_range_many(self, batches, table: torch.Tensor, first: int, step: int) -> bool:
        """``batch_range`` of ``batches[k]`` into ``table[first + k * step]`` for all k with one native call; False (and
        nothing done) when the batches are not uniform enough for that."""
        import ctypes
        uniform = self._uniform_rows(batches)
        if uniform is None:
            return False
        rows, like = uniform
        ptrs = (ctypes.c_void_p * len(rows))(*[None if r is None else r.data_ptr() for r in rows])
        scratch, _ = self._buffers(like.device)
        with ops._on(like):
            check(lib.aq_v2hist_range_many(ptrs, len(rows), _DT[like.dtype], like.shape[1], self.num_histograms,
                                           table[first].data_ptr(), step * table.stride(0), scratch.data_ptr(),
                                           torch.cuda.current_stream(like.device).cuda_stream), "aq_v2hist_range_many")
        return True

    @torch.no_grad()
    def count_many(self, batches, plans: torch.Tensor, counts: torch.Tensor, first: int, step: int) -> bool:
        """``count_batch`` of ``batches[k]`` with ``plans[first + k * step]`` into ``counts[first + k * step]``."""
        import ctypes
        uniform = self._uniform_rows(batches)
        if uniform is None:
            return False
        rows, like = uniform
        ptrs = (ctypes.c_void_p * len(rows))(*[None if r is None else r.data_ptr() for r in rows])
        with ops._on(like):
            check(lib.aq_v2hist_count_many(ptrs, len(rows), _DT[like.dtype], like.shape[1], self.num_histograms,
                                           self.num_bins, plans[first].data_ptr(), step * plans.stride(0),
                                           counts[first].data_ptr(), step * counts.stride(0),
                                           torch.cuda.current_stream(like.device).cuda_stream), "aq_v2hist_count_many")
        return True

    @torch.no_grad()
    def replay_batches(self, counts: torch.Tensor, plans: torch.Tensor, dtype: torch.dtype = torch.float32) -> None:
        """Replaces the statistics by those of feeding the counted batches one by one."""
        device = counts.device
        self._state = _new_blocks(self.num_histograms, self.num_bins, device)
        self._dtype = dtype
        with ops._on(counts):
            check(lib.aq_v2hist_replay_batches(counts.data_ptr(), plans.data_ptr(), counts.shape[0], self.num_histograms,
                                               self.num_bins, self._state.data_ptr(), self._state.stride(0) * 4,
                                               torch.cuda.current_stream(device).cuda_stream),
                  "aq_v2hist_replay_batches")

    def reset_stats(self):
        self._state = None

    def get_stats(self):
        if self._state is None:
            return [_Histogram() for _ in range(self.num_histograms)]
        return self._views(self._state, self._dtype)

    @property
    def stats(self):
        return self.get_stats()


class SqnrEncodingAnalyzer(EncodingAnalyzer):
    """SQNR calibration on the v2 histograms (reference: SqnrEncodingAnalyzer, encoding_analyzer.py:522-725): same
    constructor arguments, same candidate grids (17 deltas x 21 offsets + the observed offset, or 101 deltas when
    symmetric), same clipping-weighted noise estimate, first candidate of least noise.  One warp per candidate."""

    def __init__(self, shape: tuple, num_bins: int = 2048, *, asymmetric_delta_candidates=17,
                 symmetric_delta_candidates=101, offset_candidates=21, max_parallelism=64, gamma=3.0):
        if num_bins <= 0:
            raise ValueError('Number of bins cannot be less than or equal to 0.')
        super().__init__(_HistogramObserver(shape=shape, num_bins=num_bins))
        self.asym_delta_candidates = asymmetric_delta_candidates
        self.sym_delta_candidates = symmetric_delta_candidates
        self.num_offset_candidates = offset_candidates
        self.gamma = gamma
        self.max_parallelism = max_parallelism
        self._offsets = {}
        self._ws = None

    @torch.no_grad()
    def update_stats(self, input_tensor: torch.Tensor):
        return self.observer.update_stats(input_tensor)

    def compute_dynamic_encodings(self, input_tensor, num_steps, is_symmetric):
        return self.compute_encodings_from_stats(self.observer.collect_stats(input_tensor), num_steps, is_symmetric)

    @torch.no_grad()
    def fused_update(self, input_tensor: torch.Tensor, num_steps: int, is_symmetric: bool, qmin: int):
        """One calibration step: the statistics update (two passes over the data), then the search on THIS batch's
        histograms with the scale / offset to quantize the batch with computed in the same launch.  Returns float32
        ``(scale, offset)`` shaped like the observer."""
        if num_steps <= 0:
            raise ValueError('The number of quantization bins cannot be less than or equal to 0.')
        obs = self.observer
        stats = obs.update_stats(input_tensor)
        blocks = stats[0]._blocks
        device = blocks.device
        rows = len(stats)
        offsets = self._offset_grid(num_steps, bool(is_symmetric), device)
        need = rows * int(lib.aq_v2hist_sqnr_workspace_bytes())
        if self._ws is None or self._ws.device != device or self._ws.numel() < need:
            self._ws = torch.zeros(need, dtype=torch.uint8, device=device)
        out = torch.empty((rows, 4), dtype=torch.float32, device=device)
        num_deltas = self.sym_delta_candidates if is_symmetric else self.asym_delta_candidates
        with ops._on(out):
            check(lib.aq_v2hist_sqnr_encode_rows(blocks.data_ptr(), blocks.stride(0) * 4, rows, obs.num_bins,
                                                 float(num_steps), int(bool(is_symmetric)), int(num_deltas),
                                                 offsets.data_ptr(), offsets.numel(), float(self.gamma),
                                                 _DT[input_tensor.dtype], float(qmin), out.data_ptr(),
                                                 self._ws.data_ptr(), self._ws.numel(),
                                                 torch.cuda.current_stream(device).cuda_stream),
                  "aq_v2hist_sqnr_encode_rows")
        return out[:, 2].view(obs.shape), out[:, 3].view(obs.shape)

    def _offset_grid(self, num_steps, is_symmetric: bool, device) -> torch.Tensor:
        """The offsets the search walks: host arithmetic of a handful of values, exactly the reference's expressions
        (encoding_analyzer.py:629-632, :644), cached per (num_steps, symmetric, device)."""
        key = (num_steps, is_symmetric, str(device))
        if key not in self._offsets:
            if is_symmetric:
                t = torch.full((1,), (-num_steps) // 2, dtype=torch.float32)
            else:
                num_offsets = min(num_steps + 2, self.num_offset_candidates)
                step = num_steps / (num_offsets - 2)   # 2 fewer: the observed offset is added on the device
                t = torch.round(torch.arange(start=-num_steps, end=step, step=step, dtype=torch.float32))
            self._offsets[key] = t.to(device)
        return self._offsets[key]

    @torch.no_grad()
    def compute_encodings_from_stats(self, stats, num_steps: int, is_symmetric: bool) \
            -> Tuple[torch.Tensor, torch.Tensor]:
        if stats[0]._blocks is None:
            raise StatisticsNotFoundError('No statistics present to compute encodings.')
        if num_steps <= 0:
            raise ValueError('The number of quantization bins cannot be less than or equal to 0.')
        device = stats[0]._blocks.device
        offsets = self._offset_grid(num_steps, bool(is_symmetric), device)
        out = torch.empty((len(stats), 2), dtype=torch.float32, device=device)
        num_deltas = self.sym_delta_candidates if is_symmetric else self.asym_delta_candidates
        stream = torch.cuda.current_stream(device).cuda_stream
        blocks = _joint_blocks(stats)
        need = len(stats) * int(lib.aq_v2hist_sqnr_workspace_bytes())
        if self._ws is None or self._ws.device != device or self._ws.numel() < need:
            self._ws = torch.zeros(need, dtype=torch.uint8, device=device)
        with ops._on(out):
            check(lib.aq_v2hist_sqnr_rows(blocks.data_ptr(), blocks.stride(0) * 4, len(stats), self.observer.num_bins,
                                          float(num_steps), int(bool(is_symmetric)), int(num_deltas),
                                          offsets.data_ptr(), offsets.numel(), float(self.gamma), out.data_ptr(),
                                          self._ws.data_ptr(), self._ws.numel(), stream), "aq_v2hist_sqnr_rows")
        dtype = stats[0]._dtype
        return out[:, 0].to(dtype).view(self.observer.shape), out[:, 1].to(dtype).view(self.observer.shape)
