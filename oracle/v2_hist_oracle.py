"""TEST INFRASTRUCTURE ONLY: CPU restatement of the aimet_torch v2 histogram observer.

Follows TrainingExtensions/torch/src/python/aimet_torch/v2/quantization/encoding_analyzer.py:
_HistogramObserver.collect_stats (:145-182), _handle_inputs (:185-192), _create_bin_edges (:194-203),
_get_bin_num (:205-208) and merge_stats (:212-262), for ONE histogram.

PINNED by tests/test_oracle_pin.py against tests/golden/v2_sqnr.npz, which holds what the reference's own class
produced after every update (tests/golden/gen_golden.py).

Arithmetic is numpy float32 (one IEEE rounding per operation, like the reference's float32 tensors).  The counting
itself is ``torch.histc`` of the installed torch on CPU: that operator is third-party code the reference calls, not
something to restate.

Besides the sequential observer (``collect`` / ``merge``) the file has the same work cut into the four steps that
calibration spread over several workers uses -- ``finite_range``, ``plan_batches``, ``count`` and ``replay`` -- so
that the exchange protocol can run on CPU ranks.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

F32 = np.float32
INT_MIN = -2 ** 31


class Hist:
    """One _Histogram: float32 counts, bin edges, min, max."""

    def __init__(self, hist, edges, mn, mx):
        self.hist, self.edges, self.min, self.max = hist, edges, F32(mn), F32(mx)


def finite_range(x: np.ndarray):
    """_handle_inputs: min / max over the finite elements; None when there is none (the reference raises)."""
    x = np.asarray(x, np.float32).reshape(-1)
    f = x[np.isfinite(x)]
    if f.size == 0:
        return None
    return F32(f.min()), F32(f.max())


def bin_edges(mn, mx, bins: int) -> np.ndarray:
    """_create_bin_edges: arange(bins + 1) * step + min, equal bounds widened by 0.5 first."""
    mn, mx = F32(mn), F32(mx)
    if mx == mn:
        mn, mx = F32(mn - F32(0.5)), F32(mx + F32(0.5))
    step = F32(F32(mx - mn) / F32(bins))
    return (np.arange(bins + 1).astype(np.float32) * step + mn).astype(np.float32)


def histc(x: np.ndarray, bins: int, lo, hi) -> np.ndarray:
    t = torch.from_numpy(np.ascontiguousarray(np.asarray(x, np.float32).reshape(-1)))
    return torch.histc(t, bins=bins, min=float(lo), max=float(hi)).numpy().astype(np.float32)


def collect(x: np.ndarray, bins: int) -> Hist:
    """collect_stats for one histogram."""
    x = np.asarray(x, np.float32).reshape(-1)
    rng = finite_range(x)
    if rng is None:
        raise ValueError("Input tensor cannot contain only infinite or only NaN values")
    edges = bin_edges(rng[0], rng[1], bins)
    h = histc(x, bins, edges[0], edges[-1])
    h[0] = F32(h[0] + F32(np.sum(x < edges[0])))
    h[-1] = F32(h[-1] + F32(np.sum(x > edges[-1])))
    return Hist(h, edges, rng[0], rng[1])


def _bin_num(width, cur_min, data: np.ndarray, bins: int) -> np.ndarray:
    """_get_bin_num: float32 -> int32 conversion (INT_MIN for NaN / out of range, as x86 does), clipped to bins - 1."""
    with np.errstate(divide="ignore", invalid="ignore"):
        idx = ((data - F32(cur_min)).astype(np.float32) / F32(width)).astype(np.float32)
    ok = (idx > -2147483648.0) & (idx < 2147483648.0)
    out = np.full(idx.shape, INT_MIN, dtype=np.int64)
    out[ok] = np.trunc(idx[ok]).astype(np.int64)
    return np.minimum(out, bins - 1)


def rebin(hist: np.ndarray, cmin, cmax, umin, umax, bins: int) -> np.ndarray:
    """The old counts moved to the bins of the wider range (merge_stats :229-249), additions in the reference's order."""
    cmin, cmax, umin, umax = F32(cmin), F32(cmax), F32(umin), F32(umax)
    dest_w = F32(F32(umax - umin) / F32(bins))
    src_w = F32(F32(cmax - cmin) / F32(bins))
    upd = np.zeros(bins, np.float32)
    src_start = (cmin + (src_w * np.arange(bins).astype(np.float32)).astype(np.float32)).astype(np.float32)
    dest = _bin_num(dest_w, umin, src_start, bins)
    dest_end = (umin + (dest_w * (dest + 1).astype(np.float32)).astype(np.float32)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        frac = ((dest_end - src_start).astype(np.float32) / src_w).astype(np.float32)
        split = np.rint((frac * hist).astype(np.float32)).astype(np.float32)
    dest_upd = np.where(np.isnan(split) | np.isnan(hist), np.float32(np.nan), np.minimum(split, hist)).astype(np.float32)
    for i in range(bins):
        if dest[i] >= 0:
            upd[dest[i]] = F32(upd[dest[i]] + dest_upd[i])
    other = _bin_num(dest_w, umin, (src_start + dest_w).astype(np.float32), bins)
    rest = (hist - dest_upd).astype(np.float32)
    for i in range(bins):
        if dest_upd[i] < hist[i] and other[i] >= 0:
            upd[other[i]] = F32(upd[other[i]] + rest[i])
    return upd


def merge(state: Optional[Hist], x: np.ndarray, bins: int) -> Hist:
    """update_stats of one batch: collect_stats + merge_stats."""
    new = collect(x, bins)
    if state is None:
        return new
    x = np.asarray(x, np.float32).reshape(-1)
    # Python min(new, cur) / max(new, cur): the second argument wins only when it is strictly smaller / larger
    umin = state.min if state.min < new.min else new.min
    umax = state.max if state.max > new.max else new.max
    if umin == state.min and umax == state.max:
        upd = state.hist
    else:
        upd = rebin(state.hist, state.min, state.max, umin, umax, bins)
    h = (histc(x, bins, umin, umax) + upd).astype(np.float32)
    h[0] = F32(h[0] + F32(np.sum(x == -np.inf)))
    h[-1] = F32(h[-1] + F32(np.sum(x == np.inf)))
    return Hist(h, bin_edges(umin, umax, bins), umin, umax)


# ---- the same work in the four steps of calibration spread over several workers ---------------------------------------
# A range record is 4 int32 words: min bits, max bits, "has a finite value", "present"; all zeros = no such batch.
# A plan is 8 floats: lo, hi (the range to count over), batch min, batch max, any_finite, first, present, 0.

def range_record(x: np.ndarray) -> np.ndarray:
    rng = finite_range(x)
    rec = np.zeros(4, np.int32)
    if rng is not None:
        rec[0:2] = np.array([rng[0], rng[1]], np.float32).view(np.int32)
        rec[2] = 1
    rec[3] = 1
    return rec


def plan_batches(ranges: np.ndarray, bins: int) -> np.ndarray:
    """ranges: [n_batches, 4] int32 -> plans [n_batches, 8] float32, walking the batches in order."""
    plans = np.zeros((ranges.shape[0], 8), np.float32)
    have, smin, smax = False, F32(0), F32(0)
    for b, rec in enumerate(ranges):
        mn, mx = rec[0:2].copy().view(np.float32)
        present, some = rec[3] != 0, rec[2] != 0
        lo, hi, first = F32(0), F32(1), False
        if present and some:
            if not have:
                e = bin_edges(mn, mx, bins)
                lo, hi = e[0], e[-1]
                smin, smax, have, first = mn, mx, True, True
            else:
                lo = smin if smin < mn else mn
                hi = smax if smax > mx else mx
                smin, smax = lo, hi
        plans[b] = [lo, hi, mn, mx, float(some), float(first), float(present), 0.0]
    return plans


def count(x: np.ndarray, bins: int, plan: np.ndarray) -> np.ndarray:
    """bins + 2 integer words: torch.histc over [lo, hi], elements below lo, elements above hi."""
    x = np.asarray(x, np.float32).reshape(-1)
    lo, hi = plan[0], plan[1]
    out = np.zeros(bins + 2, np.int32)
    out[:bins] = histc(x, bins, lo, hi).astype(np.int64)
    out[bins] = np.sum(x < lo)
    out[bins + 1] = np.sum(x > hi)
    return out


def replay(counts: np.ndarray, plans: np.ndarray, bins: int) -> Optional[Hist]:
    """collect_stats of the first batch and merge_stats of the later ones from their counts, in batch order."""
    state: Optional[Hist] = None
    for cn, pl in zip(counts, plans):
        if pl[6] == 0.0:
            continue
        if pl[4] == 0.0:
            raise ValueError("Input tensor cannot contain only infinite or only NaN values")
        c = cn[:bins].astype(np.float32)
        if pl[5] != 0.0:
            h = c.copy()
            h[0] = F32(h[0] + F32(cn[bins]))
            h[-1] = F32(h[-1] + F32(cn[bins + 1]))
            state = Hist(h, bin_edges(pl[2], pl[3], bins), pl[2], pl[3])
            continue
        umin, umax = F32(pl[0]), F32(pl[1])
        if umin == state.min and umax == state.max:
            upd = state.hist
        else:
            upd = rebin(state.hist, state.min, state.max, umin, umax, bins)
        h = (c + upd).astype(np.float32)
        h[0] = F32(h[0] + F32(cn[bins]))
        h[-1] = F32(h[-1] + F32(cn[bins + 1]))
        state = Hist(h, bin_edges(umin, umax, bins), umin, umax)
    return state


def sequential(batches: Sequence[np.ndarray], bins: int) -> List[Hist]:
    """The observer's statistics after every batch."""
    out, state = [], None
    for x in batches:
        state = merge(state, x, bins)
        out.append(state)
    return out
