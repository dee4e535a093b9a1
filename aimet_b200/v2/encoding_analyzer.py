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


class StatisticsNotFoundError(RuntimeError):
    """No statistics were collected before encodings were requested (aimet_torch/v2/utils.py)."""


@dataclass
class _MinMaxRange:
    min: Optional[torch.Tensor] = None
    max: Optional[torch.Tensor] = None


class _MinMaxObserver:
    """Running min / max per encoding (reference: _MinMaxObserver, encoding_analyzer.py:92-128)."""

    def __init__(self, shape):
        if isinstance(shape, int):
            shape = (shape,)
        self.shape = tuple(shape)
        self.stats = _MinMaxRange()

    @torch.no_grad()
    def collect_stats(self, input_tensor: torch.Tensor) -> _MinMaxRange:
        if not input_tensor.is_cuda:
            raise RuntimeError("aimet_b200: statistics are collected on the GPU only (no CPU path exists)")
        x = input_tensor.detach()
        if x.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise RuntimeError(f"aimet_b200: unsupported dtype {x.dtype}")
        enc_shape = self.shape
        if len(enc_shape) > x.dim() or any(s not in (1, t) for s, t in zip(enc_shape[::-1], tuple(x.shape)[::-1])):
            raise RuntimeError(f"Shape {self.shape} is incompatible with input of shape {tuple(x.shape)}")
        g = resolve_geometry(x, enc_shape, None)
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
        mn, mx = self.stats.min, self.stats.max
        if stats.min is not None:
            mn = stats.min.clone() if mn is None else torch.minimum(mn, stats.min)
        if stats.max is not None:
            mx = stats.max.clone() if mx is None else torch.maximum(mx, stats.max)
        self.stats = _MinMaxRange(mn, mx)

    def reset_stats(self):
        self.stats = _MinMaxRange()

    def get_stats(self) -> _MinMaxRange:
        return self.stats


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
            return torch.tensor(float(v), dtype=torch.float32, device=stats.min.device)

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
