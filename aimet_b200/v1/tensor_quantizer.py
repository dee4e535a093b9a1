"""Drop-in for the static-grid quantizer wrappers of AIMET's v1 quantsim
(``aimet_torch/v1/tensor_quantizer.py``): ``StaticGridPerTensorQuantizer`` / ``StaticGridPerChannelQuantizer``
(:403-570), their base-class surface (:60-395: ``encoding``, ``compute_encoding``, ``quantize_dequantize``,
``quantize``, ``reset_encoding_stats``, ``get_stats_histogram``, ``freeze_encoding``, ``set_percentile_value``) and the
autograd functions ``QuantizeDequantize`` / ``Quantize`` (:1098-1270) with the straight-through backward of
``compute_dloss_by_dx`` (``v1/quantsim_straight_through_grad.py:91-118``).

Same names, arguments and behaviour; the arithmetic runs on the B200 through :mod:`aimet_b200.libpymo` and
:mod:`aimet_b200.ops`.  Two things are done differently on purpose:

* per-channel calibration with the min/max scheme is ONE fused launch over the whole tensor (the reference makes one
  native call per channel on a copied slice, ``:567-570``); the per-channel encodings are the same numbers;
* the backward is one kernel that recomputes the mask from the saved input (the reference runs three tensor ops).

Only integer fake-quantization is on the accelerated path; ``float`` data types other than the trivial 16-bit cast
raise.
"""
from __future__ import annotations

import enum
from typing import List, Optional, Tuple, Union

import torch

from .. import libpymo, ops
from ..libpymo import AimetTensorQuantizer, TfEncoding


class QuantScheme(enum.Enum):
    """aimet_common.defs.QuantScheme (the members the static-grid quantizers accept)."""
    post_training_tf = 1
    post_training_tf_enhanced = 2
    post_training_percentile = 6


class QuantizationDataType(enum.Enum):
    """aimet_common.defs.QuantizationDataType"""
    undefined = 0
    int = 1
    float = 2


MAP_QUANT_SCHEME_TO_PYMO = {QuantScheme.post_training_tf: libpymo.QuantizationMode.QUANTIZATION_TF,
                            QuantScheme.post_training_tf_enhanced: libpymo.QuantizationMode.QUANTIZATION_TF_ENHANCED,
                            QuantScheme.post_training_percentile: libpymo.QuantizationMode.QUANTIZATION_PERCENTILE}


class StaticGridTensorQuantizer:
    """Common surface of the static-grid quantizers (reference ``TensorQuantizer`` + ``StaticGridTensorQuantizer``)."""

    def __init__(self, bitwidth: int, round_mode, quant_scheme: QuantScheme, use_symmetric_encodings: bool,
                 enabled_by_default: bool, data_type: QuantizationDataType = QuantizationDataType.int):
        self.round_mode = round_mode
        self._quant_scheme = quant_scheme
        self.use_symmetric_encodings = use_symmetric_encodings
        self.use_strict_symmetric = False
        self.use_unsigned_symmetric = True
        self.is_unsigned_symmetric = False
        self.bitwidth = bitwidth
        self.enabled = enabled_by_default
        self.data_type = data_type
        self._encoding: Optional[List[TfEncoding]] = None
        self._is_encoding_frozen = False
        self._encoding_min_max_fixed_vals: Optional[Tuple[float, float]] = None
        self._cppOp: List[AimetTensorQuantizer] = []

    # ---- properties ------------------------------------------------------------------------------------------
    @property
    def quant_scheme(self) -> QuantScheme:
        return self._quant_scheme

    @quant_scheme.setter
    def quant_scheme(self, quant_scheme: QuantScheme):
        self._quant_scheme = quant_scheme
        mode = MAP_QUANT_SCHEME_TO_PYMO[quant_scheme]
        self._cppOp = [AimetTensorQuantizer(mode) for _ in self._cppOp]

    @property
    def encoding_min_max_fixed_vals(self):
        return self._encoding_min_max_fixed_vals

    @encoding_min_max_fixed_vals.setter
    def encoding_min_max_fixed_vals(self, min_max_vals: Tuple[float, float]):
        assert isinstance(min_max_vals, tuple) and len(min_max_vals) == 2, "Min max vals must be a tuple of two values"
        assert min_max_vals[0] < min_max_vals[1], f"Min value {min_max_vals[0]} is not less than max val {min_max_vals[1]}"
        if self.quant_scheme != QuantScheme.post_training_tf:
            self.quant_scheme = QuantScheme.post_training_tf
        self._encoding_min_max_fixed_vals = min_max_vals

    @property
    def is_encoding_frozen(self) -> bool:
        return self._is_encoding_frozen

    # ---- encodings -------------------------------------------------------------------------------------------
    def _channel_encodings(self) -> List[Tuple[TfEncoding, bool]]:
        return [op.getEncoding(self.bitwidth, self.use_symmetric_encodings, self.use_strict_symmetric,
                               self.use_unsigned_symmetric) for op in self._cppOp]

    def compute_encoding(self):
        """Reference ``compute_encoding`` (:280-321); skipped for 32-bit and 16-bit float."""
        if not (self.enabled and not self._is_encoding_frozen):
            return
        self._encoding = []
        if self.bitwidth == 32:
            self._encoding = None
            return
        if self.data_type == QuantizationDataType.float:
            if self.bitwidth == 16:
                self._encoding = None
                return
            raise ValueError("aimet_b200: 8-bit float fake-quantization is outside the accelerated path")
        for encoding, valid in self._channel_encodings():
            if not valid:
                self.enabled = False
            else:
                self._encoding.append(encoding)
        self.is_unsigned_symmetric = bool(self.use_symmetric_encodings and self.use_unsigned_symmetric and
                                          all(e.min >= 0 and e.max >= 0 for e in self._encoding))
        assert not (not self.enabled and self._encoding), \
            "At least one encoding for a multi-encoding quantizer is invalid."

    def reset_encoding_stats(self):
        if not self._is_encoding_frozen:
            for op in self._cppOp:
                op.resetEncodingStats()
            self._encoding = None

    def get_stats_histogram(self) -> List[List]:
        if self._quant_scheme != QuantScheme.post_training_tf_enhanced:
            raise RuntimeError("get_stats_histogram() can be invoked only when quantization scheme is TF-Enhanced.")
        if not self._encoding:
            raise RuntimeError("get_stats_histogram() can be invoked only when encoding is computed.")
        return [op.getStatsHistogram() for op in self._cppOp]

    def freeze_encoding(self) -> None:
        if not self._encoding:
            raise RuntimeError("Encoding can be frozen only when it is not None.")
        self._is_encoding_frozen = True

    def set_percentile_value(self, percentile_value: float):
        for op in self._cppOp:
            op.setPercentileValue(percentile_value)

    # ---- fake-quant ------------------------------------------------------------------------------------------
    def quantize_dequantize(self, tensor: torch.Tensor, round_mode) -> torch.Tensor:
        return QuantizeDequantize.apply(tensor, self, round_mode)

    def quantize(self, tensor: torch.Tensor, round_mode) -> torch.Tensor:
        return Quantize.apply(tensor, self, round_mode)


class StaticGridPerTensorQuantizer(StaticGridTensorQuantizer):
    """Per-tensor scale / offset (reference :403-470)."""

    def __init__(self, bitwidth: int, round_mode, quant_scheme: QuantScheme, use_symmetric_encodings: bool,
                 enabled_by_default: bool, data_type: QuantizationDataType = QuantizationDataType.int):
        super().__init__(bitwidth, round_mode, quant_scheme, use_symmetric_encodings, enabled_by_default, data_type)
        self._cppOp = [AimetTensorQuantizer(MAP_QUANT_SCHEME_TO_PYMO[quant_scheme])]

    @property
    def encoding(self) -> Optional[TfEncoding]:
        return self._encoding[0] if self._encoding else None

    @encoding.setter
    def encoding(self, encoding: Union[TfEncoding, List[TfEncoding]]):
        if self._is_encoding_frozen:
            raise RuntimeError("Encoding can be set only when it is not frozen.")
        self._encoding = encoding if isinstance(encoding, list) and len(encoding) == 1 else [encoding]

    def update_encoding_stats(self, tensor: torch.Tensor):
        if not (self.enabled and not self._is_encoding_frozen) or self.bitwidth == 32:
            return
        if self.data_type == QuantizationDataType.float:
            return
        if self.encoding_min_max_fixed_vals is not None:
            tensor = torch.tensor(list(self.encoding_min_max_fixed_vals), dtype=torch.float32, device=tensor.device)
        if tensor.dtype != torch.float32:
            tensor = tensor.to(torch.float32)
        for op in self._cppOp:
            op.updateStats(tensor, tensor.is_cuda)


class _ChannelMinMaxOp:
    """Stands where the reference keeps one native min/max analyzer per channel: a view of one row of a shared,
    device-resident [2, C] running min/max table that a single fused launch updates for all channels."""

    def __init__(self, owner: "StaticGridPerChannelQuantizer", index: int):
        self._owner, self._index = owner, index

    def getEncoding(self, bitwidth, symmetric, strict, unsigned_sym):
        mm = self._owner._host_minmax()
        if mm is None:
            return TfEncoding(), False
        mn, mx = mm[0][self._index], mm[1][self._index]
        return TfEncoding._from_c(ops.minmax_encoding(int(bitwidth), mn, mx, symmetric, strict, unsigned_sym)), True

    def resetEncodingStats(self):
        self._owner._reset_minmax()

    def getStatsHistogram(self):
        raise RuntimeError("aimet_b200: the TF (min/max) analyzer keeps no histogram")

    def setPercentileValue(self, percentile):
        return None


class StaticGridPerChannelQuantizer(StaticGridTensorQuantizer):
    """Per-channel scale / offset along ``ch_axis`` (reference :473-570)."""

    def __init__(self, bitwidth: int, round_mode, quant_scheme: QuantScheme, use_symmetric_encodings: bool,
                 num_channels: int, enabled_by_default: bool, ch_axis: int = 0,
                 data_type: QuantizationDataType = QuantizationDataType.int):
        super().__init__(bitwidth, round_mode, quant_scheme, use_symmetric_encodings, enabled_by_default, data_type)
        self._num_channels = int(num_channels)
        self._ch_axis = ch_axis
        self._mm_dev: Optional[torch.Tensor] = None     # running [2, C] min / max on the device (min/max scheme)
        self._mm_host = None
        self._build_ops()

    def _build_ops(self):
        if self._quant_scheme == QuantScheme.post_training_tf:
            self._cppOp = [_ChannelMinMaxOp(self, c) for c in range(self._num_channels)]
        else:
            mode = MAP_QUANT_SCHEME_TO_PYMO[self._quant_scheme]
            self._cppOp = [AimetTensorQuantizer(mode) for _ in range(self._num_channels)]

    @StaticGridTensorQuantizer.quant_scheme.setter
    def quant_scheme(self, quant_scheme: QuantScheme):
        self._quant_scheme = quant_scheme
        self._reset_minmax()
        self._build_ops()

    def _reset_minmax(self):
        self._mm_dev, self._mm_host = None, None

    def _host_minmax(self):
        if self._mm_dev is None:
            return None
        if self._mm_host is None:
            self._mm_host = self._mm_dev.tolist()   # one read-back for all channels
        return self._mm_host

    @property
    def encoding(self) -> Optional[List[TfEncoding]]:
        return self._encoding

    @encoding.setter
    def encoding(self, encoding: List[TfEncoding]):
        if self._is_encoding_frozen:
            raise RuntimeError("Encoding can be set only when it is not frozen.")
        self._encoding = encoding

    @property
    def channel_axis(self) -> int:
        return self._ch_axis

    def update_encoding_stats(self, tensor: torch.Tensor):
        if not (self.enabled and not self._is_encoding_frozen) or self.bitwidth == 32:
            return
        if self.data_type == QuantizationDataType.float:
            return
        if tensor.dtype != torch.float32:
            tensor = tensor.to(torch.float32)
        fixed = self.encoding_min_max_fixed_vals
        if self._quant_scheme == QuantScheme.post_training_tf:
            if fixed is not None:
                tensor = torch.tensor(list(fixed), dtype=torch.float32, device=tensor.device).repeat(self._num_channels, 1)
                axis = 0
            else:
                axis = self._ch_axis % tensor.dim()
            if not tensor.is_cuda:
                raise RuntimeError("aimet_b200: statistics need a CUDA tensor; there is no CPU path")
            x = tensor.contiguous()
            inner = 1
            for d in x.shape[axis + 1:]:
                inner *= d
            if x.shape[axis] != self._num_channels:
                raise RuntimeError("aimet_b200: the tensor's channel dimension does not match num_channels")
            first = self._mm_dev is None
            if first:
                self._mm_dev = torch.empty((2, self._num_channels), dtype=torch.float32, device=x.device)
            # all channels in one fused pass; later batches fold into the running table
            ops.minmax(x, self._num_channels, inner, propagate_nan=False, out=self._mm_dev, accumulate=not first)
            self._mm_host = None
            return
        if fixed is not None:
            t = torch.tensor(list(fixed), dtype=torch.float32, device=tensor.device)
            for op in self._cppOp:
                op.updateStats(t, t.is_cuda)
            return
        for channel_idx, op in enumerate(self._cppOp):
            op.updateStats(tensor.select(self._ch_axis, channel_idx).contiguous(), tensor.is_cuda)


def _encoding_bounds(tq: StaticGridTensorQuantizer, device) -> Tuple[torch.Tensor, torch.Tensor]:
    encs = tq._encoding
    mm = torch.tensor([[e.min for e in encs], [e.max for e in encs]], dtype=torch.float32)
    mm = mm.to(device, non_blocking=True)
    return mm[0], mm[1]


def _geometry(tq: StaticGridTensorQuantizer, tensor: torch.Tensor) -> Tuple[int, int]:
    if isinstance(tq, StaticGridPerChannelQuantizer):
        sizes = [*tensor.shape, 1]
        axis = tq.channel_axis % tensor.dim()
        inner = 1
        for d in sizes[axis + 1:]:
            inner *= d
        return sizes[axis], inner
    return 1, max(tensor.numel(), 1)


class QuantizeDequantize(torch.autograd.Function):
    """Fake-quantization with the saved encoding(s); straight-through backward (reference :1098-1212)."""

    @staticmethod
    def forward(ctx, tensor: torch.Tensor, tensor_quantizer: StaticGridTensorQuantizer, round_mode):
        tq = tensor_quantizer
        ctx.tensor_quantizer = tq
        ctx.active = bool(tq.enabled and tq.bitwidth != 32)
        if not ctx.active:
            return tensor
        if tq.data_type == QuantizationDataType.float:
            if tq.bitwidth != 16:
                raise ValueError("aimet_b200: float data_type supports only the 16-bit cast on this path")
            ctx.save_for_backward(tensor)
            if tensor.dtype == torch.float32 and tensor.is_cuda:
                return ops.qdq_fp16(tensor)   # one pass instead of two casts
            return tensor.half().float()
        dtype = tensor.dtype
        x = tensor.to(torch.float32)
        if isinstance(tq, StaticGridPerChannelQuantizer):
            num_ch, inner = _geometry(tq, x)
            y = libpymo.quantize_dequantize_per_channel(x, tq._encoding, num_ch, x.numel(), inner, round_mode, x.is_cuda)
        else:
            y = tq._cppOp[0].quantizeDequantize(x, tq.encoding, round_mode, x.is_cuda)
        ctx.save_for_backward(tensor)   # the input is what the backward's mask is computed from
        return y.to(dtype)

    @staticmethod
    def backward(ctx, output_grad):
        tq = ctx.tensor_quantizer
        if not (ctx.active and tq.data_type == QuantizationDataType.int):
            return output_grad, None, None
        (tensor,) = ctx.saved_tensors
        x = tensor.to(torch.float32).contiguous()
        g = output_grad.to(torch.float32).contiguous()
        mn, mx = _encoding_bounds(tq, x.device)
        num_ch, inner = _geometry(tq, x)
        dx = ops.ste_backward_v1(x, g, mn, mx, num_ch, inner)
        return dx.to(output_grad.dtype), None, None


class Quantize(torch.autograd.Function):
    """Integer codes with the saved encoding(s) (reference :1215-1290); the gradient passes straight through.  Codes
    are signed unless the quantizer is symmetric with the unsigned-symmetric option, as in the reference."""

    @staticmethod
    def forward(ctx, tensor: torch.Tensor, tensor_quantizer: StaticGridTensorQuantizer, round_mode):
        tq = tensor_quantizer
        assert tq.enabled, "Tensor quantizer must be enabled to perform quantize only."
        assert tq.data_type == QuantizationDataType.int, \
            "Tensor quantizer must be performing integer quantization to perform quantize only."
        assert tq.bitwidth != 32, "Tensor quantizer bitwidth must be < 32 to perform quantize only."
        assert tq.encoding is not None, "Tensor quantizer encoding must be valid to perform quantize only."
        shift_to_signed = not (tq.use_symmetric_encodings and tq.use_unsigned_symmetric)
        x = tensor.to(torch.float32)
        if isinstance(tq, StaticGridPerChannelQuantizer):
            parts = []
            for index, enc in enumerate(tq._encoding):
                part = x.select(tq.channel_axis, index).contiguous()
                parts.append(ops.quantize_per_tensor(part, enc.min, enc.max, enc.bw, shift_to_signed, int(round_mode)))
            return torch.stack(tuple(parts), dim=tq.channel_axis).to(tensor.dtype)
        enc = tq.encoding
        return ops.quantize_per_tensor(libpymo._dense(x), enc.min, enc.max, enc.bw, shift_to_signed,
                                       int(round_mode)).to(tensor.dtype)

    @staticmethod
    def backward(ctx, output_grad):
        return output_grad, None, None
