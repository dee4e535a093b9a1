"""Affine quantizer modules on the B200 kernels: ``Quantize`` and ``QuantizeDequantize``.

Same constructor signatures, parameters (``min`` / ``max``), calibration context and accessor methods as
aimet_torch/v2/quantization/affine/quantizer.py:66-697 (AffineQuantizerBase, MinMaxQuantizer, Quantize,
QuantizeDequantize) and aimet_torch/v2/quantization/base/quantizer.py:59-219 (initialisation tracking, overwrite
flag); ``AffineEncoding`` carries what aimet_torch/v2/quantization/affine/encoding.py:54-280 exposes as properties.
The forward passes go through :mod:`aimet_b200.v2.backend` (one fused kernel each way); statistics go through the
analyzers of :mod:`aimet_b200.v2.encoding_analyzer`.

Host-side differences, on purpose:

* scale and offset are cached between forward passes while ``min`` / ``max`` are unchanged and no gradient is
  being recorded (the reference recomputes them with five small tensor operations per call);
* ``plain_outputs = True`` on a quantizer makes it return plain tensors instead of the tensor subclasses that carry
  the encoding (:mod:`aimet_b200.v2.qtensor`);
* ``scale = (max - min) / num_steps`` divides by a tensor, so that the CUDA result equals the reference's CPU
  result bit for bit (a CUDA tensor divided by a Python number is multiplied by its reciprocal instead).
"""
from __future__ import annotations

import contextlib
import math
from typing import List, Optional, Sequence, Tuple

import torch
from torch import nn

from . import backend
from .encoding_analyzer import EncodingAnalyzer, MinMaxEncodingAnalyzer, StatisticsNotFoundError, device_scalar
from .qtensor import DequantizedTensor, QuantizedTensor

__all__ = ["AffineEncoding", "MinMaxQuantizer", "Quantize", "QuantizeDequantize", "GroupedBlockQuantizeDequantize"]


def derive_qmin_qmax(bitwidth: int, signed: bool) -> Tuple[int, int]:
    """Integer grid of a bit-width (backends/__init__.py:359-370): signed grids are [-ceil(n/2), floor(n/2)]."""
    steps = 2 ** bitwidth - 1
    if signed:
        return -math.ceil(steps / 2), math.floor(steps / 2)
    return 0, steps


def _grid_bitwidth(qmin: int, qmax: int, owner: str) -> int:
    """Bit-width of a grid of the form [0, 2^B - 1] or [-2^(B-1), 2^(B-1) - 1]; undefined (RuntimeError) for any
    other grid (affine/_utils.py:88-113)."""
    if qmin + qmax == -1 or qmin == 0:
        bits = math.log2(qmax - qmin + 1)
        if bits == int(bits):
            return int(bits)
    raise RuntimeError(f"{owner}.bitwidth is undefined in the quantization grid [{qmin}, {qmax}].")


def _grid_signed(qmin: int, qmax: int, owner: str) -> bool:
    """Signedness under the same condition (affine/_utils.py:146-167)."""
    if qmin + qmax == -1 or qmin == 0:
        return qmin < 0 <= qmax
    raise RuntimeError(f"{owner}.signed is undefined in the quantization grid [{qmin}, {qmax}].")


class _RoundSte(torch.autograd.Function):
    """torch.round with an identity gradient (aimet_torch/v2/utils.py:195-199)."""

    @staticmethod
    def forward(ctx, x):
        return torch.round(x)

    @staticmethod
    def backward(ctx, g):
        return g


class AffineEncoding:
    """Scale / offset / integer grid of one quantizer (affine/encoding.py:54-280)."""

    def __init__(self, scale: torch.Tensor, offset: torch.Tensor, *args, **kwargs):
        """``AffineEncoding(scale, offset, qmin, qmax, symmetry=False, block_size=None)`` or
        ``AffineEncoding(scale, offset, bitwidth, signed=False, symmetry=False, block_size=None)``: the second form is
        recognised by a boolean (or missing) fourth argument, as in the reference (encoding.py:60-110)."""
        pos = list(args) + [None] * (4 - len(args))
        first = kwargs.pop("qmin", kwargs.pop("bitwidth", pos[0]))
        second = kwargs.pop("qmax", kwargs.pop("signed", pos[1]))
        symmetry = kwargs.pop("symmetry", pos[2])
        block_size = kwargs.pop("block_size", pos[3])
        if kwargs:
            raise TypeError(f"AffineEncoding.__init__ got unexpected keyword argument: {', '.join(kwargs.keys())}")
        if second is None or isinstance(second, bool):
            if first is None:
                raise TypeError("AffineEncoding: expected (scale, offset, qmin, qmax, ...) or (scale, offset, bitwidth, "
                                "signed, ...)")
            qmin, qmax = derive_qmin_qmax(int(first), signed=bool(second))
        else:
            if first is None:
                raise TypeError("AffineEncoding: qmin is missing")
            qmin, qmax = first, second
        if qmin >= qmax:
            raise ValueError(f"qmax should be strictly larger than qmin. Got qmax={qmax}, qmin={qmin}")
        self.scale, self.offset, self.qmin, self.qmax = scale, offset, int(qmin), int(qmax)
        self.symmetry, self.block_size = bool(symmetry) if symmetry is not None else False, block_size

    mapping = "affine"

    @property
    def granularity(self) -> str:
        if self.scale.dim() == 0:
            return "pertensor"
        if self.block_size is not None:
            return "blockwise"
        return "perchannel" if sum(d > 1 for d in self.scale.shape) == 1 else "unknown"

    @property
    def num_steps(self) -> int:
        return self.qmax - self.qmin

    @property
    def bitwidth(self) -> int:
        return _grid_bitwidth(self.qmin, self.qmax, "AffineEncoding")

    @property
    def signed(self) -> bool:
        return _grid_signed(self.qmin, self.qmax, "AffineEncoding")

    @property
    def min(self) -> torch.Tensor:
        return (self.offset + self.qmin) * self.scale

    @property
    def max(self) -> torch.Tensor:
        return (self.offset + self.qmax) * self.scale

    @property
    def dtype(self) -> torch.dtype:
        """Smallest integer type that holds the grid (encoding.py:201-215)."""
        if 0 <= self.qmin < self.qmax < 256:
            return torch.uint8
        if -128 <= self.qmin < self.qmax < 128:
            return torch.int8
        if -32768 <= self.qmin < self.qmax < 32768:
            return torch.int16
        return torch.int32

    def to(self, *args, **kwargs) -> "AffineEncoding":
        """Moves / casts scale and offset like ``Tensor.to``; only floating-point types (encoding.py:224-243)."""
        device, dtype, _, _ = torch._C._nn._parse_to(*args, **kwargs)   # pylint: disable=protected-access
        dtype = dtype or self.scale.dtype
        device = device or self.scale.device
        if dtype is self.scale.dtype and device == self.scale.device:
            return self
        if not dtype.is_floating_point:
            raise RuntimeError(f"Cannot change encoding data dtype to {dtype}, "
                               "only floating point data types are supported")
        return AffineEncoding(self.scale.to(dtype=dtype, device=device), self.offset.to(dtype=dtype, device=device),
                              self.qmin, self.qmax, self.symmetry, self.block_size)

    def _clone(self) -> "AffineEncoding":
        return AffineEncoding(self.scale.clone(), self.offset.clone(), self.qmin, self.qmax, self.symmetry,
                              self.block_size)

    def _detach(self) -> "AffineEncoding":
        return AffineEncoding(self.scale.detach(), self.offset.detach(), self.qmin, self.qmax, self.symmetry,
                              self.block_size)

    def quantize(self, x: torch.Tensor) -> torch.Tensor:
        x = x.as_subclass(torch.Tensor)
        return backend.quantize(x, self.scale.to(x.dtype).as_subclass(torch.Tensor),
                                self.offset.to(x.dtype).as_subclass(torch.Tensor), self.qmin, self.qmax,
                                self.block_size)

    def dequantize(self, x: torch.Tensor) -> torch.Tensor:
        x = x.as_subclass(torch.Tensor)
        return backend.dequantize(x, self.scale.to(x.dtype).as_subclass(torch.Tensor),
                                  self.offset.to(x.dtype).as_subclass(torch.Tensor), self.block_size)

    def _to_legacy_format(self) -> List[dict]:
        """One dict per channel / block, in flat order, as the exported encodings files hold them
        (encoding.py:267-280): the offset is shifted by qmin, i.e. it is the code of the real value 0 relative to
        an unsigned grid, and ``is_symmetric`` is the STRING "True" / "False"."""
        rows = torch.stack([self.min.flatten().double(), self.max.flatten().double(), self.scale.flatten().double(),
                            (self.offset.flatten() + self.qmin).double()]).cpu().tolist()
        return [{"min": float(mn), "max": float(mx), "scale": float(sc), "offset": int(of), "bitwidth": self.bitwidth,
                 "dtype": "int", "is_symmetric": str(self.symmetry)} for mn, mx, sc, of in zip(*rows)]


def _encoding_shape_with_blocks(shape: Sequence[int], block_size: Optional[Sequence[int]]) -> Tuple[int, ...]:
    """Shape of the statistics when blocks are split out: [d0, 1, d1, 1, ...] (torch_builtins.py:387-403)."""
    if block_size is None:
        return tuple(shape)
    out: List[int] = []
    for d in shape:
        out += [d, 1]
    return tuple(out)


def _reshape_for_blocks(x: torch.Tensor, enc_shape: Sequence[int], block_size: Optional[Sequence[int]]) -> torch.Tensor:
    """View [.., d_k, ..] as [.., d_k / B_k, B_k, ..] for the trailing len(block_size) dimensions
    (torch_builtins.py:366-403); -1 stands for "one block spans the whole dimension share"."""
    if block_size is None:
        return x
    view: List[int] = []
    for i in range(1, len(block_size) + 1):
        blocks = enc_shape[-i]
        width = x.shape[-i] // blocks if block_size[-i] == -1 else block_size[-i]
        view = [blocks, width] + view
    return x.view(list(x.shape[:-len(block_size)]) + view)


class MinMaxQuantizer(nn.Module):
    """Affine quantizer whose trainable parameters are ``min`` and ``max`` (affine/quantizer.py:66-437).

    ``MinMaxQuantizer(shape, bitwidth, symmetric, encoding_analyzer=None, block_size=None)`` or
    ``MinMaxQuantizer(shape, qmin, qmax, symmetric, encoding_analyzer=None, block_size=None)``.
    """

    def __init__(self, shape, *args, **kwargs):
        super().__init__()
        self.shape = (shape,) if isinstance(shape, int) else tuple(shape)
        pos = list(args) + [None] * (5 - len(args))
        first = kwargs.pop("qmin", kwargs.pop("bitwidth", pos[0]))
        second = kwargs.pop("qmax", pos[1])
        if second is not None and not isinstance(second, bool):
            qmin, qmax = first, second
            symmetric = kwargs.pop("symmetric", pos[2])
            analyzer, block_size = kwargs.pop("encoding_analyzer", pos[3]), kwargs.pop("block_size", pos[4])
            if qmin is None or qmax is None or symmetric is None:
                raise TypeError(f"{type(self).__qualname__}: expected (shape, qmin, qmax, symmetric, ...)")
        else:
            symmetric = kwargs.pop("symmetric", pos[1])
            if first is None or symmetric is None:
                raise TypeError(f"{type(self).__qualname__}: expected (shape, bitwidth, symmetric, ...)")
            qmin, qmax = derive_qmin_qmax(first, signed=symmetric)
            analyzer, block_size = kwargs.pop("encoding_analyzer", pos[2]), kwargs.pop("block_size", pos[3])
        if kwargs:
            raise TypeError(f"{type(self).__qualname__}.__init__ got unexpected keyword argument: "
                            f"{', '.join(kwargs.keys())}")
        if qmin >= qmax:
            raise ValueError(f"qmax should be strictly larger than qmin. Got qmax={qmax}, qmin={qmin}")
        self.qmin, self.qmax, self._symmetric = int(qmin), int(qmax), bool(symmetric)
        self.block_size = tuple(block_size) if block_size is not None else None
        self.encoding_analyzer: EncodingAnalyzer = analyzer or MinMaxEncodingAnalyzer(
            _encoding_shape_with_blocks(self.shape, self.block_size))
        if self.block_size is None and not backend._is_expandable(self.encoding_analyzer.observer.shape, self.shape):
            raise RuntimeError(f"Encoding analyzer of shape {self.encoding_analyzer.observer.shape} "
                               f"is incompatible with quantizer of shape {self.shape}.")
        self._allow_overwrite = True
        self.plain_outputs = False
        self._calibrating = False
        self._cache = None
        self.min = nn.Parameter(-torch.ones(self.shape))
        self.max = nn.Parameter(torch.ones(self.shape))
        # a parameter counts as initialised once it has been written after construction (base/quantizer.py:109-135)
        self._initial_versions = {"min": (self.min, self.min._version), "max": (self.max, self.max._version)}

    # ---- bookkeeping -------------------------------------------------------------------------------------------
    @property
    def symmetric(self) -> bool:
        return self._symmetric

    @symmetric.setter
    def symmetric(self, value: bool):
        self._symmetric = bool(value)
        self._cache = None

    @property
    def bitwidth(self) -> int:
        return _grid_bitwidth(self.qmin, self.qmax, type(self).__qualname__)

    @bitwidth.setter
    def bitwidth(self, bitwidth: int):
        self.qmin, self.qmax = derive_qmin_qmax(bitwidth, signed=self.signed)
        self._cache = None

    @property
    def signed(self) -> bool:
        return _grid_signed(self.qmin, self.qmax, type(self).__qualname__)

    def allow_overwrite(self, mode: bool):
        self._allow_overwrite = bool(mode)

    def is_initialized(self) -> bool:
        for name, (tensor, version) in self._initial_versions.items():
            current = getattr(self, name)
            if current is tensor and current._version == version:
                return False
        return True

    def get_extra_state(self):
        return {name: torch.tensor(self.is_initialized()) for name in ("min", "max")}

    @torch.no_grad()
    def set_extra_state(self, state):
        for name in ("min", "max"):
            p = getattr(self, name)
            self._initial_versions[name] = (p, p._version)
            if name in state and bool(state[name]):
                p.mul_(1.0)   # bumps the version: marks the loaded value as initialised
        self._cache = None

    @torch.no_grad()
    def __deepcopy__(self, memo):
        # a copied parameter starts a new version count: carry the "has been written" facts over explicitly
        import copy
        new = self.__new__(type(self))
        memo[id(self)] = new
        new.__dict__ = copy.deepcopy(self.__dict__, memo)
        new.set_extra_state(self.get_extra_state())
        return new

    # ---- encodings ---------------------------------------------------------------------------------------------
    def _scale_offset(self, dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        recording = torch.is_grad_enabled() and (self.min.requires_grad or self.max.requires_grad)
        key = (self.min, self.min._version, self.max, self.max._version, dtype, self._symmetric, self.qmin, self.qmax)
        if not recording and self._cache is not None and all(a is b if isinstance(a, torch.Tensor) else a == b
                                                             for a, b in zip(self._cache[0], key)):
            return self._cache[1], self._cache[2]
        steps = device_scalar(self.qmax - self.qmin, dtype, self.min.device)
        scale = self._transform_scale(((self.max.to(dtype) - self.min.to(dtype)) / steps).to(dtype))
        if self._symmetric:
            offset = torch.zeros_like(self.min, requires_grad=False, dtype=dtype)
        else:
            offset = (_RoundSte.apply(self.min.to(dtype) / scale) - self.qmin).to(dtype)
        if not recording:
            self._cache = (key, scale.detach(), offset.detach())
        return scale, offset

    def _transform_scale(self, scale: torch.Tensor) -> torch.Tensor:
        """Hook for quantizers whose effective scale is derived from the min/max scale (grouped blocks)."""
        return scale

    def get_scale(self, dtype=None) -> Optional[torch.Tensor]:
        if not self.is_initialized():
            return None
        return self._scale_offset(dtype or torch.float32)[0]

    def get_offset(self, dtype=None) -> Optional[torch.Tensor]:
        if not self.is_initialized():
            return None
        return self._scale_offset(dtype or torch.float32)[1]

    def get_min(self, dtype=None) -> Optional[torch.Tensor]:
        if not self.is_initialized():
            return None
        scale, offset = self._scale_offset(dtype or torch.float32)
        return scale * (offset + self.qmin)

    def get_max(self, dtype=None) -> Optional[torch.Tensor]:
        if not self.is_initialized():
            return None
        scale, offset = self._scale_offset(dtype or torch.float32)
        return scale * (offset + self.qmax)

    def get_encoding(self) -> Optional[AffineEncoding]:
        if not self.is_initialized():
            return None
        scale, offset = self._scale_offset(torch.float32)
        return AffineEncoding(scale, offset, self.qmin, self.qmax, self._symmetric, self.block_size)

    @torch.no_grad()
    def get_legacy_encodings(self) -> Optional[List[dict]]:
        """The encodings as the list of dicts the exported files hold (affine/quantizer.py:222-232)."""
        if not self.is_initialized():
            return None
        return self.get_encoding()._to_legacy_format()   # pylint: disable=protected-access

    @torch.no_grad()
    def set_legacy_encodings(self, encodings: List[dict]):
        """Inverse of :meth:`get_legacy_encodings` (affine/quantizer.py:234-263): bit-width and symmetry come from
        the first entry (symmetric means a signed grid, anything else an unsigned one), the range from every entry's
        ``min`` / ``max``; scale and offset are re-derived from the range."""
        flag = str(encodings[0]["is_symmetric"]).lower()
        if flag not in ("true", "false"):
            raise ValueError(f"is_symmetric must be 'True' or 'False', got {encodings[0]['is_symmetric']!r}")
        symmetric = flag == "true"
        self.qmin, self.qmax = derive_qmin_qmax(int(encodings[0]["bitwidth"]), signed=symmetric)
        self.symmetric = symmetric
        self.set_range(torch.tensor([e["min"] for e in encodings]).view(self.shape),
                       torch.tensor([e["max"] for e in encodings]).view(self.shape))

    @torch.no_grad()
    def set_range(self, min: torch.Tensor, max: torch.Tensor):   # pylint: disable=redefined-builtin
        self.min.copy_(min)
        self.max.copy_(max)
        self._cache = None

    # ---- calibration -------------------------------------------------------------------------------------------
    @contextlib.contextmanager
    def compute_encodings(self):
        """Observes the inputs seen inside the context and sets ``min`` / ``max`` from their statistics on exit;
        inside the context every forward pass quantizes with the statistics of its own batch
        (affine/quantizer.py:317-374)."""
        if not self._allow_overwrite:
            yield
            return
        self.encoding_analyzer.reset_stats()
        self._calibrating = True
        try:
            yield
        finally:
            self._calibrating = False
        steps = self.qmax - self.qmin
        try:
            enc_min, enc_max = self.encoding_analyzer.compute_encodings(steps, self._symmetric)
        except StatisticsNotFoundError:
            return
        if enc_min is None or enc_max is None:
            return
        self.set_range(enc_min.view(self.min.shape) if self.block_size is not None else enc_min,
                       enc_max.view(self.max.shape) if self.block_size is not None else enc_max)

    def _dynamic_scale_offset(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        fused = getattr(self.encoding_analyzer, "fused_update", None)
        if (fused is not None and type(self)._transform_scale is MinMaxQuantizer._transform_scale
                and math.prod(self.encoding_analyzer.observer.shape) == math.prod(self.shape)):
            got = fused(_reshape_for_blocks(x, self.shape, self.block_size), self.qmax - self.qmin, self._symmetric,
                        self.qmin)
            if got is not None:
                return got[0].view(self.min.shape), got[1].view(self.min.shape)
        stats = self.encoding_analyzer.update_stats(_reshape_for_blocks(x, self.shape, self.block_size))
        steps = self.qmax - self.qmin
        dmin, dmax = self.encoding_analyzer.compute_encodings_from_stats(stats, steps, self._symmetric)
        if self.block_size is not None:
            dmin, dmax = dmin.view(self.min.shape), dmax.view(self.max.shape)
        dmin = dmin.to(dtype=self.min.dtype, device=self.min.device).expand_as(self.min)
        dmax = dmax.to(dtype=self.max.dtype, device=self.max.device).expand_as(self.max)
        div = device_scalar(steps, torch.float32, dmin.device)
        scale = self._transform_scale((dmax.to(torch.float32) - dmin.to(torch.float32)) / div)
        offset = torch.zeros_like(scale) if self._symmetric else torch.round(dmin.to(torch.float32) / scale) - self.qmin
        return scale, offset

    def _observe_only(self, x: torch.Tensor) -> bool:
        """True when the calibration context is open and the analyzer only wants to see the input."""
        if self._calibrating and getattr(self.encoding_analyzer, "calibration_passthrough", False):
            self.encoding_analyzer.update_stats(_reshape_for_blocks(x, self.shape, self.block_size))
            return True
        return False

    def _wrap(self, out: torch.Tensor, cls, scale: torch.Tensor, offset: torch.Tensor) -> torch.Tensor:
        """Outputs carry their encoding as the reference's do (affine/quantizer.py:549-563, 683-697) unless
        ``plain_outputs`` is set: every later operation on such a tensor passes through a Python-level dispatch,
        which a model wrapper that never looks at the encoding does not need to pay for."""
        if self.plain_outputs:
            return out
        out = out.as_subclass(cls)
        out.encoding = AffineEncoding(scale, offset, self.qmin, self.qmax, self._symmetric, self.block_size)
        return out

    def _encoding_for(self, x: torch.Tensor, what: str) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._calibrating:
            return self._dynamic_scale_offset(x)
        if not self.is_initialized():
            raise RuntimeError(f"Failed to run {what} since quantization parameters are not initialized."
                               " Please initialize the quantization parameters using `compute_encodings()`.")
        return self._scale_offset(torch.float32)


class Quantize(MinMaxQuantizer):
    """out = clamp(round(input / scale) - offset, qmin, qmax)  (affine/quantizer.py:440-563)."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:   # pylint: disable=redefined-builtin
        if self._observe_only(input):
            return input
        input = input.as_subclass(torch.Tensor)
        scale, offset = self._encoding_for(input, "Quantize")
        out = backend.quantize(input, scale, offset, self.qmin, self.qmax, block_size=self.block_size)
        return self._wrap(out, QuantizedTensor, scale, offset)


class QuantizeDequantize(MinMaxQuantizer):
    """out = (clamp(round(input / scale) - offset, qmin, qmax) + offset) * scale  (affine/quantizer.py:566-697)."""

    def forward(self, input: torch.Tensor) -> torch.Tensor:   # pylint: disable=redefined-builtin
        if self._observe_only(input):
            return input
        input = input.as_subclass(torch.Tensor)
        scale, offset = self._encoding_for(input, "QuantizeDequantize")
        out = backend.quantize_dequantize(input, scale, offset, self.qmin, self.qmax, block_size=self.block_size)
        return self._wrap(out, DequantizedTensor, scale, offset)


class GroupedBlockQuantizeDequantize(QuantizeDequantize):
    """Blockwise quantize-dequantize whose per-block scales are themselves restricted to an integer multiple
    (1 .. 2^(decompressed_bw - bitwidth)) of one scale per group of blocks -- "LPBQ"
    (affine/quantizer.py:700-815: same constructor, ``get_scale`` override, ``get_expanded_scale_shape``,
    ``get_per_channel_scale``, ``get_per_block_integer_scale``).  The element arithmetic is the blockwise kernel; the
    scale adjustment is one small quantize-dequantize of the scale tensor."""

    def __init__(self, shape, bitwidth: int, symmetric: bool, decompressed_bw: int,
                 encoding_analyzer: Optional[EncodingAnalyzer] = None, block_size: Optional[Tuple[int, ...]] = None,
                 block_grouping: Optional[Tuple[int, ...]] = None):
        super().__init__(shape, bitwidth, symmetric, encoding_analyzer, block_size)
        self.decompressed_bw = decompressed_bw
        self.block_grouping = block_grouping if block_grouping is not None else tuple(1 for _ in self.shape)
        if block_grouping is not None:
            if len(block_grouping) != len(self.shape):
                raise RuntimeError(f'Length of block grouping {block_grouping} must equal length of shape {shape}.')
            for idx, block_group in enumerate(block_grouping):
                if block_group != -1 and self.shape[idx] % block_group != 0:
                    raise RuntimeError(f'Quantizer shape dimensions must divide evenly with corresponding block '
                                       f'grouping values for shapes {shape} and block grouping {block_grouping}.')
        if self.decompressed_bw < self.bitwidth:
            raise RuntimeError(f'Decompressed bitwidth {decompressed_bw} cannot be smaller than self.bitwidth '
                               f'{bitwidth}')
        if not symmetric:
            raise RuntimeError('GroupedBlockQuantizeDequantize only supports symmetric quantization.')

    def get_expanded_scale_shape(self) -> Tuple[int, ...]:
        """Every scale dimension split into (groups, blocks per group); -1 groups the whole dimension."""
        expanded: List[int] = []
        for idx, block_group in enumerate(self.block_grouping):
            if block_group == -1:
                expanded += [1, self.shape[idx]]
            else:
                expanded += [self.shape[idx] // block_group, block_group]
        return tuple(expanded)

    def _group_scale(self, scale: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        expanded = scale.view(self.get_expanded_scale_shape())
        max_scale = torch.amax(expanded, list(range(1, len(scale.shape) * 2, 2)), keepdim=True)
        # a power of two: dividing and multiplying by the reciprocal give the same bits
        return expanded, max_scale / 2 ** (self.decompressed_bw - self.bitwidth)

    def _transform_scale(self, scale: torch.Tensor) -> torch.Tensor:
        expanded, per_channel_scale = self._group_scale(scale)
        updated = backend.quantize_dequantize(expanded.contiguous(), per_channel_scale,
                                              torch.zeros_like(per_channel_scale), 1,
                                              2 ** (self.decompressed_bw - self.bitwidth))
        return updated.as_subclass(torch.Tensor).view(scale.shape)

    def _raw_scale(self, dtype=None) -> torch.Tensor:
        dtype = dtype or torch.float32
        steps = device_scalar(self.qmax - self.qmin, dtype, self.min.device)
        return ((self.max.to(dtype) - self.min.to(dtype)) / steps).to(dtype)

    def get_per_channel_scale(self, dtype=None) -> torch.Tensor:
        return self._group_scale(self._raw_scale(dtype))[1]

    def get_per_block_integer_scale(self) -> torch.Tensor:
        per_channel_scale = self.get_per_channel_scale()
        expanded = self.get_scale().view(self.get_expanded_scale_shape())
        return torch.round(expanded / per_channel_scale).int().view(self.get_scale().shape)

