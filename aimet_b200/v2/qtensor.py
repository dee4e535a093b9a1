"""Tensors that remember how they were quantized: ``QuantizedTensor`` (integer codes held in a floating-point
tensor) and ``DequantizedTensor`` (fake-quantized values), each with an ``encoding`` attribute.

Same classes, methods and propagation rules as aimet_torch/v2/quantization/tensor.py:62-484: ``quantize()`` /
``dequantize()`` are idempotent and go through the encoding (hence through the CUDA backend); ``quantized_repr()``
returns the codes in the encoding's integer dtype; casts and moves keep the encoding, re-layout operations
(views, slices, permutes, gathers ...) keep it only when it is per-tensor, an in-place arithmetic operation
invalidates it, and every other operation returns a plain ``torch.Tensor``.
"""
from __future__ import annotations

import copy

import torch
from torch.utils._pytree import tree_map

__all__ = ["QuantizedTensorBase", "QuantizedTensor", "DequantizedTensor", "EncodingError"]


class EncodingError(RuntimeError):
    """The tensor carries no (valid) encoding (tensor.py:487-488)."""


def _ops(names, *owners):
    found = set()
    for name in names.split():
        for owner in owners:
            fn = getattr(owner, name, None)
            if fn is not None:
                found.add(fn)
    return found


# dtype / device changes: the values are the same numbers, so the encoding still describes them
_CAST_OPS = _ops("half float double char short int long cuda cpu to type type_as", torch.Tensor)
# always harmless
_KEEP_OPS = _ops("contiguous requires_grad_ share_memory_", torch.Tensor)
# operations that move, select or repeat elements without changing any value: valid under ONE scale / offset
_LAYOUT_OPS = _ops(
    "__getitem__ as_strided broadcast_to chunk dsplit expand expand_as flatten flip fliplr flipud gather hsplit "
    "index_select kthvalue masked_select movedim moveaxis msort narrow permute repeat reshape reshape_as resize "
    "resize_ resize_as resize_as_ select split squeeze squeeze_ swapaxes swapdims t t_ take take_along_dim "
    "tensor_split tile transpose unflatten unsqueeze unsqueeze_ view view_as",
    torch.Tensor,
) | _ops(
    "as_strided as_strided_copy chunk dsplit expand_copy flatten flip fliplr flipud gather hsplit index_select "
    "masked_select moveaxis movedim narrow narrow_copy permute permute_copy reshape select split squeeze "
    "squeeze_copy swapaxes swapdims t take take_along_dim tensor_split tile t_copy unbind unflatten unsqueeze "
    "unsqueeze_copy vsplit view_copy",
    torch,
)


def _stamp(value, encoding):
    """Gives every quantized tensor inside ``value`` (a tensor or a container of tensors) its own copy of ``encoding``."""

    def one(t):
        if isinstance(t, QuantizedTensorBase):
            t.encoding = copy.copy(encoding)
        return t

    return tree_map(one, value)


def _plain(value):
    return tree_map(lambda t: t.as_subclass(torch.Tensor) if isinstance(t, QuantizedTensorBase) else t, value)


def _plain_unless_encoded(value):
    """Results of operations that are not known to preserve the quantization: plain tensors -- except a result that
    already carries an encoding of its own (a deep copy brings its copied attributes along)."""

    def one(t):
        if isinstance(t, QuantizedTensorBase) and getattr(t, "encoding", None) is None:
            return t.as_subclass(torch.Tensor)
        return t

    return tree_map(one, value)


class QuantizedTensorBase(torch.Tensor):
    """Common behaviour of the two classes below (tensor.py:62-358)."""

    encoding = None

    @classmethod
    def __new__(cls, *args, **kwargs):
        encoding = kwargs.pop("encoding", None)
        out = super().__new__(*args, **kwargs)
        if not out.is_floating_point():
            raise RuntimeError(f"Non-floating point dtype `{out.dtype}` is not allowed for quantized tensors.")
        out.encoding = encoding
        return out

    # deep copies are built through new_empty; the result must be of this class and keep the encoding slot
    def new_empty(self, size, *, dtype=None, device=None, requires_grad=False, layout=torch.strided,
                  pin_memory=False, **kwargs):
        encoding = kwargs.pop("encoding", None)
        out = super().new_empty(size, dtype=dtype, device=device, requires_grad=requires_grad, layout=layout,
                                pin_memory=pin_memory, **kwargs).as_subclass(type(self))
        out.encoding = encoding
        return out

    def quantize(self) -> "QuantizedTensor":
        raise NotImplementedError

    def dequantize(self) -> "DequantizedTensor":
        raise NotImplementedError

    def quantized_repr(self) -> torch.Tensor:
        """The integer codes as a plain tensor of ``encoding.dtype``."""
        if self.encoding is None:
            raise EncodingError("Encoding does not exist")
        return self.quantize().as_subclass(torch.Tensor).to(self.encoding.dtype)

    def clone(self, *, memory_format=torch.preserve_format):
        out = self.as_subclass(torch.Tensor).clone(memory_format=memory_format).as_subclass(type(self))
        out.encoding = self.encoding and self.encoding._clone()   # pylint: disable=protected-access
        return out

    def detach(self):
        out = self.as_subclass(torch.Tensor).detach().as_subclass(type(self))
        out.encoding = self.encoding and self.encoding._detach()   # pylint: disable=protected-access
        return out

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func in (torch.clone, torch.Tensor.clone) and isinstance(args[0], QuantizedTensorBase):
            return QuantizedTensorBase.clone(*args, **kwargs)
        if func in (torch.detach, torch.Tensor.detach) and isinstance(args[0], QuantizedTensorBase):
            return QuantizedTensorBase.detach(*args, **kwargs)
        out = super().__torch_function__(func, types, args, kwargs)
        first = args[0] if args else None
        if not isinstance(first, QuantizedTensorBase):
            return _plain(out)   # e.g. plain_tensor + qtensor
        if func in _CAST_OPS:
            if not out.dtype.is_floating_point:
                raise RuntimeError(f"Type casting to non-floating point dtype `{out.dtype}` is not allowed for "
                                   "quantized tensors. To cast quantized tensors to integer, use "
                                   "`qtensor.quantzed_repr()`.")
            out.encoding = first.encoding and first.encoding.to(device=out.device)
            return out
        if func in _KEEP_OPS:
            return out if out is first else _stamp(out, first.encoding)
        if func in _LAYOUT_OPS:
            if out is first:
                return out
            per_tensor = first.encoding is not None and first.encoding.granularity == "pertensor"
            return _stamp(out, first.encoding if per_tensor else None)
        if out is first:
            out.encoding = None   # changed in place: whatever described the old values is stale
            return out
        return _plain_unless_encoded(out)


class QuantizedTensor(QuantizedTensorBase):
    """Integer codes in a floating-point tensor (tensor.py:361-411)."""

    def quantize(self) -> "QuantizedTensor":
        return self

    def dequantize(self) -> "DequantizedTensor":
        if self.encoding is None:
            raise EncodingError("Encoding does not exist")
        out = self.encoding.dequantize(self.as_subclass(torch.Tensor)).as_subclass(DequantizedTensor)
        out.encoding = copy.copy(self.encoding)
        return out


class DequantizedTensor(QuantizedTensorBase):
    """Fake-quantized real values (tensor.py:414-484)."""

    def quantize(self) -> QuantizedTensor:
        if self.encoding is None:
            raise EncodingError("Encoding does not exist")
        out = self.encoding.quantize(self.as_subclass(torch.Tensor)).as_subclass(QuantizedTensor)
        out.encoding = copy.copy(self.encoding)
        return out

    def dequantize(self) -> "DequantizedTensor":
        return self
