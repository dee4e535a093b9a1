"""Learned-grid ("range learning") fake-quantization of the v1 flow on the B200 kernels.

Replaces, with the same function names and argument meaning,

* ``get_computed_encodings`` (aimet_torch/v1/quantsim_straight_through_grad.py:121-160),
* ``calculate_forward_pass`` / ``calculate_gradients`` (``:191-346``) as used by
* ``QuantizeDequantizeFunc`` (aimet_torch/v1/tensor_quantizer.py:898-985): ``QuantizeDequantizeFunc.apply(tensor,
  encoding_min, encoding_max, tensor_quantizer)`` where ``tensor_quantizer`` is any object with the attributes
  ``bitwidth, use_symmetric_encodings, use_strict_symmetric, is_unsigned_symmetric, channel_axis``.

Forward: ``x_round = round_half_even(x / delta) - offset``, clamp to ``[0, num_steps]``, ``(x_quant + offset) * delta``,
mask on the rounded value -- one fused kernel (the reference runs about ten tensor operations and saves ``x_quant``).
Backward: ``dx = grad * mask`` in one kernel; the element-wise terms of the encoding gradients,
``(x_quant + offset - x * mask / delta) * grad`` and ``delta * grad * ~mask``, are the scale / offset terms of the v2
backward kernel evaluated with ``qmin = 0, qmax = num_steps``; they are summed over everything but the channel axis
and combined into the min / max gradients exactly as the reference combines them.
Arithmetic runs in the tensor's dtype like the reference's (16-bit tensors with a bit-width of 16 or more are
computed in float32 and cast back).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from . import _lib
from .v2 import backend

__all__ = ["get_computed_encodings", "QuantizeDequantizeFunc", "quantize_dequantize"]


def _const(value, like: torch.Tensor) -> torch.Tensor:
    return torch.tensor(value, dtype=like.dtype, device=like.device)


def get_computed_encodings(bitwidth: int, encoding_min: torch.Tensor, encoding_max: torch.Tensor,
                           use_symmetric_encodings: bool, use_strict_symmetric: bool,
                           is_unsigned_symmetric: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(delta, offset, num_steps) from the learnable min / max, in their dtype
    (quantsim_straight_through_grad.py:121-160)."""
    num_steps = 2 ** bitwidth - 1
    if use_symmetric_encodings and use_strict_symmetric:
        num_steps -= 1
    half = num_steps / 2
    steps_t = _const(num_steps, encoding_min)
    if use_symmetric_encodings and not is_unsigned_symmetric:
        delta = encoding_max / _const(math.floor(half), encoding_min)
        offset = -_const(math.ceil(half), encoding_min)
    else:
        delta = (encoding_max - encoding_min) / steps_t
        if use_symmetric_encodings:
            offset = encoding_min / delta
        else:
            b_zero = torch.round(-encoding_min / delta)
            b_zero = torch.min(steps_t, torch.max(_const(0.0, encoding_min), b_zero))
            offset = -b_zero
    return delta, offset, steps_t


def _encoding_shape(tensor: torch.Tensor, encoding: torch.Tensor, ch_axis: int) -> Tuple[int, ...]:
    """Per tensor: (); per channel: 1 everywhere but the channel axis (broadcast_to_tensor, ``:69-88``)."""
    if encoding.numel() == 1:
        return ()
    if encoding.numel() != tensor.shape[ch_axis]:
        raise RuntimeError(f"encoding of {encoding.numel()} values does not match dimension {ch_axis} "
                           f"of a tensor of shape {tuple(tensor.shape)}")
    return tuple(d if a == ch_axis else 1 for a, d in enumerate(tensor.shape))


class QuantizeDequantizeFunc(torch.autograd.Function):
    """``QuantizeDequantizeFunc.apply(tensor, encoding_min, encoding_max, tensor_quantizer)``."""

    @staticmethod
    def forward(ctx, tensor, encoding_min, encoding_max, tensor_quantizer):
        bw = int(tensor_quantizer.bitwidth)
        ctx.passthrough = bw == 32
        if ctx.passthrough:
            return tensor
        if encoding_max is None or encoding_min is None:
            raise RuntimeError("Forward pass used for compute_encodings differs from forward pass used during "
                               "training")
        if tensor.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            raise RuntimeError("Invalid input data type. Expected torch.float32 or torch.float16. "
                               f"Got {tensor.dtype}.")
        if not tensor.dtype == encoding_min.dtype == encoding_max.dtype:
            raise RuntimeError("Data type mismatch. Expected the input and encoding min & max to be of same dtype."
                               f"Got {tensor.dtype} input, {encoding_min.dtype} encoding_min, "
                               f"and {encoding_max.dtype} encoding_max")
        if bw >= 32:
            raise RuntimeError(f"Invalid bitwidth: {bw}")
        if not tensor.is_cuda:
            raise RuntimeError("aimet_b200: range learning runs on CUDA tensors only (no CPU path exists)")
        orig_dtype = tensor.dtype
        emin, emax = encoding_min.detach(), encoding_max.detach()
        x = tensor.detach()
        if orig_dtype != torch.float32 and bw >= 16:
            x, emin, emax = x.float(), emin.float(), emax.float()
        sym, strict = bool(tensor_quantizer.use_symmetric_encodings), bool(tensor_quantizer.use_strict_symmetric)
        num_steps = 2 ** bw - 1 - (1 if (sym and strict) else 0)
        delta, offset, steps_t = get_computed_encodings(bw, emin, emax, sym, strict,
                                                        bool(tensor_quantizer.is_unsigned_symmetric))
        ch_axis = int(getattr(tensor_quantizer, "channel_axis", 0))
        shape = _encoding_shape(x, delta, ch_axis)
        want_param = encoding_min.requires_grad or encoding_max.requires_grad
        # the fused forward of the v2 kernels on the grid [0, num_steps], arithmetic in the tensor's own dtype
        with torch.enable_grad():
            xs = x.requires_grad_(tensor.requires_grad or want_param)
            sc = delta.reshape(shape).requires_grad_(want_param)
            of = offset.expand(delta.shape).reshape(shape).clone().requires_grad_(want_param)
            y = backend._QuantDequantFn.apply(xs, sc, of, 0, num_steps, None, _lib.AQ_V2_OUT_QDQ,
                                              x.dtype != torch.float32)
        ctx.graph = (xs, sc, of, y) if (xs.requires_grad or want_param) else None
        ctx.sym, ctx.orig_dtype, ctx.work_dtype = sym, orig_dtype, x.dtype
        ctx.want_x, ctx.want_param = tensor.requires_grad, want_param
        ctx.save_for_backward(emin, emax, steps_t)
        return y.detach().to(orig_dtype)

    @staticmethod
    def backward(ctx, grad):
        if ctx.passthrough:
            return grad, None, None, None
        emin, emax, steps_t = ctx.saved_tensors
        xs, sc, of, y = ctx.graph
        g = grad.to(ctx.work_dtype)
        wanted = ([xs] if ctx.want_x else []) + ([sc, of] if ctx.want_param else [])
        got = list(torch.autograd.grad(y, wanted, g, allow_unused=True))
        dx = got.pop(0).to(ctx.orig_dtype) if ctx.want_x else None
        dmin = dmax = None
        if ctx.want_param:
            ds, do = got
            ds, do = ds.reshape(emin.shape).to(emin.dtype), do.reshape(emin.shape).to(emin.dtype)
            if ctx.sym:
                # symmetric_gradients (``:290-328``)
                dmax = ds / torch.div(steps_t, 2, rounding_mode="floor")
                dmin = -dmax
            else:
                # asymmetric_gradients (``:252-288``)
                term1 = ds / steps_t
                term2 = steps_t / (emax - emin) ** 2 * do
                dmin = -term1 + emax * term2
                dmax = term1 - emin * term2
            dmin, dmax = dmin.to(ctx.orig_dtype), dmax.to(ctx.orig_dtype)
        return dx, dmin, dmax, None


def quantize_dequantize(tensor: torch.Tensor, encoding_min: torch.Tensor, encoding_max: torch.Tensor, bitwidth: int,
                        use_symmetric_encodings: bool = False, use_strict_symmetric: bool = False,
                        is_unsigned_symmetric: bool = False, channel_axis: int = 0) -> torch.Tensor:
    """Functional form: the quantizer attributes are passed directly."""
    class _Q:   # pylint: disable=too-few-public-methods
        pass
    q = _Q()
    q.bitwidth, q.use_symmetric_encodings, q.use_strict_symmetric = bitwidth, use_symmetric_encodings, use_strict_symmetric
    q.is_unsigned_symmetric, q.channel_axis = is_unsigned_symmetric, channel_axis
    return QuantizeDequantizeFunc.apply(tensor, encoding_min, encoding_max, q)
