"""B200 quantization backend with the interface of ``aimet_torch.v2.quantization.affine.backends``.

A module satisfying ``_QuantizationBackendProtocol``
(TrainingExtensions/torch/src/python/aimet_torch/v2/quantization/affine/backends/utils.py:45-69): the three
functions ``quantize``, ``dequantize`` and ``quantize_dequantize`` have the signatures, dtype policy, error
behaviour and autograd behaviour of the default ``torch_builtins`` backend (``torch_builtins.py:90-344``), but
each forward and each tensor-gradient is one fused sm_100a kernel launched through the C ABI.

Register it with the reference's own plugin hook::

    from aimet_torch.v2.quantization.affine.backends import add_backend, set_global_backend
    import aimet_b200.v2.backend as b200
    add_backend("aimet_b200", b200); set_global_backend("aimet_b200")

There is no CPU path: CPU tensors raise ``RuntimeError``.
"""
from __future__ import annotations

import functools
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _lib, ops

__all__ = ["quantize", "dequantize", "quantize_dequantize", "resolve_geometry"]


# ---------------------------------------------------------------------------------------------------
# dtype policy (torch_builtins.py:52-87)
# ---------------------------------------------------------------------------------------------------
def _is_value_representable(dtype: torch.dtype, value: int) -> bool:
    r = torch.tensor(value, dtype=dtype)
    return bool(r.isfinite()) and int(r.long()) == value


@functools.lru_cache(None)
def _is_grid_representable(dtype: torch.dtype, qmin: int, qmax: int) -> bool:
    return _is_value_representable(dtype, qmax) and _is_value_representable(dtype, qmax - 1) and \
        _is_value_representable(dtype, qmin + 1) and _is_value_representable(dtype, qmin)


@functools.lru_cache(None)
def _is_numerically_stable(dtype: torch.dtype, qmin: int, qmax: int) -> bool:
    if not _is_grid_representable(dtype, qmin, qmax):
        return False
    if qmin == qmax:
        return True
    if torch.finfo(dtype).eps > 1e-1 / (qmax - qmin):
        return False
    return True


def _is_expandable(src_shape: Sequence[int], target_shape: Sequence[int]) -> bool:
    if len(src_shape) > len(target_shape):
        return False
    for s, t in zip(src_shape[::-1], target_shape[::-1]):
        if s not in (1, t):
            return False
    return True


def _validate_arguments(tensor: torch.Tensor, scale: torch.Tensor, qmin: Optional[int] = None,
                        qmax: Optional[int] = None, block_size: Optional[Sequence[int]] = None):
    """Same checks and messages as torch_builtins._validate_arguments (torch_builtins.py:90-112)."""
    if block_size is not None:
        if len(scale.shape) != len(block_size):
            raise RuntimeError(f'Length of scale shape {scale.shape} must equal length of block size {block_size}')
        for i in range(1, len(block_size) + 1):
            if block_size[-i] == -1:
                if tensor.shape[-i] % scale.shape[-i] != 0:
                    raise RuntimeError(f'Each tensor dimension size for tensor shape {tensor.shape} must divide '
                                       f'evenly with corresponding scale dimension value for scale shape {scale.shape}')
            else:
                if block_size[-i] * scale.shape[-i] != tensor.shape[-i]:
                    raise RuntimeError(f'Each tensor dimension size for tensor shape {tensor.shape} must equal the '
                                       f'corresponding scale dimension size * block size for scale shape {scale.shape} '
                                       f'and block size {block_size}')
    elif not _is_expandable(scale.shape, tensor.shape):
        raise RuntimeError(f"Scale of shape {scale.shape} cannot be expanded like input tensor of shape {tensor.shape}")
    if qmin is not None and qmax is not None:
        if qmin > qmax:
            raise RuntimeError(f"qmin ({qmin}) must be smaller than or equal to qmax ({qmax})")


# ---------------------------------------------------------------------------------------------------
# geometry: (tensor layout, encoding shape, block size) -> "channel = (i / inner) % num_ch" on flat memory
# ---------------------------------------------------------------------------------------------------
class _Geometry:
    """How the flat, dense buffer the kernels walk maps to encodings.

    x_work:       tensor whose storage is walked (the input itself whenever it is dense in memory)
    num_ch/inner: channel of flat element i is (i / inner) % num_ch
    enc_view/enc_perm: reshape + permutation that turn an encoding tensor into channel order when flattened
    t_log/order:  set only when the input had to be permuted (encoding dims interleaved with broadcast dims):
                  x_work == input.reshape(t_log).permute(order).contiguous()
    """
    __slots__ = ("x_work", "num_ch", "inner", "enc_view", "enc_perm", "t_log", "order", "shape")

    def to_work(self, t: torch.Tensor) -> torch.Tensor:
        """Lay ``t`` (logical shape of the input) out like x_work."""
        if self.order is not None:
            return t.reshape(self.t_log).permute(self.order).contiguous()
        if t.shape == self.x_work.shape and t.stride() == self.x_work.stride():
            return t
        w = torch.empty_like(self.x_work, dtype=t.dtype)
        w.copy_(t)
        return w

    def from_work(self, y: torch.Tensor) -> torch.Tensor:
        """Inverse of to_work for results."""
        if self.order is not None:
            inv = [self.order.index(d) for d in range(len(self.order))]
            return y.permute(inv).reshape(self.shape).contiguous()
        return y


def _expanded_shapes(tshape: Sequence[int], sshape: Sequence[int], block_size: Optional[Sequence[int]]):
    """Logical shapes after the reference's block reshape (torch_builtins.py:347-403): every blocked dim d becomes
    (num_blocks_d, block_d) on the tensor side and (num_blocks_d, 1) on the encoding side."""
    if block_size is None:
        pad = len(tshape) - len(sshape)
        return list(tshape), [1] * pad + list(sshape)
    nb = len(block_size)
    t_out: List[int] = list(tshape[:len(tshape) - nb])
    s_out: List[int] = [1] * len(t_out)
    for i in range(nb):
        d = len(tshape) - nb + i
        blocks = sshape[i]
        bs = tshape[d] // blocks if block_size[i] == -1 else block_size[i]
        t_out += [blocks, bs]
        s_out += [blocks, 1]
    return t_out, s_out


def _dense_perm(t: torch.Tensor) -> Optional[List[int]]:
    """Dim order (outermost first) in which ``t`` is a dense row-major buffer, or None if it is not dense."""
    if t.is_contiguous():
        return list(range(t.dim()))
    order = sorted(range(t.dim()), key=lambda d: (-t.stride(d), d))
    expect = 1
    for d in reversed(order):
        if t.shape[d] != 1 and t.stride(d) != expect:
            return None
        expect *= t.shape[d]
    return order


def resolve_geometry(tensor: torch.Tensor, enc_shape: Sequence[int], block_size: Optional[Sequence[int]]) -> _Geometry:
    g = _Geometry()
    g.order, g.t_log, g.shape = None, None, tuple(tensor.shape)
    x = tensor
    if block_size is None:
        perm = _dense_perm(tensor)
    else:
        perm = list(range(tensor.dim())) if tensor.is_contiguous() else None
    if perm is None:
        x = tensor.contiguous()   # strided view (or blocked and not row-major): one dense copy
        perm = list(range(tensor.dim()))
    t_log, s_log = _expanded_shapes(tuple(x.shape), tuple(enc_shape), block_size)
    if block_size is not None:
        perm = list(range(len(t_log)))
    t_phys = [t_log[d] for d in perm]
    s_phys = [s_log[d] for d in perm]
    keep = [i for i, v in enumerate(t_phys) if v != 1]
    t_sq = [t_phys[i] for i in keep]
    s_sq = [s_phys[i] for i in keep]
    nz = [i for i, v in enumerate(s_sq) if v != 1]
    g.enc_view, g.enc_perm = list(s_log), list(perm)
    if not nz:
        g.x_work, g.num_ch, g.inner = x, 1, max(x.numel(), 1)
        return g
    first, last = nz[0], nz[-1]
    if all(s_sq[i] == t_sq[i] for i in range(first, last + 1)):
        inner = 1
        for v in t_sq[last + 1:]:
            inner *= v
        num_ch = 1
        for v in s_sq[first:last + 1]:
            num_ch *= v
        g.x_work, g.num_ch, g.inner = x, num_ch, inner
        return g
    # Encoding dims are interleaved with broadcast dims: bring the encoding dims to the front with one copy.
    enc_dims = [d for d in range(len(t_log)) if s_log[d] != 1]
    rest = [d for d in range(len(t_log)) if s_log[d] == 1]
    g.order, g.t_log = enc_dims + rest, list(t_log)
    xw = x.reshape(t_log).permute(g.order).contiguous()
    num_ch = 1
    for d in enc_dims:
        num_ch *= t_log[d]
    g.x_work, g.num_ch, g.inner = xw, num_ch, max(xw.numel() // max(num_ch, 1), 1)
    g.enc_perm = list(range(len(t_log)))   # logical order of the encoding dims already is channel order
    return g


def _flat_encoding(e: torch.Tensor, g: _Geometry, narrow: Optional[torch.dtype]) -> torch.Tensor:
    """Encoding tensor -> float32 vector in channel order (rounded through ``narrow`` first when the reference
    would hold it in that dtype)."""
    if narrow is not None:
        e = e.to(narrow)
    e = e.to(torch.float32).reshape(g.enc_view)
    if g.enc_perm != list(range(len(g.enc_view))):
        e = e.permute(g.enc_perm)
    return e.reshape(-1).contiguous()


def _encoding_from_flat(flat: torch.Tensor, g: _Geometry, enc_shape) -> torch.Tensor:
    """Inverse of _flat_encoding: a float32 vector in channel order -> the encoding's own shape."""
    view = list(g.enc_view)
    if g.enc_perm != list(range(len(view))):
        inv = [g.enc_perm.index(d) for d in range(len(view))]
        flat = flat.reshape([view[d] for d in g.enc_perm]).permute(inv)
    return flat.reshape(enc_shape)


def _check_inputs(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor):
    if not tensor.is_cuda:
        raise RuntimeError("aimet_b200 backend: input must be a CUDA tensor (no CPU path exists)")
    if scale.device != tensor.device or offset.device != tensor.device:
        raise RuntimeError("aimet_b200 backend: tensor, scale and offset must be on the same device "
                           f"({tensor.device}, {scale.device}, {offset.device})")
    if tensor.dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise RuntimeError(f"aimet_b200 backend: unsupported dtype {tensor.dtype}")


def _offset_like_scale(offset: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return offset if offset.shape == scale.shape else offset.expand(scale.shape)


# ---------------------------------------------------------------------------------------------------
# autograd functions
# ---------------------------------------------------------------------------------------------------
class _QuantDequantFn(torch.autograd.Function):
    """Forward: one kernel (optionally also writes the clamp mask).  Backward: dx = grad * mask in one kernel;
    scale / offset gradients element-wise in one kernel and then summed over the broadcast dims, which is what
    autograd does with the reference's un-reduced returns (torch_builtins.py:329-344)."""

    @staticmethod
    def forward(ctx, tensor, scale, offset, qmin, qmax, block_size, out_kind, narrow):
        g = resolve_geometry(tensor, scale.shape, block_size)
        narrow_dt = tensor.dtype if narrow == 1 else None
        sc = _flat_encoding(scale.detach(), g, narrow_dt)
        of = _flat_encoding(_offset_like_scale(offset.detach(), scale), g, narrow_dt)
        need_mask = tensor.requires_grad or scale.requires_grad or offset.requires_grad
        x = g.x_work
        y = torch.empty_like(x)
        mask = torch.empty_like(x, dtype=torch.uint8) if need_mask else None
        ops.v2_quantize(x, y, mask, sc, of, qmin, qmax, g.num_ch, g.inner, out_kind, narrow)
        param_grad = scale.requires_grad or offset.requires_grad
        ctx.g = g
        ctx.qmin, ctx.qmax = qmin, qmax
        ctx.enc_shape, ctx.off_shape, ctx.block_size = tuple(scale.shape), tuple(offset.shape), block_size
        ctx.save_for_backward(mask, sc if param_grad else None, of if param_grad else None)
        out = g.from_work(y)
        # the layout record stays, the activation itself is kept only when encoding gradients need it
        g.x_work = None
        ctx.x_keep = x if param_grad else None
        return out

    @staticmethod
    def backward(ctx, grad):
        mask, sc, of = ctx.saved_tensors
        g = ctx.g
        need_x, need_s, need_o = ctx.needs_input_grad[0], ctx.needs_input_grad[1], ctx.needs_input_grad[2]
        # grad in the layout the forward kernel walked
        if g.order is not None:
            gw = grad.reshape(g.t_log).permute(g.order).contiguous()
        elif grad.shape == mask.shape and grad.stride() == mask.stride():
            gw = grad
        else:
            gw = torch.empty_like(mask, dtype=grad.dtype)
            gw.copy_(grad)
        dx = ds = do = None
        if need_x:
            dxw = torch.empty_like(gw)
            ops.v2_qdq_backward(gw, mask, dxw)
            dx = g.from_work(dxw)
        if need_s or need_o:
            # summed per encoding channel inside the kernel: the un-reduced tensors of the reference never exist
            dsf, dof = ops.v2_qdq_backward_params_reduced(ctx.x_keep, gw, mask, need_s, need_o, sc, of, ctx.qmin,
                                                          ctx.qmax, g.num_ch, g.inner)
            if dsf is not None:
                ds = _encoding_from_flat(dsf, g, ctx.enc_shape)
            if dof is not None:
                do = _encoding_from_flat(dof, g, ctx.enc_shape)
                if ctx.off_shape != ctx.enc_shape:
                    do = do.sum_to_size(ctx.off_shape)
        return dx, ds, do, None, None, None, None, None


def _reduce_to_encoding(full: torch.Tensor, enc_shape: Tuple[int, ...], block_size) -> torch.Tensor:
    """Sum an element-wise gradient over the dims an encoding is broadcast along (what autograd's sum_to_size does
    for the reference's un-reduced returns)."""
    t_log, s_log = _expanded_shapes(tuple(full.shape), enc_shape, block_size)
    v = full.reshape(t_log)
    dims = [d for d in range(len(t_log)) if s_log[d] == 1 and t_log[d] != 1]
    if dims:
        v = v.sum(dim=dims, keepdim=True)
    return v.reshape(enc_shape)


class _QuantFn(torch.autograd.Function):
    """Integer codes with the gradients of QuantizeFunc (torch_builtins.py:208-247): with masked = grad * mask,
    dx = masked / scale, dscale = -(masked / scale) * (x / scale), doffset = -masked, the last two summed over the dims
    the encoding is broadcast along (autograd's reduction of the reference's un-reduced returns).  Forward and the
    mask product are kernels; the two divisions are tensor expressions on the device (codes are not on the
    fake-quant training path)."""

    @staticmethod
    def forward(ctx, tensor, scale, offset, qmin, qmax, block_size, narrow):
        g = resolve_geometry(tensor, scale.shape, block_size)
        narrow_dt = tensor.dtype if narrow else None
        sc = _flat_encoding(scale.detach(), g, narrow_dt)
        of = _flat_encoding(_offset_like_scale(offset.detach(), scale), g, narrow_dt)
        need_mask = tensor.requires_grad or scale.requires_grad or offset.requires_grad
        x = g.x_work
        y = torch.empty_like(x)
        mask = torch.empty_like(x, dtype=torch.uint8) if need_mask else None
        ops.v2_quantize(x, y, mask, sc, of, qmin, qmax, g.num_ch, g.inner, _lib.AQ_V2_OUT_CODES, narrow)
        out = g.from_work(y)
        g.x_work = None
        ctx.g, ctx.block_size = g, block_size
        ctx.enc_shape, ctx.off_shape = tuple(scale.shape), tuple(offset.shape)
        ctx.save_for_backward(mask, tensor.detach() if scale.requires_grad else None,
                              scale.detach() if (tensor.requires_grad or scale.requires_grad) else None)
        return out

    @staticmethod
    def backward(ctx, grad):
        mask, tensor, scale = ctx.saved_tensors
        g = ctx.g
        if g.order is not None:
            gw = grad.reshape(g.t_log).permute(g.order).contiguous()
        elif grad.shape == mask.shape and grad.stride() == mask.stride():
            gw = grad
        else:
            gw = torch.empty_like(mask, dtype=grad.dtype)
            gw.copy_(grad)
        mw = torch.empty_like(gw)
        ops.v2_qdq_backward(gw, mask, mw)
        masked = g.from_work(mw)
        dx = ds = do = None
        if scale is not None:
            t_log, s_log = _expanded_shapes(tuple(masked.shape), tuple(scale.shape), ctx.block_size)
            by_scale = (masked.reshape(t_log) / scale.reshape(s_log).to(masked.dtype)).reshape(masked.shape)
            if ctx.needs_input_grad[0]:
                dx = by_scale
            if ctx.needs_input_grad[1]:
                ratio = (tensor.reshape(t_log) / scale.reshape(s_log).to(tensor.dtype)).reshape(masked.shape)
                ds = _reduce_to_encoding(-by_scale * ratio, tuple(scale.shape), ctx.block_size).to(scale.dtype)
        if ctx.needs_input_grad[2]:
            do = _reduce_to_encoding(-masked, ctx.enc_shape, ctx.block_size)
            if ctx.off_shape != ctx.enc_shape:
                do = do.sum_to_size(ctx.off_shape)
        return dx, ds, do, None, None, None, None


class _DequantFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tensor, scale, offset, block_size, narrow):
        g = resolve_geometry(tensor, scale.shape, block_size)
        narrow_dt = tensor.dtype if narrow else None
        sc = _flat_encoding(scale.detach(), g, narrow_dt)
        of = _flat_encoding(_offset_like_scale(offset.detach(), scale), g, narrow_dt)
        x = g.x_work
        y = torch.empty_like(x)
        ops.v2_dequantize(x, y, sc, of, g.num_ch, g.inner, narrow)
        ctx.save_for_backward(tensor, scale, offset)
        ctx.block_size = block_size
        return g.from_work(y)

    @staticmethod
    def backward(ctx, grad):
        # DequantizeFunc.backward (torch_builtins.py:279-286).  Dequantize gradients are not on the fake-quant
        # training path; they are evaluated with plain tensor expressions on the device.
        tensor, scale, offset = ctx.saved_tensors
        t_log, s_log = _expanded_shapes(tuple(tensor.shape), tuple(scale.shape), ctx.block_size)
        gv, tv = grad.reshape(t_log), tensor.reshape(t_log)
        sv = scale.reshape(s_log)
        ov = _offset_like_scale(offset, scale).reshape(s_log)
        dx = ds = do = None
        if ctx.needs_input_grad[0]:
            dx = (gv * sv).reshape(tensor.shape)
        if ctx.needs_input_grad[1]:
            ds = _reduce_to_encoding((gv * (tv + ov)).reshape(tensor.shape), tuple(scale.shape), ctx.block_size)
        if ctx.needs_input_grad[2]:
            do = _reduce_to_encoding((gv * sv).reshape(tensor.shape), tuple(scale.shape), ctx.block_size)
            if offset.shape != scale.shape:
                do = do.sum_to_size(offset.shape)
        return dx, ds, do, None, None


# ---------------------------------------------------------------------------------------------------
# public functions (same signatures as torch_builtins.quantize / quantize_dequantize / dequantize)
# ---------------------------------------------------------------------------------------------------
def quantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, qmin: int, qmax: int,
             block_size: Optional[List] = None) -> torch.Tensor:
    """Integer codes in the tensor's own dtype: clamp(round(x / scale) - offset, qmin, qmax)
    (torch_builtins.py:115-144).  The arithmetic dtype is the tensor's dtype, as in the reference."""
    _validate_arguments(tensor, scale, qmin, qmax, block_size)
    _check_inputs(tensor, scale, offset)
    if not _is_grid_representable(tensor.dtype, qmin, qmax):
        raise RuntimeError(f"{tensor.dtype} is unable to represent quantized output of range [{qmin}, {qmax}].")
    narrow = tensor.dtype != torch.float32
    return _QuantFn.apply(tensor, scale, offset, int(qmin), int(qmax), _bs(block_size), narrow)


def quantize_dequantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, qmin: int, qmax: int,
                        block_size: Optional[List] = None) -> torch.Tensor:
    """Fake-quantization (torch_builtins.py:147-180): same dtype, shape and memory format as the input."""
    _validate_arguments(tensor, scale, qmin, qmax, block_size)
    _check_inputs(tensor, scale, offset)
    internal = tensor.dtype
    if not _is_numerically_stable(internal, qmin, qmax):
        internal = torch.float32
        if not _is_numerically_stable(internal, qmin, qmax):
            internal = torch.float64
    if not _is_grid_representable(internal, qmin, qmax):
        raise RuntimeError(f"{internal} is unable to represent quantized output of range [{qmin}, {qmax}].")
    # 0: float32 intermediates, 1: the tensor's own dtype, 2: float64 (grids of 2^24 steps or more)
    narrow = 2 if internal == torch.float64 else int(internal != torch.float32)
    return _QuantDequantFn.apply(tensor, scale, offset, int(qmin), int(qmax), _bs(block_size),
                                 _lib.AQ_V2_OUT_QDQ, narrow)


def dequantize(tensor: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor,
               block_size: Optional[List] = None) -> torch.Tensor:
    """(x + offset) * scale in the tensor's dtype (torch_builtins.py:182-204)."""
    _validate_arguments(tensor, scale, block_size=block_size)
    _check_inputs(tensor, scale, offset)
    narrow = tensor.dtype != torch.float32
    return _DequantFn.apply(tensor, scale, offset, _bs(block_size), narrow)


def _bs(block_size) -> Optional[Tuple[int, ...]]:
    return None if block_size is None else tuple(int(b) for b in block_size)
