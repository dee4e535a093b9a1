"""TEST INFRASTRUCTURE ONLY: numpy restatement of the aimet_torch v2 affine arithmetic (CPU).

Follows TrainingExtensions/torch/src/python/aimet_torch/v2/quantization/affine/backends/torch_builtins.py
(:115-204 dtype policy and block reshape, :208-344 forward/backward formulas) and
aimet_torch/v2/quantization/encoding_analyzer.py:350-386 (MinMax encodings).

PINNED by tests/test_oracle_pin.py against tests/golden/v2_backend.npz and v2_minmax.npz, which were produced
by the reference's own torch_builtins / MinMaxEncodingAnalyzer (tests/golden/gen_golden.py).

Arithmetic is done in numpy float32 (IEEE, one rounding per operation).  fp16 uses numpy's float16 (which, like
torch on CPU, computes in float32 and rounds once); bf16 is emulated by rounding float32 results to 8 mantissa
bits with round-to-nearest-even.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np

F32 = np.float32
EPS32 = float(np.finfo(np.float32).eps)


def bf16_round(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even), returned as float32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    bias = ((u >> 16) & 1) + 0x7FFF
    r = ((u + bias) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32)
    return np.where(np.isnan(a), a, out).astype(np.float32)


def to_storage(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round float32 values to the storage dtype ('float32' | 'float16' | 'bfloat16'); result as float32."""
    if dtype == "float32":
        return np.asarray(a, np.float32)
    if dtype == "float16":
        with np.errstate(over="ignore"):
            return np.asarray(a, np.float32).astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        return bf16_round(a)
    raise ValueError(dtype)


def _finfo_eps(dtype: str) -> float:
    return {"float32": EPS32, "float16": 2.0 ** -10, "bfloat16": 2.0 ** -7}[dtype]


def _representable(dtype: str, v: int) -> bool:
    r = to_storage(np.array([v], np.float32), dtype)[0]
    return bool(np.isfinite(r)) and int(r) == v and (dtype != "float32" or abs(v) <= 2 ** 24)


def is_grid_representable(dtype: str, qmin: int, qmax: int) -> bool:
    return all(_representable(dtype, v) for v in (qmax, qmax - 1, qmin + 1, qmin))


def is_numerically_stable(dtype: str, qmin: int, qmax: int) -> bool:
    if not is_grid_representable(dtype, qmin, qmax):
        return False
    if qmin == qmax:
        return True
    return not (_finfo_eps(dtype) > 1e-1 / (qmax - qmin))


def internal_dtype(dtype: str, qmin: int, qmax: int) -> str:
    """torch_builtins.py:162-171"""
    if is_numerically_stable(dtype, qmin, qmax):
        return dtype
    if is_numerically_stable("float32", qmin, qmax):
        return "float32"
    return "float64"


def expand(shape: Sequence[int], enc_shape: Sequence[int], block_size: Optional[Sequence[int]]):
    """Shapes after reshape_tensor_for_blocks / get_encoding_shape_with_blocks (torch_builtins.py:347-403)."""
    if block_size is None or len(block_size) == 0:
        return list(shape), [1] * (len(shape) - len(enc_shape)) + list(enc_shape)
    nb = len(block_size)
    t = list(shape[:len(shape) - nb])
    s = [1] * len(t)
    for i in range(nb):
        d = len(shape) - nb + i
        blocks = enc_shape[i]
        bs = shape[d] // blocks if block_size[i] == -1 else block_size[i]
        t += [blocks, bs]
        s += [blocks, 1]
    return t, s


def _ops(dtype: str):
    """Arithmetic helpers that round every result to `dtype` (identity rounding for float32)."""
    def rnd(a):
        return to_storage(a, dtype) if dtype != "float32" else np.asarray(a, np.float32)
    return rnd


def quantize_dequantize(x: np.ndarray, scale: np.ndarray, offset: np.ndarray, qmin: int, qmax: int,
                        block_size=None, dtype: str = "float32", codes_only: bool = False,
                        arithmetic: Optional[str] = None):
    """x: float32 array holding values already representable in `dtype`.  Returns (y, mask) with y rounded to
    `dtype`; mask is (qmin <= round(x/s) - o <= qmax).  `arithmetic` overrides the internal dtype (quantize()
    and dequantize() use the storage dtype itself)."""
    arith = arithmetic or internal_dtype(dtype, qmin, qmax)
    if arith == "float64":
        raise NotImplementedError("float64 internal arithmetic")
    rnd = _ops(arith)
    t_shape, s_shape = expand(x.shape, scale.shape, block_size)
    xv = np.asarray(x, np.float32).reshape(t_shape)
    s = rnd(np.asarray(scale, np.float32)).reshape(s_shape)
    o = rnd(np.broadcast_to(np.asarray(offset, np.float32), scale.shape)).reshape(s_shape)
    with np.errstate(all="ignore"):
        r = rnd(xv / s)
        r = np.rint(r).astype(np.float32)
        r = rnd(r - o)
        mask = (F32(qmin) <= r) & (r <= F32(qmax))
        q = np.where(np.isnan(r), r, np.clip(r, F32(qmin), F32(qmax))).astype(np.float32)
        if codes_only:
            y = q
        else:
            y = rnd(rnd(q + o) * s)
    return to_storage(y, dtype).reshape(x.shape), mask.reshape(x.shape)


def dequantize(x: np.ndarray, scale: np.ndarray, offset: np.ndarray, block_size=None, dtype: str = "float32"):
    rnd = _ops(dtype)
    t_shape, s_shape = expand(x.shape, scale.shape, block_size)
    xv = np.asarray(x, np.float32).reshape(t_shape)
    s = rnd(np.asarray(scale, np.float32)).reshape(s_shape)
    o = rnd(np.broadcast_to(np.asarray(offset, np.float32), scale.shape)).reshape(s_shape)
    with np.errstate(all="ignore"):
        y = rnd(rnd(xv + o) * s)
    return y.reshape(x.shape)


def backward(x: np.ndarray, gy: np.ndarray, scale: np.ndarray, offset: np.ndarray, qmin: int, qmax: int,
             block_size=None, dtype: str = "float32"):
    """QuantDequantFunc.backward (torch_builtins.py:329-344) for the float32-internal case, plus the sum over
    broadcast dims that autograd applies.  Returns (dx in `dtype`, dscale, doffset)."""
    t_shape, s_shape = expand(x.shape, scale.shape, block_size)
    xv = np.asarray(x, np.float32).reshape(t_shape)
    g = np.asarray(gy, np.float32).reshape(t_shape)
    s = np.asarray(scale, np.float32).reshape(s_shape)
    o = np.broadcast_to(np.asarray(offset, np.float32), scale.shape).reshape(s_shape)
    with np.errstate(all="ignore"):
        t = (xv / s).astype(np.float32)
        r = (np.rint(t) - o).astype(np.float32)
        mask = (F32(qmin) <= r) & (r <= F32(qmax))
        m = mask.astype(np.float32)
        dx = (g * m).astype(np.float32)
        c = np.clip(np.rint(t), o + F32(qmin), o + F32(qmax)).astype(np.float32)
        ds = (g * (c - (t * m).astype(np.float32)).astype(np.float32)).astype(np.float32)
        do = (g * ((1 - m) * s).astype(np.float32)).astype(np.float32)
    axes = tuple(d for d in range(len(t_shape)) if s_shape[d] == 1 and t_shape[d] != 1)
    return (to_storage(dx, dtype).reshape(x.shape), ds.reshape(t_shape), do.reshape(t_shape), axes, s_shape)


def minmax_encodings(mn: np.ndarray, mx: np.ndarray, num_steps: int, symmetric: bool, dtype: str = "float32"):
    """MinMaxEncodingAnalyzer.compute_encodings_from_stats (encoding_analyzer.py:350-386), in the stats dtype."""
    # Type promotion in the reference: min/max clamping and the range test run in the stats dtype, but
    # `_MINIMUM_SCALE * (diff < _MINIMUM_SCALE)` is a float32 tensor, so everything it touches (the adjusted
    # max, and the whole symmetric branch) is float32 until the final `.to(stats dtype)`.
    rnd = _ops(dtype)
    mn = rnd(np.minimum(np.asarray(mn, np.float32), F32(0)))
    mx = rnd(np.maximum(np.asarray(mx, np.float32), F32(0)))
    fmax = {"float32": np.finfo(np.float32).max, "float16": 65504.0, "bfloat16": 3.3895313892515355e38}[dtype]
    with np.errstate(all="ignore"):
        diff = rnd(rnd(mx - mn) / F32(num_steps))
        adj = (F32(EPS32) * (diff < F32(EPS32)).astype(np.float32)).astype(np.float32)
        if symmetric:
            pos, neg = math.floor(num_steps / 2), math.ceil(num_steps / 2)
            umax = (mx + (F32(pos) * adj).astype(np.float32)).astype(np.float32)
            umin = (mn - (F32(neg) * adj).astype(np.float32)).astype(np.float32)
            delta = np.maximum((umax / F32(pos)).astype(np.float32), ((-umin) / F32(neg)).astype(np.float32))
            umin = (F32(-neg) * delta).astype(np.float32)
            umax = (F32(pos) * delta).astype(np.float32)
        else:
            umax = (mx + (F32(num_steps) * adj).astype(np.float32)).astype(np.float32)
            umin = mn
        umax = to_storage(np.minimum(umax, F32(fmax)), dtype)
        umin = to_storage(np.maximum(umin, F32(-fmax)), dtype)
    return umin, umax
