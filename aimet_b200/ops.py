"""Tensor-level wrappers over the C ABI.  torch is used only for device memory and streams.

Every function here launches hand-written sm_100a kernels through ``libaimet_b200.so`` on the current
torch stream of the tensor's device.  CPU tensors are rejected: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Dict, Optional, Tuple

import torch

from . import _lib
from ._lib import lib, check

_DT = {torch.float32: _lib.AQ_F32, torch.float16: _lib.AQ_F16, torch.bfloat16: _lib.AQ_BF16}


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise RuntimeError(f"aimet_b200: unsupported dtype {t.dtype}") from None


def _cuda(t: torch.Tensor, name: str = "tensor") -> torch.Tensor:
    if not t.is_cuda:
        raise RuntimeError(f"aimet_b200: {name} must be a CUDA tensor (no CPU path exists), got {t.device}")
    return t


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _same_device(a: torch.Tensor, *others: torch.Tensor):
    for o in others:
        if o.device != a.device:
            raise RuntimeError(f"aimet_b200: tensors on different devices ({a.device} vs {o.device})")


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NO_GUARD = _NoGuard()


def _on(t: torch.Tensor):
    """Context that makes t's device current (kernels launch on the current device); free when it already is."""
    if t.device.index is None or t.device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(t.device)


_WS: Dict[Tuple[int, int], torch.Tensor] = {}


def workspace(t: torch.Tensor, nbytes: int) -> torch.Tensor:
    """Zero-initialised, 256-byte aligned scratch, cached per (device, stream).  The kernels that use a ticket
    counter in it leave the counter at zero, so the buffer is zeroed only when it is created or grown."""
    key = (t.device.index if t.device.index is not None else torch.cuda.current_device(), _stream(t))
    ws = _WS.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(int(nbytes), 1 << 16), dtype=torch.uint8, device=t.device)
        _WS[key] = ws
    return ws


# ---------------------------------------------------------------------------------------------------
# libpymo semantics
# ---------------------------------------------------------------------------------------------------
def fill_encoding(bw: int, enc_min: float, enc_max: float) -> _lib.AqEncoding:
    e = _lib.AqEncoding()
    check(lib.aq_fill_encoding(int(bw), float(enc_min), float(enc_max), C.byref(e)), "aq_fill_encoding")
    return e


def computed_encodings(bw: int, mn: float, mx: float, symmetric=False, strict=False, unsigned_sym=False):
    e = _lib.AqEncoding()
    check(lib.aq_computed_encodings(int(bw), float(mn), float(mx), int(symmetric), int(strict), int(unsigned_sym),
                                    C.byref(e)), "aq_computed_encodings")
    return e


def minmax_encoding(bw: int, stat_min: float, stat_max: float, symmetric=False, strict=False, unsigned_sym=False):
    e = _lib.AqEncoding()
    check(lib.aq_minmax_encoding(int(bw), float(stat_min), float(stat_max), int(symmetric), int(strict),
                                 int(unsigned_sym), C.byref(e)), "aq_minmax_encoding")
    return e


def _f32c(t: torch.Tensor, name: str) -> torch.Tensor:
    _cuda(t, name)
    if t.dtype != torch.float32:
        raise RuntimeError(f"aimet_b200: {name} must be float32 for libpymo-semantics ops, got {t.dtype}")
    return t


def qdq_per_tensor(x: torch.Tensor, enc_min: float, enc_max: float, bw: int, rounding_mode: int = 0,
                   out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x`` must be dense in memory (any memory format); the output has the same layout."""
    x = _f32c(x, "input")
    out = torch.empty_like(x) if out is None else out
    with _on(x):
        check(lib.aq_qdq_per_tensor(x.data_ptr(), out.data_ptr(), x.numel(), float(enc_min), float(enc_max), int(bw),
                                    int(rounding_mode), _stream(x)), "aq_qdq_per_tensor")
    return out


def quantize_per_tensor(x: torch.Tensor, enc_min: float, enc_max: float, bw: int, shift_to_signed: bool = False,
                        rounding_mode: int = 0) -> torch.Tensor:
    x = _f32c(x, "input")
    out = torch.empty_like(x)
    with _on(x):
        check(lib.aq_quantize_per_tensor(x.data_ptr(), out.data_ptr(), x.numel(), float(enc_min), float(enc_max),
                                         int(bw), int(rounding_mode), int(shift_to_signed), _stream(x)),
              "aq_quantize_per_tensor")
    return out


def qdq_per_channel(x: torch.Tensor, enc_min: torch.Tensor, enc_max: torch.Tensor, num_ch: int, inner: int,
                    num_steps: float, rounding_mode: int = 0) -> torch.Tensor:
    x = _f32c(x, "input").contiguous()
    enc_min = _f32c(enc_min, "enc_min").contiguous()
    enc_max = _f32c(enc_max, "enc_max").contiguous()
    _same_device(x, enc_min, enc_max)
    if enc_min.numel() != num_ch or enc_max.numel() != num_ch:
        raise RuntimeError("aimet_b200: need one min and one max per channel")
    out = torch.empty_like(x)
    with _on(x):
        check(lib.aq_qdq_per_channel(x.data_ptr(), out.data_ptr(), x.numel(), int(num_ch), int(inner),
                                     enc_min.data_ptr(), enc_max.data_ptr(), float(num_steps), int(rounding_mode),
                                     _stream(x)), "aq_qdq_per_channel")
    return out


def qdq_broadcast(x: torch.Tensor, in_strides, enc_strides, enc_min, enc_max, enc_delta, enc_offset) -> torch.Tensor:
    x = _f32c(x, "input").contiguous()
    encs = [_f32c(e, "encoding").contiguous() for e in (enc_min, enc_max, enc_delta, enc_offset)]
    _same_device(x, *encs)
    nd = len(in_strides)
    ins = (C.c_int64 * nd)(*[int(s) for s in in_strides])
    ens = (C.c_int64 * nd)(*[int(s) for s in enc_strides])
    out = torch.empty_like(x)
    with _on(x):
        check(lib.aq_qdq_broadcast(x.data_ptr(), out.data_ptr(), x.numel(), nd, ins, ens,
                                   *[e.data_ptr() for e in encs], _stream(x)), "aq_qdq_broadcast")
    return out


def ste_backward_v1(x: torch.Tensor, grad: torch.Tensor, enc_min: torch.Tensor, enc_max: torch.Tensor,
                    num_ch: int = 1, inner: Optional[int] = None) -> torch.Tensor:
    x = _f32c(x, "input").contiguous()
    grad = _f32c(grad, "grad").contiguous()
    enc_min = _f32c(enc_min, "enc_min").contiguous()
    enc_max = _f32c(enc_max, "enc_max").contiguous()
    _same_device(x, grad, enc_min, enc_max)
    if inner is None:
        inner = max(x.numel(), 1)
    dx = torch.empty_like(grad)
    with _on(x):
        check(lib.aq_ste_backward_v1(x.data_ptr(), grad.data_ptr(), dx.data_ptr(), x.numel(), int(num_ch),
                                     int(inner), enc_min.data_ptr(), enc_max.data_ptr(), _stream(x)),
              "aq_ste_backward_v1")
    return dx


# ---------------------------------------------------------------------------------------------------
# v2 semantics (flat, physically-contiguous tensors; geometry resolved by the caller)
# ---------------------------------------------------------------------------------------------------
def v2_quantize(x: torch.Tensor, y: torch.Tensor, mask: Optional[torch.Tensor], scale: torch.Tensor,
                offset: torch.Tensor, qmin: int, qmax: int, num_ch: int, inner: int, out_kind: int,
                narrow_internal: bool = False) -> None:
    with _on(x):
        check(lib.aq_v2_quantize(x.data_ptr(), y.data_ptr(), mask.data_ptr() if mask is not None else None, _dt(x),
                                 x.numel(), int(num_ch), int(inner), scale.data_ptr(), offset.data_ptr(),
                                 float(qmin), float(qmax), int(out_kind), int(narrow_internal), _stream(x)),
              "aq_v2_quantize")


def v2_dequantize(x: torch.Tensor, y: torch.Tensor, scale: torch.Tensor, offset: torch.Tensor, num_ch: int,
                  inner: int, narrow_internal: bool = False) -> None:
    with _on(x):
        check(lib.aq_v2_dequantize(x.data_ptr(), y.data_ptr(), _dt(x), x.numel(), int(num_ch), int(inner),
                                   scale.data_ptr(), offset.data_ptr(), int(narrow_internal), _stream(x)),
              "aq_v2_dequantize")


def v2_qdq_backward_params(x: torch.Tensor, grad: torch.Tensor, mask: torch.Tensor, dscale: Optional[torch.Tensor],
                           doffset: Optional[torch.Tensor], scale: torch.Tensor, offset: torch.Tensor, qmin: int,
                           qmax: int, num_ch: int, inner: int) -> None:
    with _on(x):
        check(lib.aq_v2_qdq_backward_params(x.data_ptr(), grad.data_ptr(), mask.data_ptr(),
                                            dscale.data_ptr() if dscale is not None else None,
                                            doffset.data_ptr() if doffset is not None else None, _dt(x), x.numel(),
                                            int(num_ch), int(inner), scale.data_ptr(), offset.data_ptr(),
                                            float(qmin), float(qmax), _stream(x)), "aq_v2_qdq_backward_params")


def v2_qdq_backward(grad: torch.Tensor, mask: torch.Tensor, dx: torch.Tensor) -> None:
    with _on(grad):
        check(lib.aq_v2_qdq_backward(grad.data_ptr(), mask.data_ptr(), dx.data_ptr(), _dt(grad), grad.numel(),
                                     _stream(grad)), "aq_v2_qdq_backward")


# ---------------------------------------------------------------------------------------------------
# statistics
# ---------------------------------------------------------------------------------------------------
def minmax(x: torch.Tensor, num_ch: int = 1, inner: Optional[int] = None, propagate_nan: bool = False,
           out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """Fused min/max.  Returns a float32 tensor [2, num_ch] (row 0 = min, row 1 = max) on x's device.
    ``x`` must be dense in memory.  With ``accumulate`` the result is folded into the values already held by
    ``out`` (running statistics)."""
    _cuda(x, "input")
    n = x.numel()
    if inner is None:
        inner = max(n, 1)
    if out is None:
        out = torch.empty((2, num_ch), dtype=torch.float32, device=x.device)
    need = int(lib.aq_minmax_workspace_bytes(n, int(num_ch), int(inner)))
    if need < 0:
        check(need, "aq_minmax_workspace_bytes")
    ws = workspace(x, need)
    p = out.data_ptr()
    with _on(x):
        check(lib.aq_minmax(x.data_ptr(), _dt(x), n, int(num_ch), int(inner), p, p + 4 * num_ch,
                            int(propagate_nan), int(accumulate), ws.data_ptr(), ws.numel(), _stream(x)), "aq_minmax")
    return out


_INIT_OFF = _lib.AqTfeState.initialized.offset
_HIST_ROW_BYTES = _lib.AQ_PDF_SIZE * 4


_FLAG_POOL: List[torch.Tensor] = []
_FLAG_NEXT = [0]


def _pinned_flag() -> torch.Tensor:
    """One int32 of pinned host memory for an asynchronous flag read.  Slots come from pooled 4 KiB pinned blocks
    (pinning memory per object would cost more than the synchronisation the probe avoids) and are handed out
    round-robin: a probe lives for a few batches, the pool for the process."""
    if not _FLAG_POOL or _FLAG_NEXT[0] >= _FLAG_POOL[-1].numel():
        if len(_FLAG_POOL) >= 16:
            _FLAG_NEXT[0] = 0
            _FLAG_POOL.append(_FLAG_POOL.pop(0))   # recycle the oldest block
        else:
            _FLAG_POOL.append(torch.zeros(1024, dtype=torch.int32).pin_memory())
            _FLAG_NEXT[0] = 0
    i = _FLAG_NEXT[0]
    _FLAG_NEXT[0] = i + 1
    slot = _FLAG_POOL[-1][i:i + 1]
    slot.zero_()
    return slot


class TfeDeviceState:
    """Device-resident TF-Enhanced statistics of one quantizer: bucket grid + per-batch histogram rows.

    ``hists`` is [capacity, 512] uint32 (stored as int32) and ``counts`` [capacity] int64; row b belongs to the
    b-th batch offered.  A batch seen before the grid exists (all-zero data) keeps count 0 and is skipped by
    the replay, exactly as the reference drops it.
    """

    def __init__(self, device, capacity: int = 256):
        self.device = torch.device(device)
        # one zero-filled allocation, carved into the state record, the PDF, the result and the iteration count
        sb = (_lib.TFE_STATE_BYTES + 15) // 16 * 16
        pb = _lib.AQ_PDF_SIZE * 8
        blob = torch.zeros(sb + pb + 48 + 16, dtype=torch.uint8, device=self.device)
        self.state = blob[:_lib.TFE_STATE_BYTES]
        self.pdf = blob[sb:sb + pb].view(torch.float64)
        self.encoding = blob[sb + pb:sb + pb + 40].view(torch.float64)
        self.iterations = blob[sb + pb + 48:sb + pb + 52].view(torch.int32)
        self.num_batches = 0
        self.initialized_on_host = False
        self._alloc_rows(capacity)

    def _alloc_rows(self, capacity: int, keep: bool = False):
        rows = torch.zeros(capacity * (_lib.AQ_PDF_SIZE + 2), dtype=torch.int32, device=self.device)
        h = rows[:capacity * _lib.AQ_PDF_SIZE].view(capacity, _lib.AQ_PDF_SIZE)
        c = rows[capacity * _lib.AQ_PDF_SIZE:].view(torch.int64)
        if keep:
            old = self.hists.shape[0]
            h[:old].copy_(self.hists)
            c[:old].copy_(self.counts)
        self.hists, self.counts = h, c
        self._hp, self._cp, self._sp = h.data_ptr(), c.data_ptr(), self.state.data_ptr()

    def reserve(self, capacity: int):
        if capacity > self.hists.shape[0]:
            self._alloc_rows(max(capacity, 2 * self.hists.shape[0]), keep=True)

    def init_grid_from(self, minmax_dev: torch.Tensor):
        """minmax_dev: float32 tensor holding {min, max} on the device."""
        with _on(self.state):
            check(lib.aq_tfe_init_grid(minmax_dev.data_ptr(), self._sp, _stream(self.state)), "aq_tfe_init_grid")

    def is_initialized(self) -> bool:
        """Host view of the device flag (synchronises once per call until it turns true, then cached)."""
        if not self.initialized_on_host:
            self.initialized_on_host = bool(self.state[_INIT_OFF:_INIT_OFF + 4].view(torch.int32).item())
        return self.initialized_on_host

    def poll_initialized(self) -> bool:
        """Like is_initialized(), but never waits for the device: True once an asynchronous read of the flag
        (start_probe) that saw 1 has completed.  Callers keep offering min/max to init_grid_from() (a no-op on the
        device once the grid exists), each offer followed by start_probe(), while the answer is False."""
        if self.initialized_on_host:
            return True
        probe = getattr(self, "_probe", None)
        if probe is not None and probe[1].query() and int(probe[0].item()) == 1:
            self.initialized_on_host = True
            self._probe = None
        return self.initialized_on_host

    def start_probe(self) -> None:
        """Queues a copy of the flag, as it is after everything enqueued so far, to pinned host memory."""
        probe = getattr(self, "_probe", None)
        if probe is not None and not probe[1].query():
            return   # the previous read is still in flight
        flag = _pinned_flag() if probe is None else probe[0]
        flag.copy_(self.state[_INIT_OFF:_INIT_OFF + 4].view(torch.int32), non_blocking=True)
        event = torch.cuda.Event() if probe is None else probe[1]
        event.record(torch.cuda.current_stream(self.device))
        self._probe = (flag, event)

    def add_batch(self, x: torch.Tensor, row: Optional[int] = None):
        """Histogram of one batch into row ``row`` (default: the next one).  ``x``: dense float32 CUDA tensor."""
        if x.dtype != torch.float32 or not x.is_cuda:
            raise RuntimeError("aimet_b200: TF-Enhanced statistics take float32 CUDA input (callers upcast)")
        if row is None:
            row = self.num_batches
        if row >= self.hists.shape[0]:
            self.reserve(row + 1)
        if row >= self.num_batches:
            self.num_batches = row + 1
        with _on(x):
            check(lib.aq_tfe_histogram(x.data_ptr(), x.numel(), self._sp, self._hp + row * _HIST_ROW_BYTES,
                                       self._cp + row * 8, torch.cuda.current_stream().cuda_stream),
                  "aq_tfe_histogram")

    def replay(self, num_batches: Optional[int] = None):
        nb = self.num_batches if num_batches is None else num_batches
        with _on(self.state):
            check(lib.aq_tfe_pdf_replay(self._hp, self._cp, nb, self.pdf.data_ptr(), self.iterations.data_ptr(),
                                        _stream(self.state)), "aq_tfe_pdf_replay")

    def search(self, stats_updated: bool, bw: int, symmetric: bool, strict: bool, unsigned_sym: bool) -> torch.Tensor:
        need = int(lib.aq_tfe_search_workspace_bytes())
        ws = workspace(self.state, need)
        with _on(self.state):
            check(lib.aq_tfe_search(self._sp, self.pdf.data_ptr(), int(stats_updated), int(bw), int(symmetric),
                                    int(strict), int(unsigned_sym), self.encoding.data_ptr(), ws.data_ptr(),
                                    ws.numel(), _stream(self.state)), "aq_tfe_search")
        return self.encoding

    def x_left(self) -> torch.Tensor:
        return self.state[:_lib.AQ_PDF_SIZE * 8].view(torch.float64)
