"""Tensor-level wrappers over the C ABI.  torch is used only for device memory and streams.

Every function here launches hand-written sm_100a kernels through ``libaimet_b200.so`` on the current
torch stream of the tensor's device.  CPU tensors are rejected: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Dict, Optional, Sequence, Tuple

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


def qdq_fp16(x: torch.Tensor) -> torch.Tensor:
    """float32 -> float16 -> float32 in one pass (the 16-bit float fake-quantization of the v1 flow)."""
    x = _f32c(x, "input")
    out = torch.empty_like(x)
    with _on(x):
        check(lib.aq_qdq_fp16(x.data_ptr(), out.data_ptr(), x.numel(), _stream(x)), "aq_qdq_fp16")
    return out


_PACKED_DTYPES = {(8, False): torch.uint8, (8, True): torch.int8, (16, False): torch.uint16, (16, True): torch.int16,
                  (32, False): torch.uint32, (32, True): torch.int32}


def quantize_packed(x: torch.Tensor, enc_min: float, enc_max: float, bw: int, shift_to_signed: bool = False,
                    rounding_mode: int = 0) -> torch.Tensor:
    """Integer codes in uint8/16/32 (or int8/16/32) containers, one code per container of max(bw, 8) bits."""
    x = _f32c(x, "input")
    out = torch.empty(x.shape, dtype=_PACKED_DTYPES[(max(int(bw), 8), bool(shift_to_signed))], device=x.device)
    with _on(x):
        check(lib.aq_quantize_packed(x.data_ptr(), out.data_ptr(), x.numel(), float(enc_min), float(enc_max), int(bw),
                                     int(rounding_mode), int(shift_to_signed), _stream(x)), "aq_quantize_packed")
    return out


def dequantize_packed(codes: torch.Tensor, enc_min: float, enc_max: float, bw: int,
                      shift_to_signed: bool = False) -> torch.Tensor:
    _cuda(codes, "codes")
    if codes.dtype != _PACKED_DTYPES[(max(int(bw), 8), bool(shift_to_signed))]:
        raise RuntimeError(f"aimet_b200: {bw}-bit {'signed' if shift_to_signed else 'unsigned'} codes cannot live in "
                           f"{codes.dtype}")
    codes = codes.contiguous()
    out = torch.empty(codes.shape, dtype=torch.float32, device=codes.device)
    with _on(codes):
        check(lib.aq_dequantize_packed(codes.data_ptr(), out.data_ptr(), codes.numel(), float(enc_min), float(enc_max),
                                       int(bw), int(shift_to_signed), _stream(codes)), "aq_dequantize_packed")
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


def v2_qdq_backward_params_reduced(x: torch.Tensor, grad: torch.Tensor, mask: torch.Tensor, want_scale: bool,
                                   want_offset: bool, scale: torch.Tensor, offset: torch.Tensor, qmin: int, qmax: int,
                                   num_ch: int, inner: int) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Scale / offset gradients summed per encoding channel: float32 [num_ch] each (or None)."""
    ds = torch.empty(num_ch, dtype=torch.float32, device=x.device) if want_scale else None
    do = torch.empty(num_ch, dtype=torch.float32, device=x.device) if want_offset else None
    with _on(x):
        check(lib.aq_v2_qdq_backward_params_reduced(x.data_ptr(), grad.data_ptr(), mask.data_ptr(),
                                                    ds.data_ptr() if ds is not None else None,
                                                    do.data_ptr() if do is not None else None, _dt(x), x.numel(),
                                                    int(num_ch), int(inner), scale.data_ptr(), offset.data_ptr(),
                                                    float(qmin), float(qmax), _stream(x)),
              "aq_v2_qdq_backward_params_reduced")
    return ds, do


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


_FLAG_BLOCKS: List[torch.Tensor] = []     # pinned blocks, kept for the life of the process
_FLAG_FREE: List[torch.Tensor] = []       # slots nobody holds


def _pinned_flag() -> torch.Tensor:
    """One int32 of pinned host memory for an asynchronous flag read.  Slots are carved from pooled 4 KiB pinned
    blocks (pinning memory per object would cost more than the synchronisation the probe avoids).  A slot belongs
    to one statistics object until that object hands it back (_release_flag); a slot that is still held is never
    given to anybody else, and a new block is pinned when none is free."""
    if not _FLAG_FREE:
        block = torch.zeros(1024, dtype=torch.int32).pin_memory()
        _FLAG_BLOCKS.append(block)
        _FLAG_FREE.extend(block[i:i + 1] for i in range(block.numel() - 1, -1, -1))
    slot = _FLAG_FREE.pop()
    slot.zero_()
    return slot


def _release_flag(slot: torch.Tensor) -> None:
    _FLAG_FREE.append(slot)


class TfeDeviceState:
    """Device-resident TF-Enhanced statistics of one quantizer: bucket grid + per-batch histogram rows.

    One int32 buffer holds the whole exchangeable part: ``[capacity, 512]`` histogram rows (uint32 stored as int32),
    then ``capacity`` int64 counts (as int32 pairs), then two int32 flags (flag 0: "this rank offered a batch").
    Row b belongs to the b-th batch offered (or to global batch b in a data-parallel calibration).  A batch seen
    before the grid exists (all-zero data) keeps count 0 and is skipped by the replay, exactly as the reference
    drops it.  Pass ``capacity`` = the number of batches of the job when it is known: growing the table later costs a
    reallocation and a copy in the middle of the job.
    """

    def __init__(self, device, capacity: int = 256):
        self.device = torch.device(device)
        # one zero-filled allocation, carved into the state record, the PDF, the result, the iteration count, the
        # gate of the cross-rank grid agreement and this rank's (min, max, present) triple
        sb = (_lib.TFE_STATE_BYTES + 15) // 16 * 16
        pb = _lib.AQ_PDF_SIZE * 8
        blob = torch.zeros(sb + pb + 48 + 16 + 16, dtype=torch.uint8, device=self.device)
        self.state = blob[:_lib.TFE_STATE_BYTES]
        self.pdf = blob[sb:sb + pb].view(torch.float64)
        self.encoding = blob[sb + pb:sb + pb + 40].view(torch.float64)
        self.iterations = blob[sb + pb + 48:sb + pb + 52].view(torch.int32)
        self.gate = blob[sb + pb + 52:sb + pb + 56].view(torch.int32)
        self.range = blob[sb + pb + 64:sb + pb + 76].view(torch.float32)
        self.num_batches = 0
        self.initialized_on_host = False
        self._probe = None
        self._alloc_rows(max(int(capacity), 1))

    def _alloc_rows(self, capacity: int, keep: bool = False):
        P = _lib.AQ_PDF_SIZE
        buf = torch.zeros(capacity * (P + 2) + 2, dtype=torch.int32, device=self.device)
        h = buf[:capacity * P].view(capacity, P)
        c = buf[capacity * P:capacity * (P + 2)].view(torch.int64)
        if keep:
            old = min(self.hists.shape[0], capacity)
            h[:old].copy_(self.hists[:old])
            c[:old].copy_(self.counts[:old])
            buf[-2:].copy_(self.flags)
        self.buffer, self.hists, self.counts, self.flags = buf, h, c, buf[-2:]
        self._hp, self._cp, self._sp = h.data_ptr(), c.data_ptr(), self.state.data_ptr()

    @property
    def capacity(self) -> int:
        return self.hists.shape[0]

    def reserve(self, capacity: int):
        if capacity > self.hists.shape[0]:
            self._alloc_rows(max(capacity, 2 * self.hists.shape[0]), keep=True)

    def resize_exact(self, capacity: int):
        """Makes the table hold exactly ``capacity`` rows, so that ``buffer`` is the dense thing to exchange."""
        if capacity != self.hists.shape[0]:
            self._alloc_rows(capacity, keep=True)
        self.num_batches = capacity

    # ---- grid ----------------------------------------------------------------------------------------------
    def init_grid_from(self, minmax_dev: torch.Tensor):
        """minmax_dev: float32 tensor holding {min, max} on the device."""
        with _on(self.state):
            check(lib.aq_tfe_init_grid(minmax_dev.data_ptr(), self._sp, _stream(self.state)), "aq_tfe_init_grid")

    def _offer(self, x: torch.Tensor, init: bool, want_range: bool):
        _tfe_input(x)
        need = int(lib.aq_tfe_offer_grid_workspace_bytes())
        ws = workspace(x, need)
        with _on(x):
            check(lib.aq_tfe_offer_grid(x.data_ptr(), x.numel(), self._sp, self.range.data_ptr() if want_range else None,
                                        int(init), ws.data_ptr(), ws.numel(), _stream(x)), "aq_tfe_offer_grid")

    def offer_grid(self, x: torch.Tensor):
        """One launch: min/max of the batch and, unless a grid exists or the batch is all zeros, the grid from it."""
        self._offer(x, True, False)

    def batch_range(self, x: Optional[torch.Tensor]) -> torch.Tensor:
        """(min, max, present) of a batch on the device, for the cross-rank grid agreement; leaves the state alone."""
        if x is None:
            self.range.zero_()
        else:
            self._offer(x, False, True)
        return self.range

    def select_grid(self, ranges: torch.Tensor, num_ranks: int, rank: int):
        with _on(self.state):
            check(lib.aq_tfe_select_grid(ranges.data_ptr(), int(num_ranks), int(rank), self._sp, self.gate.data_ptr(),
                                         _stream(self.state)), "aq_tfe_select_grid")

    def is_initialized(self) -> bool:
        """Host view of the device flag (synchronises once per call until it turns true, then cached)."""
        if not self.initialized_on_host:
            self.initialized_on_host = bool(self.state[_INIT_OFF:_INIT_OFF + 4].view(torch.int32).item())
        return self.initialized_on_host

    def poll_initialized(self, wait: bool = False) -> bool:
        """Like is_initialized(), but by default never waits for the device: True once an asynchronous read of the
        flag (start_probe) that saw 1 has completed.  Callers keep offering batches (a no-op on the device once the
        grid exists), each offer followed by start_probe(), while the answer is False.  ``wait`` blocks until the
        read in flight has landed (the device goes on with whatever was queued behind it)."""
        if self.initialized_on_host:
            return True
        probe = self._probe
        if probe is not None and wait:
            probe[1].synchronize()
        if probe is not None and probe[1].query() and int(probe[0].item()) == 1:
            self.initialized_on_host = True
            self._drop_probe()
        return self.initialized_on_host

    def _drop_probe(self) -> None:
        """Hands the pinned slot back.  Only when no copy into it can still be in flight: otherwise the slot stays
        out of circulation (a later owner must never see this object's flag arrive)."""
        probe = self._probe
        self._probe = None
        if probe is not None and probe[1].query():
            _release_flag(probe[0])

    def __del__(self):
        try:
            self._drop_probe()
        except Exception:
            pass

    def start_probe(self) -> None:
        """Queues a copy of the flag, as it is after everything enqueued so far, to pinned host memory."""
        probe = self._probe
        if probe is not None and not probe[1].query():
            return   # the previous read is still in flight
        flag = _pinned_flag() if probe is None else probe[0]
        flag.copy_(self.state[_INIT_OFF:_INIT_OFF + 4].view(torch.int32), non_blocking=True)
        event = torch.cuda.Event() if probe is None else probe[1]
        event.record(torch.cuda.current_stream(self.device))
        self._probe = (flag, event)

    # ---- rows ------------------------------------------------------------------------------------------------
    def add_batch(self, x: torch.Tensor, row: Optional[int] = None, gated: bool = False):
        """Histogram of one batch into row ``row`` (default: the next one).  ``x``: dense float32 CUDA tensor.
        ``gated``: the batch only counts if the last select_grid() said so."""
        _tfe_input(x)
        if row is None:
            row = self.num_batches
        if row >= self.hists.shape[0]:
            self.reserve(row + 1)
        if row >= self.num_batches:
            self.num_batches = row + 1
        with _on(x):
            if gated:
                xs, ns = (C.c_void_p * 1)(x.data_ptr()), (C.c_int64 * 1)(x.numel())
                check(lib.aq_tfe_histogram_many(xs, ns, 1, 1, self._sp, self._hp + row * _HIST_ROW_BYTES,
                                                self._cp + row * 8, self.gate.data_ptr(), _stream(x)),
                      "aq_tfe_histogram_many")
            else:
                check(lib.aq_tfe_histogram(x.data_ptr(), x.numel(), self._sp, self._hp + row * _HIST_ROW_BYTES,
                                           self._cp + row * 8, _stream(x)), "aq_tfe_histogram")

    def add_batches(self, xs: Sequence[torch.Tensor], row0: Optional[int] = None, row_stride: int = 1):
        """Histograms of several resident batches, ``AQ_TFE_HIST_MANY`` per launch, into rows row0, row0 + row_stride,
        ...  Only valid once the grid exists (every batch of a launch sees the same state)."""
        if row0 is None:
            row0 = self.num_batches
        if not xs:
            return
        last = row0 + (len(xs) - 1) * row_stride
        if last >= self.hists.shape[0]:
            self.reserve(last + 1)
        self.num_batches = max(self.num_batches, last + 1)
        M = _lib.AQ_TFE_HIST_MANY
        with _on(xs[0]):
            st = _stream(xs[0])
            for i in range(0, len(xs), M):
                part = xs[i:i + M]
                for x in part:
                    _tfe_input(x)
                m = len(part)
                ptrs = (C.c_void_p * m)(*[x.data_ptr() for x in part])
                ns = (C.c_int64 * m)(*[x.numel() for x in part])
                row = row0 + i * row_stride
                check(lib.aq_tfe_histogram_many(ptrs, ns, m, int(row_stride), self._sp,
                                                self._hp + row * _HIST_ROW_BYTES, self._cp + row * 8, None, st),
                      "aq_tfe_histogram_many")

    # ---- encoding ----------------------------------------------------------------------------------------------
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

    def compute_encoding(self, stats_updated, bw: int, symmetric: bool, strict: bool, unsigned_sym: bool,
                         num_batches: Optional[int] = None) -> torch.Tensor:
        """Replay of the running mean over the rows, then the SQNR search: one call, two dependent launches.
        ``stats_updated``: a bool, or None to take the flag from ``flags[0]`` on the device."""
        nb = self.num_batches if num_batches is None else num_batches
        need = int(lib.aq_tfe_search_workspace_bytes())
        ws = workspace(self.state, need)
        with _on(self.state):
            check(lib.aq_tfe_compute_encoding(self._sp, self._hp, self._cp, nb, self.pdf.data_ptr(),
                                              self.iterations.data_ptr(), int(bool(stats_updated)),
                                              self.flags.data_ptr() if stats_updated is None else None, int(bw),
                                              int(symmetric), int(strict), int(unsigned_sym),
                                              self.encoding.data_ptr(), ws.data_ptr(), ws.numel(),
                                              _stream(self.state)), "aq_tfe_compute_encoding")
        return self.encoding

    def percentile_encoding(self, stats_updated, percentile: float, bw: int, symmetric: bool, strict: bool,
                            unsigned_sym: bool, num_batches: Optional[int] = None) -> torch.Tensor:
        """Replay, then the percentile analyzer's range and grid on the same statistics (one call)."""
        nb = self.num_batches if num_batches is None else num_batches
        with _on(self.state):
            check(lib.aq_tfe_percentile_encoding(self._sp, self._hp, self._cp, nb, self.pdf.data_ptr(),
                                                 self.iterations.data_ptr(), int(bool(stats_updated)),
                                                 self.flags.data_ptr() if stats_updated is None else None,
                                                 float(percentile), int(bw), int(symmetric), int(strict),
                                                 int(unsigned_sym), self.encoding.data_ptr(), _stream(self.state)),
                  "aq_tfe_percentile_encoding")
        return self.encoding

    def mse_encoding(self, stats_updated, bw: int, symmetric: bool, strict: bool, unsigned_sym: bool,
                     num_batches: Optional[int] = None) -> torch.Tensor:
        """Replay, then the MSE analyzer's candidate search on the same statistics (one call)."""
        nb = self.num_batches if num_batches is None else num_batches
        # scratch of its own: the shared per-stream workspace must stay zero where other kernels keep their tickets
        ws = getattr(self, "_mse_ws", None)
        if ws is None:
            ws = self._mse_ws = torch.empty(int(lib.aq_tfe_mse_workspace_bytes()), dtype=torch.uint8,
                                            device=self.state.device)
        with _on(self.state):
            check(lib.aq_tfe_mse_encoding(self._sp, self._hp, self._cp, nb, self.pdf.data_ptr(),
                                          self.iterations.data_ptr(), int(bool(stats_updated)),
                                          self.flags.data_ptr() if stats_updated is None else None, int(bw),
                                          int(symmetric), int(strict), int(unsigned_sym), self.encoding.data_ptr(),
                                          ws.data_ptr(), ws.numel(), _stream(self.state)), "aq_tfe_mse_encoding")
        return self.encoding

    def x_left(self) -> torch.Tensor:
        return self.state[:_lib.AQ_PDF_SIZE * 8].view(torch.float64)


def _tfe_input(x: torch.Tensor) -> None:
    if x.dtype != torch.float32 or not x.is_cuda:
        raise RuntimeError("aimet_b200: TF-Enhanced statistics take float32 CUDA input (callers upcast)")
