"""aq_minmax_static: min/max statistics for callers that are not allowed to allocate device memory.

A runtime with a frozen device arena, or an operator callback that its host framework runs with allocation
disabled, cannot hand aq_minmax the workspace it needs.  aq_minmax_static keeps that scratch in a fixed array
inside the library instead.  This test calls it through the C ABI, twice in a row (the array is shared between
calls and keeps the previous call's contents), and requires bit-identical results to aq_minmax.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(x, num_ch, inner, propagate_nan, lib, stream):
    """Returns (reference result via aq_minmax, result via aq_minmax_static), each float32 [2, num_ch]."""
    n = x.numel()
    want = torch.empty((2, num_ch), dtype=torch.float32, device=x.device)
    got = torch.full((2, num_ch), 12345.0, dtype=torch.float32, device=x.device)
    dt = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[x.dtype]
    need = int(lib.aq_minmax_workspace_bytes(n, num_ch, inner))
    ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=x.device)
    rc = lib.aq_minmax(x.data_ptr(), dt, n, num_ch, inner, want[0].data_ptr(), want[1].data_ptr(), int(propagate_nan), 0,
                       ws.data_ptr(), ws.numel(), stream)
    assert rc == 0
    # outputs are allocated by the caller beforehand; the entry point itself gets pointers only
    rc = lib.aq_minmax_static(x.data_ptr(), dt, n, num_ch, inner, got[0].data_ptr(), got[1].data_ptr(),
                              int(propagate_nan), stream)
    assert rc == 0
    return want, got


def _same_bits(a, b):
    a, b = a.cpu().numpy(), b.cpu().numpy()
    return np.array_equal(a.view(np.uint32), b.view(np.uint32)) or \
        np.array_equal(np.nan_to_num(a, nan=7.0), np.nan_to_num(b, nan=7.0))


def test_static_scratch_minmax_matches_workspace_version_twice(cuda):
    from aimet_b200._lib import lib
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=cuda)
    g.manual_seed(11)
    cases = [
        (torch.randn(3_000_017, device=cuda, generator=g) * 3, 1, 3_000_017, False),        # whole tensor, ragged size
        (torch.randn(512, 2304, device=cuda, generator=g), 512, 2304, False),               # per output channel
        (torch.randn(6, 40, 48, device=cuda, generator=g), 40, 48, True),                   # channel wraps over an outer dim
        ((torch.randn(4096, 64, device=cuda, generator=g) * 0.02).to(torch.bfloat16), 4096, 64, False),   # blocks of 64
    ]
    for x, num_ch, inner, prop in cases:
        for call in range(2):   # second call sees the scratch as the first one left it
            want, got = _both(x, num_ch, inner, prop, lib, stream)
            torch.cuda.synchronize()
            assert _same_bits(want, got), (tuple(x.shape), num_ch, inner, call)
    # a different geometry right after: whole tensor again, after the per-channel calls used the same scratch
    x = torch.randn(1 << 20, device=cuda, generator=g)
    x[77] = float("nan")
    want, got = _both(x, 1, x.numel(), True, lib, stream)
    torch.cuda.synchronize()
    assert torch.isnan(got).all() and torch.isnan(want).all()
    want, got = _both(x, 1, x.numel(), False, lib, stream)
    torch.cuda.synchronize()
    assert _same_bits(want, got)


def test_static_scratch_direct_rows_fit_at_any_size(cuda):
    """Block statistics whose rows map one to one to the outputs never touch the array, however many rows there are:
    300,000 blocks of 64 (more than the 131,071 partial pairs the array could hold) are accepted."""
    from aimet_b200._lib import lib
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=cuda)
    g.manual_seed(3)
    x = (torch.randn(300_000, 64, device=cuda, generator=g) * 0.02).to(torch.bfloat16)
    assert lib.aq_minmax_workspace_bytes(x.numel(), 300_000, 64) > (1 << 20)
    want, got = _both(x, 300_000, 64, False, lib, stream)
    torch.cuda.synchronize()
    assert _same_bits(want, got)
    xf = x.float()
    assert torch.equal(got[0], xf.amin(dim=1)) and torch.equal(got[1], xf.amax(dim=1))


def test_static_scratch_allocates_nothing_and_follows_stream_and_device(cuda):
    """The point of the entry: device memory in use does not move across calls.  Also run on a side stream, and on a
    second GPU where there is one (the scratch address is looked up per device)."""
    from aimet_b200._lib import lib
    g = torch.Generator(device=cuda)
    g.manual_seed(5)
    x = torch.randn(6, 40, 4800, device=cuda, generator=g)
    out = torch.empty((2, 40), device=cuda)
    ref_mn = x.permute(1, 0, 2).reshape(40, -1).amin(dim=1)
    ref_mx = x.permute(1, 0, 2).reshape(40, -1).amax(dim=1)
    side = torch.cuda.Stream(cuda)
    side.wait_stream(torch.cuda.current_stream())
    call = lambda st: lib.aq_minmax_static(x.data_ptr(), 0, x.numel(), 40, 4800, out[0].data_ptr(), out[1].data_ptr(),
                                           0, st)
    assert call(side.cuda_stream) == 0   # the first call may look the array up; it still allocates nothing
    side.synchronize()
    allocs = lambda: torch.cuda.memory_stats(cuda).get("allocation.all.allocated", 0)
    for _ in range(3):
        out.fill_(0)
        side.wait_stream(torch.cuda.current_stream())
        torch.cuda.synchronize(cuda)
        free0, allocs0 = torch.cuda.mem_get_info(cuda)[0], allocs()
        assert call(side.cuda_stream) == 0
        side.synchronize()
        assert torch.cuda.mem_get_info(cuda)[0] == free0 and allocs() == allocs0
        assert torch.equal(out[0], ref_mn) and torch.equal(out[1], ref_mx)   # against plain tensor reductions
    if torch.cuda.device_count() > 1:
        d1 = torch.device("cuda:1")
        with torch.cuda.device(d1):
            x1 = x.to(d1)
            o1 = torch.empty((2, 40), device=d1)
            rc = lib.aq_minmax_static(x1.data_ptr(), 0, x1.numel(), 40, 4800, o1[0].data_ptr(), o1[1].data_ptr(), 0,
                                      torch.cuda.current_stream(d1).cuda_stream)
            assert rc == 0
            torch.cuda.synchronize(d1)
            assert torch.equal(o1[0].cpu(), ref_mn.cpu()) and torch.equal(o1[1].cpu(), ref_mx.cpu())


def test_static_scratch_rejects_oversized_geometry(cuda):
    from aimet_b200._lib import lib
    # 400,000 rows of 4 elements need 2 x 400,000 partial floats: more than the 1 MiB array holds... unless the
    # rows are written straight to the outputs (outer == 1); an outer dimension of 2 forces partials.
    rows, inner, num_ch = 400_000, 4, 200_000
    n = rows * inner
    assert lib.aq_minmax_workspace_bytes(n, num_ch, inner) > (1 << 20)
    x = torch.zeros(n, device=cuda)
    out = torch.zeros((2, num_ch), device=cuda)
    rc = lib.aq_minmax_static(x.data_ptr(), 0, n, num_ch, inner, out[0].data_ptr(), out[1].data_ptr(), 0,
                              torch.cuda.current_stream().cuda_stream)
    assert rc == -5   # AQ_ERR_TOO_LARGE, with nothing launched
    assert lib.aq_status_string(rc) == b"size beyond the documented maximum"
    assert lib.aq_minmax_static(None, 0, 8, 1, 8, None, None, 0, None) == -1
