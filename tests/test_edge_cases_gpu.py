"""Edge cases through the public entry points: empty tensors, pointers that are not 16-byte aligned, one element
per channel, and sizes around the packet / chunk boundaries -- each against the CPU oracle."""
import numpy as np
import pytest
import torch

from _data import assert_bits_equal, normal

pytestmark = pytest.mark.gpu


def test_empty_inputs(cuda):
    import aimet_b200.v2.backend as b200
    from aimet_b200 import ops
    from aimet_b200._lib import lib
    s, o = torch.tensor(0.1, device=cuda), torch.tensor(0.0, device=cuda)
    for shape in [(0,), (3, 0, 4)]:
        for dt in (torch.float32, torch.bfloat16):
            x = torch.empty(shape, device=cuda, dtype=dt)
            y = b200.quantize_dequantize(x, s, o, -128, 127)
            assert y.shape == x.shape and y.dtype == dt
            assert b200.quantize(x, s, o, -128, 127).shape == x.shape
    mm = ops.minmax(torch.empty(0, device=cuda))
    assert mm[0].item() == float("inf") and mm[1].item() == float("-inf")
    # an empty batch leaves the histogram row untouched and records its size
    st = ops.TfeDeviceState(cuda, capacity=2)
    st.init_grid_from(torch.tensor([-1.0, 1.0], device=cuda))
    st.add_batch(torch.empty(0, device=cuda), 0)
    torch.cuda.synchronize()
    assert int(st.hists[0].sum()) == 0 and int(st.counts[0]) == 0
    assert lib.aq_qdq_per_tensor(None, None, 0, -1.0, 1.0, 8, 0, None) == 0


@pytest.mark.parametrize("shape,num_ch,inner", [((0, 3, 64), 3, 64), ((0, 2, 4), 2, 4), ((0, 512, 2304), 512, 2304)])
def test_empty_per_channel_statistics(cuda, shape, num_ch, inner):
    """No rows at all: every channel reports +inf / -inf, running statistics stay as they were; aq_minmax,
    aq_minmax_static and the size query all accept the geometry."""
    from aimet_b200 import ops
    from aimet_b200._lib import lib
    x = torch.empty(shape, device=cuda)
    assert lib.aq_minmax_workspace_bytes(0, num_ch, inner) >= 0
    mm = ops.minmax(x, num_ch, inner)
    assert mm.shape == (2, num_ch)
    assert (mm[0] == float("inf")).all() and (mm[1] == float("-inf")).all()
    acc = torch.tensor([[-1.0] * num_ch, [2.0] * num_ch], device=cuda)
    ops.minmax(x, num_ch, inner, out=acc, accumulate=True)
    assert (acc[0] == -1.0).all() and (acc[1] == 2.0).all()
    out = torch.zeros((2, num_ch), device=cuda)
    rc = lib.aq_minmax_static(x.data_ptr(), 0, 0, num_ch, inner, out[0].data_ptr(), out[1].data_ptr(), 0,
                              torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    assert (out[0] == float("inf")).all() and (out[1] == float("-inf")).all()


@pytest.mark.parametrize("shift", [1, 2, 3])
@pytest.mark.parametrize("n", [1, 7, 4095, 4096, 4097, 8191, 8193, 100003])
def test_unaligned_pointers_and_ragged_sizes(cuda, oracle, shift, n):
    """Slices that start 4, 8 or 12 bytes past a 16-byte boundary take the narrower packet paths."""
    import aimet_b200.v2.backend as b200
    from oracle import v2_oracle as v2
    from aimet_b200 import ops
    base = normal(n + 8, seed=n + shift, scale=2.0)
    xd = torch.from_numpy(base).to(cuda)[shift:shift + n]
    xn = base[shift:shift + n]
    assert xd.data_ptr() % 16 == 4 * shift
    sc, of = np.float32(0.0371), np.float32(-120.0)
    want, _ = v2.quantize_dequantize(xn, np.array(sc), np.array(of), 0, 255, None, "float32")
    got = b200.quantize_dequantize(xd, torch.tensor(sc, device=cuda), torch.tensor(of, device=cuda), 0, 255)
    assert_bits_equal(got.cpu().numpy(), want, "v2 qdq")
    assert_bits_equal(ops.qdq_per_tensor(xd, -3.0, 4.5, 8).cpu().numpy(), oracle.qdq_per_tensor(xn, -3.0, 4.5, 8), "libpymo qdq")
    mm = ops.minmax(xd).cpu().numpy().reshape(-1)
    assert mm[0] == xn.min() and mm[1] == xn.max()
    # histogram of an unaligned batch
    st = ops.TfeDeviceState(cuda, capacity=1)
    st.init_grid_from(torch.tensor([float(xn.min()), float(xn.max())], device=cuda))
    st.add_batch(xd, 0)
    x_left = oracle.pdf_init(np.float32(xn.min()), np.float32(xn.max()))
    bs, po = oracle.pdf_geometry(x_left)
    np.testing.assert_array_equal(st.hists[0].cpu().numpy().astype(np.int64), oracle.hist512(xn, bs, po).astype(np.int64))


def test_one_element_per_channel_and_tiny_channels(cuda):
    import aimet_b200.v2.backend as b200
    from oracle import v2_oracle as v2
    for shape, enc in [((64, 1), (64, 1)), ((5, 3), (1, 3)), ((2, 3, 2), (2, 3, 2)), ((1000, 2), (1000, 1))]:
        x = normal(shape, 3, 0.5)
        scale = (np.abs(normal(enc, 4, 0.01)) + np.float32(0.002)).astype(np.float32)
        offset = np.zeros(enc, np.float32)
        want, _ = v2.quantize_dequantize(x, scale, offset, -8, 7, None, "float32")
        got = b200.quantize_dequantize(torch.from_numpy(x).to(cuda), torch.from_numpy(scale).to(cuda),
                                       torch.from_numpy(offset).to(cuda), -8, 7)
        assert_bits_equal(got.cpu().numpy(), want, f"{shape} / {enc}")


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("shift", [0, 8, 16, 24])
@pytest.mark.parametrize("rows", [1, 33, 1000])
def test_16bit_forward_at_every_32_byte_phase(cuda, dtype, shift, rows):
    """The 16-bit forward moves a thread's two adjacent packets as one 32-byte access when input and output are 32-byte
    aligned and keeps 16-byte accesses otherwise; tensors that start 0, 16, 32 or 48 bytes past a 64-byte boundary, with
    whole and ragged last tiles, per tensor and in blocks of 64, must give the same bits either way."""
    import aimet_b200.v2.backend as b200
    from oracle import v2_oracle as v2
    tdt = getattr(torch, dtype)
    cols = 192
    n = rows * cols
    base = v2.to_storage(normal(n + 32, seed=rows + shift, scale=0.05), dtype)
    xn = base[shift:shift + n].reshape(rows, cols)
    hold = torch.from_numpy(base).to(cuda).to(tdt)
    xd = hold[shift:shift + n].view(rows, cols)
    assert xd.data_ptr() % 64 == (2 * shift) % 64
    # per tensor, 16-bit grid (the wide guard band) and 8-bit grid
    for qmin, qmax, sc, of in ((0, 65535, 3.1e-6, -32768.0), (-128, 127, 1.7e-3, 3.0)):
        want, _ = v2.quantize_dequantize(xn, np.array(np.float32(sc)), np.array(np.float32(of)), qmin, qmax, None, dtype)
        got = b200.quantize_dequantize(xd, torch.tensor(sc, device=cuda), torch.tensor(of, device=cuda), qmin, qmax)
        assert got.dtype == tdt
        assert_bits_equal(got.float().cpu().numpy(), want, f"per tensor [{qmin}, {qmax}]")
    # blocks of 64 along the last axis, 4-bit symmetric grid
    scale = (np.abs(normal((rows, cols // 64), 7, 0.004)) + np.float32(0.002)).astype(np.float32)
    offset = np.zeros_like(scale)
    want, _ = v2.quantize_dequantize(xn, scale, offset, -8, 7, [1, 64], dtype)
    got = b200.quantize_dequantize(xd, torch.from_numpy(scale).to(cuda), torch.from_numpy(offset).to(cuda), -8, 7,
                                   block_size=[1, 64])
    assert_bits_equal(got.float().cpu().numpy(), want, "blocks of 64")
