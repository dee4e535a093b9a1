"""Randomised geometry sweep of the v2 backend against the numpy oracle: tensor shapes, encoding shapes that
broadcast in every possible way, block sizes, dtypes, permuted memory layouts and grids from 2 to 16 bits."""
import numpy as np
import pytest
import torch

from _data import assert_bits_equal

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def _random_case(rng):
    ndim = int(rng.integers(1, 5))
    blocked = ndim >= 1 and rng.random() < 0.35
    if blocked:
        nb = int(rng.integers(1, min(ndim, 2) + 1))                 # trailing dims that are split into blocks
        blocks = [int(rng.choice([1, 2, 4, 8, 16, 32, 64])) for _ in range(nb)]
        counts = [int(rng.integers(1, 7)) for _ in range(nb)]
        lead = [int(rng.integers(1, 6)) for _ in range(ndim - nb)]
        shape = lead + [b * c for b, c in zip(blocks, counts)]
        enc = [int(rng.choice([1, d])) for d in lead] + counts
        enc = enc[len(enc) - max(nb, int(rng.integers(nb, ndim + 1))):]   # encoding may have fewer dims than the tensor
        block_size = [(-1 if rng.random() < 0.5 else b) for b in blocks]
        pad = len(enc) - nb
        block_size = [int(rng.choice([1, -1])) if enc[i] == shape[len(shape) - len(enc) + i] else -1
                      for i in range(pad)] + block_size
        # a leading encoding dim that equals the tensor dim is "block size 1"; one that is 1 spans the whole dim
        block_size = [(-1 if enc[i] == 1 else bs) for i, bs in enumerate(block_size[:pad])] + block_size[pad:]
    else:
        shape = [int(rng.choice([1, 2, 3, 5, 8, 16, 33, 64, 130])) for _ in range(ndim)]
        k = int(rng.integers(0, ndim + 1))
        enc = [int(rng.choice([1, d])) for d in shape[ndim - k:]]
        block_size = None
    return shape, enc, block_size


@pytest.mark.parametrize("seed", range(12))
def test_random_geometries(cuda, seed):
    import aimet_b200.v2.backend as b200
    from oracle import v2_oracle as v2
    rng = np.random.default_rng(1000 + seed)
    for _ in range(25):
        shape, enc, block_size = _random_case(rng)
        dtype = str(rng.choice(["float32", "float32", "bfloat16", "float16"]))
        bw = int(rng.choice([2, 4, 8, 8, 12, 16]))
        signed = bool(rng.random() < 0.5)
        steps = 2 ** bw - 1
        qmin, qmax = (-(steps + 1) // 2, steps // 2) if signed else (0, steps)
        x = (rng.standard_normal(shape) * 2).astype(np.float32)
        x = v2.to_storage(x, dtype)
        scale = np.asarray(np.abs(rng.standard_normal(enc)) * 4.0 / steps + 1e-3, dtype=np.float32).reshape(enc)
        offset = np.asarray(np.zeros(enc) if signed else -np.round(rng.random(enc) * steps), dtype=np.float32).reshape(enc)
        try:
            want, wmask = v2.quantize_dequantize(x, scale, offset, qmin, qmax, block_size, dtype)
        except Exception:   # the oracle rejects the combination (grid not representable in the dtype, ...)
            with pytest.raises(RuntimeError):
                b200.quantize_dequantize(torch.from_numpy(x).to(cuda).to(DT[dtype]), torch.tensor(scale, device=cuda),
                                         torch.tensor(offset, device=cuda), qmin, qmax, block_size)
            continue
        xd = torch.from_numpy(x).to(cuda).to(DT[dtype])
        if xd.dim() >= 2 and rng.random() < 0.3:   # same values, permuted memory layout
            perm = list(rng.permutation(xd.dim()))
            inv = [perm.index(d) for d in range(xd.dim())]
            xd = xd.permute(perm).contiguous().permute(inv)
        xd.requires_grad_(True)
        what = f"shape {shape} enc {enc} block {block_size} {dtype} bw {bw} signed {signed}"
        y = b200.quantize_dequantize(xd, torch.tensor(scale, device=cuda), torch.tensor(offset, device=cuda),
                                     qmin, qmax, block_size)
        assert_bits_equal(y.detach().float().cpu().numpy(), want, what)
        y.backward(torch.ones_like(y))
        np.testing.assert_array_equal(xd.grad.float().cpu().numpy() != 0, wmask, err_msg=what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape,enc,block", [
    ((257, 4100), (257, 1), None),                 # rows a little longer than a tile
    ((64, 4160), (64, 65), (-1, 64)),              # 65 blocks of 64 per row: tiles start inside blocks
    ((3, 130, 17, 9), (130, 1, 1), None),          # channel index wraps over the batch dimension, odd run length
    ((5000, 48), (5000, 1), None),                 # many short runs, one encoding each
    ((5000, 16), (5000, 1), None),                 # run = exactly one thread's share of 16-bit packets
    ((7, 5000, 32), (1, 5000, 1), None),           # short runs whose channel wraps
    ((1, 300001), (), None),                       # per tensor, ragged
    ((640, 2304), (640, 1), None),                 # conv-weight rows
    ((96, 2, 2048), (96, 2, 16), (1, 1, 128)),     # blocks of 128 on the last of three dims
])
def test_larger_geometries(cuda, dtype, shape, enc, block):
    import aimet_b200.v2.backend as b200
    from oracle import v2_oracle as v2
    rng = np.random.default_rng(abs(hash((shape, dtype))) % (2 ** 31))
    x = v2.to_storage((rng.standard_normal(shape) * 0.7).astype(np.float32), dtype)
    scale = np.asarray(np.abs(rng.standard_normal(enc)) * 0.02 + 0.01, dtype=np.float32).reshape(enc)
    offset = np.asarray(-np.round(rng.random(enc) * 200), dtype=np.float32).reshape(enc)
    want, wmask = v2.quantize_dequantize(x, scale, offset, 0, 255, block, dtype)
    xd = torch.from_numpy(x).to(cuda).to(DT[dtype]).requires_grad_(True)
    y = b200.quantize_dequantize(xd, torch.tensor(scale, device=cuda), torch.tensor(offset, device=cuda), 0, 255, block)
    assert_bits_equal(y.detach().float().cpu().numpy(), want, "qdq")
    y.backward(torch.ones_like(y))
    np.testing.assert_array_equal(xd.grad.float().cpu().numpy() != 0, wmask)
