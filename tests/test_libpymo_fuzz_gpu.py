"""Randomised channel geometries for the libpymo-semantics per-channel kernels (quantize-dequantize, straight-through
backward) and the per-channel min/max reduction, against the CPU oracle."""
import numpy as np
import pytest
import torch

from _data import assert_bits_equal, normal

pytestmark = pytest.mark.gpu


def _geometries(rng, count):
    out = []
    for _ in range(count):
        num_ch = int(rng.choice([1, 2, 3, 5, 16, 64, 100, 513, 3000]))
        inner = int(rng.choice([1, 2, 3, 4, 7, 8, 16, 48, 64, 100, 255, 256, 1000, 2304, 4096, 5000]))
        outer = int(rng.choice([1, 1, 2, 3, 7]))
        if num_ch * inner * outer > 6_000_000:
            outer = 1
        if num_ch * inner > 6_000_000:
            num_ch = max(1, 6_000_000 // inner)
        out.append((outer, num_ch, inner))
    return out


@pytest.mark.parametrize("seed", range(6))
def test_random_channel_geometries(cuda, oracle, seed):
    from aimet_b200 import ops
    rng = np.random.default_rng(500 + seed)
    for outer, num_ch, inner in _geometries(rng, 12):
        what = f"outer {outer} channels {num_ch} inner {inner}"
        x = normal((outer, num_ch, inner), seed=seed + num_ch + inner, scale=1.0)
        g = normal((outer, num_ch, inner), seed=seed + 1, scale=1.0)
        mins = -(rng.random(num_ch) * 2 + 0.2)
        maxs = rng.random(num_ch) * 2 + 0.2
        if rng.random() < 0.5:
            mins = -maxs                       # value-symmetric first channel: one step fewer (the reference's rule)
        grid = oracle.per_channel_grid(mins, maxs, 8)
        steps = 255.0 - (1 if mins[0] == -maxs[0] else 0)
        xd = torch.from_numpy(x).to(cuda)
        mn_d = torch.from_numpy(mins.astype(np.float32)).to(cuda)
        mx_d = torch.from_numpy(maxs.astype(np.float32)).to(cuda)
        got = ops.qdq_per_channel(xd, mn_d, mx_d, num_ch, inner, steps).cpu().numpy()
        assert_bits_equal(got.reshape(-1), oracle.qdq_per_channel(x, num_ch, inner, *grid).reshape(-1), "qdq " + what)
        # straight-through backward with per-channel bounds (the grid's gated min / max)
        emn, emx = grid[0], grid[1]
        dx = ops.ste_backward_v1(xd, torch.from_numpy(g).to(cuda), torch.from_numpy(emn).to(cuda),
                                 torch.from_numpy(emx).to(cuda), num_ch, inner).cpu().numpy()
        bmn = np.broadcast_to(emn.reshape(1, num_ch, 1), x.shape)
        bmx = np.broadcast_to(emx.reshape(1, num_ch, 1), x.shape)
        want_dx = np.where((bmn <= x) & (x <= bmx), g, np.float32(0)).astype(np.float32)
        assert_bits_equal(dx.reshape(-1), want_dx.reshape(-1), "ste " + what)
        # per-channel min / max
        mm = ops.minmax(xd, num_ch, inner).cpu().numpy()
        ch_first = np.moveaxis(x, 1, 0).reshape(num_ch, -1)
        np.testing.assert_array_equal(mm[0], ch_first.min(axis=1), err_msg="min " + what)
        np.testing.assert_array_equal(mm[1], ch_first.max(axis=1), err_msg="max " + what)
