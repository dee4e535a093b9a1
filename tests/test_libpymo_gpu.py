"""GPU parity of the libpymo-semantics kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from _data import SPECIALS, assert_bits_equal, conv_weight, normal, relu_activations

pytestmark = pytest.mark.gpu


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


SIZES = [0, 1, 3, 127, 128, 129, 1023, 4096, 4097, 100003]


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("enc", [(-0.46, 0.72, 8), (-3.1, 4.2, 8), (-2.0, 2.0, 8), (0.0, 5.0, 4), (-7.0, 3.0, 16),
                                 (0.5, 0.5, 8)])
def test_qdq_per_tensor(oracle, cuda, n, enc):
    from aimet_b200 import ops
    mn, mx, bw = enc
    x = np.concatenate([normal(n, seed=n, scale=2.0), SPECIALS])[:max(n, 0)] if n else np.zeros(0, np.float32)
    if n >= SPECIALS.size:
        x[:SPECIALS.size] = SPECIALS
    want = oracle.qdq_per_tensor(x, mn, mx, bw)
    got = ops.qdq_per_tensor(dev(x, cuda), mn, mx, bw).cpu().numpy()
    assert_bits_equal(got, want, "qdq")
    for shift in (False, True):
        want = oracle.quantize_per_tensor(x, mn, mx, bw, shift)
        got = ops.quantize_per_tensor(dev(x, cuda), mn, mx, bw, shift).cpu().numpy()
        assert_bits_equal(got, want, "codes")


def test_qdq_per_tensor_misaligned(oracle, cuda):
    from aimet_b200 import ops
    x = normal(10001, seed=3)
    xd = dev(x, cuda)
    for off in (1, 2, 3):
        want = oracle.qdq_per_tensor(x[off:], -1.0, 2.0, 8)
        got = ops.qdq_per_tensor(xd[off:], -1.0, 2.0, 8).cpu().numpy()
        assert_bits_equal(got, want, f"offset {off}")


@pytest.mark.parametrize("shape", [(64, 32, 3, 3), (16, 7, 3, 3), (5, 1, 1, 1), (512, 2304), (3, 10000), (8, 4, 2)])
@pytest.mark.parametrize("bw", [8, 4])
def test_qdq_per_channel(oracle, cuda, shape, bw):
    from aimet_b200 import ops
    w = conv_weight(shape, seed=1) if len(shape) == 4 else normal(shape, seed=2, scale=0.05)
    num_ch = shape[0]
    inner = int(np.prod(shape[1:]))
    flat = w.reshape(num_ch, inner)
    # symmetric (value-symmetric min/max on channel 0 -> one step fewer) and asymmetric encodings
    for symmetric in (True, False):
        if symmetric:
            m = np.abs(flat).max(axis=1).astype(np.float64)
            mins, maxs = -m, m
        else:
            mins, maxs = flat.min(axis=1).astype(np.float64), flat.max(axis=1).astype(np.float64)
        g = oracle.per_channel_grid(mins, maxs, bw)
        want = oracle.qdq_per_channel(w, num_ch, inner, *g)
        steps = 2.0 ** bw - 1 - (1 if mins[0] == -maxs[0] else 0)
        got = ops.qdq_per_channel(dev(w, cuda), dev(mins.astype(np.float32), cuda), dev(maxs.astype(np.float32), cuda),
                                  num_ch, inner, steps).cpu().numpy()
        assert_bits_equal(got.reshape(-1), want.reshape(-1), f"per-channel sym={symmetric}")


def test_qdq_per_channel_wraps_over_outer(oracle, cuda):
    from aimet_b200 import ops
    # activations [N, C, H, W] quantized per channel C: channel = (i / (H*W)) % C
    x = normal((6, 5, 4, 12), seed=4)
    mins = np.linspace(-1.5, -0.5, 5)
    maxs = np.linspace(0.5, 2.0, 5)
    g = oracle.per_channel_grid(mins, maxs, 8)
    want = oracle.qdq_per_channel(x, 5, 48, *g)
    got = ops.qdq_per_channel(dev(x, cuda), dev(mins.astype(np.float32), cuda), dev(maxs.astype(np.float32), cuda), 5, 48,
                              255.0).cpu().numpy()
    assert_bits_equal(got.reshape(-1), want.reshape(-1))


def test_qdq_broadcast_reference_vectors(oracle, cuda):
    """The three known-answer cases of DlQuantization/test/TestQuantizationFunctions.cpp:119-277."""
    from aimet_b200 import ops
    import json, os
    kats = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")))["broadcast"]
    for k in kats:
        x = np.array(k["input"], np.float32)
        enc = [np.array(k[n], np.float32) for n in ("enc_min", "enc_max", "enc_delta", "enc_offset")]
        got = ops.qdq_broadcast(dev(x, cuda), k["in_strides"], k["enc_strides"], *[dev(e, cuda) for e in enc])
        assert_bits_equal(got.cpu().numpy(), np.array(k["expected"], np.float32), "broadcast KAT")
        assert_bits_equal(got.cpu().numpy(), oracle.qdq_broadcast(x, k["in_strides"], k["enc_strides"], *enc))


def test_qdq_broadcast_blockwise(oracle, cuda):
    from aimet_b200 import ops
    # weight [O, I] with block 64 on the input dim: encodings [O, I/64]
    O, I, B = 48, 256, 64
    w = normal((O, I), seed=5, scale=0.02)
    blocks = w.reshape(O, I // B, B)
    m = np.abs(blocks).max(axis=2).reshape(-1).astype(np.float32)
    delta = (m / 7).astype(np.float32)
    offset = np.full_like(delta, -8)
    emin, emax = (delta * -8).astype(np.float32), (delta * 7).astype(np.float32)
    in_strides, enc_strides = [I, B, 1], [I // B, 1, 0]
    want = oracle.qdq_broadcast(w, in_strides, enc_strides, emin, emax, delta, offset)
    got = ops.qdq_broadcast(dev(w, cuda), in_strides, enc_strides, dev(emin, cuda), dev(emax, cuda), dev(delta, cuda),
                            dev(offset, cuda)).cpu().numpy()
    assert_bits_equal(got.reshape(-1), want.reshape(-1))


@pytest.mark.parametrize("n", [1, 5, 4096, 100003])
def test_ste_backward_v1(oracle, cuda, n):
    from aimet_b200 import ops
    x = normal(n, seed=6, scale=2.0)
    g = normal(n, seed=7)
    mn, mx = np.float32(-1.25), np.float32(1.75)
    want = oracle.ste_bwd(x, g, mn, mx)
    got = ops.ste_backward_v1(dev(x, cuda), dev(g, cuda), dev(np.array([mn]), cuda), dev(np.array([mx]), cuda))
    assert_bits_equal(got.cpu().numpy(), want)


def test_ste_backward_v1_per_channel(oracle, cuda):
    from aimet_b200 import ops
    x = normal((8, 36), seed=8, scale=2.0)
    g = normal((8, 36), seed=9)
    mins = np.linspace(-2, -0.5, 8).astype(np.float32)
    maxs = np.linspace(0.5, 2, 8).astype(np.float32)
    want = np.stack([oracle.ste_bwd(x[c], g[c], mins[c], maxs[c]) for c in range(8)])
    got = ops.ste_backward_v1(dev(x, cuda), dev(g, cuda), dev(mins, cuda), dev(maxs, cuda), 8, 36)
    assert_bits_equal(got.cpu().numpy(), want)


def test_ste_backward_v1_matches_reference_fixture(cuda):
    """The kernel against compute_dloss_by_dx of the reference itself (tests/golden/v1_ste.npz): bounds inclusive,
    NaN / Inf inputs, per tensor and per channel on axis 0 and 1."""
    import os
    from aimet_b200 import ops
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "v1_ste.npz"))
    names = sorted({k.split("/")[0] for k in g.files})
    for name in names:
        x, grad, want = g[f"{name}/x"], g[f"{name}/grad"], g[f"{name}/dx"]
        mins, maxs = g[f"{name}/min"].reshape(-1), g[f"{name}/max"].reshape(-1)
        axis = int(g[f"{name}/axis"])
        num_ch, inner = (1, x.size) if mins.size == 1 else (x.shape[axis], int(np.prod(x.shape[axis + 1:])))
        got = ops.ste_backward_v1(dev(x, cuda), dev(grad, cuda), dev(mins, cuda), dev(maxs, cuda), num_ch, inner)
        assert_bits_equal(got.cpu().numpy(), want, name)


@pytest.mark.parametrize("n", [1, 3, 128, 4097, 1 << 20, (1 << 22) + 5])
def test_minmax_per_tensor(oracle, cuda, n):
    from aimet_b200 import ops
    x = normal(n, seed=n, scale=3.0)
    if n > 100:
        x[17] = np.nan   # the reference's std::min/std::max folds never pick NaN up
    want = oracle.min_max(x)
    got = ops.minmax(dev(x, cuda)).cpu().numpy().reshape(-1)
    assert_bits_equal(got, want)
    # twice in a row: the ticket counter must have been left at zero
    got = ops.minmax(dev(x, cuda)).cpu().numpy().reshape(-1)
    assert_bits_equal(got, want)


@pytest.mark.parametrize("shape", [(512, 2304), (64, 64), (4096, 64), (3, 50176), (7, 9), (2, 1 << 20)])
def test_minmax_per_channel(oracle, cuda, shape):
    from aimet_b200 import ops
    x = normal(shape, seed=11, scale=2.0)
    want = np.stack([x.min(axis=1), x.max(axis=1)])
    got = ops.minmax(dev(x, cuda), shape[0], shape[1]).cpu().numpy()
    assert_bits_equal(got, want)


def test_minmax_per_channel_with_outer(cuda):
    from aimet_b200 import ops
    x = normal((6, 5, 4, 12), seed=12)
    want = np.stack([x.min(axis=(0, 2, 3)), x.max(axis=(0, 2, 3))])
    got = ops.minmax(dev(x, cuda), 5, 48).cpu().numpy()
    assert_bits_equal(got, want)
