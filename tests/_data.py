"""Seeded synthetic inputs shaped like the benchmark configurations (numpy, CPU)."""
import numpy as np

SPECIALS = np.array([0.0, -0.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 0.49999997, -0.49999997, 1e-40, -1e-40, 3e38, -3e38,
                     np.inf, -np.inf, np.nan, 1.0, -1.0, 127.5, 255.5, -128.5], dtype=np.float32)


def normal(shape, seed, scale=1.0, shift=0.0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(shape) * scale + shift).astype(np.float32)


def conv_weight(shape=(64, 32, 3, 3), seed=0):
    """Kaiming-normal conv weight with the 1% largest-magnitude entries scaled x8 (benchmark config 2)."""
    rng = np.random.default_rng(seed)
    fan_in = int(np.prod(shape[1:]))
    w = (rng.standard_normal(shape) * np.sqrt(2.0 / fan_in)).astype(np.float32)
    flat = w.reshape(-1)
    k = int(np.ceil(0.01 * flat.size))
    idx = np.argsort(-np.abs(flat), kind="stable")[:k]
    flat[idx] *= 8
    return w


def relu_activations(shape, seed):
    """ReLU(N(0,1)) with 0.1% outliers x20 (benchmark config 3)."""
    rng = np.random.default_rng(seed)
    a = np.maximum(rng.standard_normal(shape), 0).astype(np.float32)
    m = rng.random(shape) < 1e-3
    a[m] *= 20
    return a


def bits(a):
    a = np.ascontiguousarray(a)
    return a.view({2: np.uint16, 4: np.uint32, 8: np.uint64}[a.dtype.itemsize])


def assert_bits_equal(a, b, what=""):
    """Bit-for-bit equality, except that +0.0 and -0.0 and any two NaNs count as equal."""
    a = np.ascontiguousarray(a)
    b = np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype, (what, a.shape, b.shape, a.dtype, b.dtype)
    same = bits(a) == bits(b)
    if a.dtype.kind == "f":
        same |= (a == b) | (np.isnan(a) & np.isnan(b))
    bad = np.flatnonzero(~same.reshape(-1))
    assert bad.size == 0, f"{what}: {bad.size} mismatches, first at {bad[:5]}: {a.reshape(-1)[bad[:5]]} vs {b.reshape(-1)[bad[:5]]}"
