"""Seeded synthetic inputs shared by the tests (shapes and value
distributions of the benchmark configurations)."""
import numpy as np


def tanh_normal(n, seed=0):
    rng = np.random.default_rng(seed)
    return np.tanh(rng.standard_normal(n, dtype=np.float32)).astype(np.float32)


def normal(n, seed=0):
    return np.random.default_rng(seed).standard_normal(n, dtype=np.float32)


def uniform(n, seed=0):
    return np.random.default_rng(seed).uniform(-1, 1, n).astype(np.float32)


def relu_normal(n, zero_fraction, seed=0):
    """max(0, N(mu, 1)) with mu set for the requested share of zeros."""
    mu = {0.5: 0.0, 0.75: -0.6745, 0.9: -1.2816}[zero_fraction]
    rng = np.random.default_rng(seed)
    return np.maximum(0.0, rng.standard_normal(n, dtype=np.float32) + np.float32(mu)).astype(np.float32)


def block_zoo(n, seed=0):
    """A mix of awkward 64-value blocks: zeros, constants, single spikes,
    alternating signs, smooth ramps, wide dynamic range, tiny values."""
    rng = np.random.default_rng(seed)
    a = np.zeros(n, dtype=np.float32)
    nb = n // 64
    for b in range(nb):
        k = b % 9
        s = slice(64 * b, 64 * b + 64)
        if k == 0:
            pass
        elif k == 1:
            a[s] = rng.standard_normal()
        elif k == 2:
            a[64 * b + rng.integers(64)] = rng.standard_normal() * 10.0 ** rng.integers(-5, 5)
        elif k == 3:
            a[s] = np.where(np.arange(64) % 2 == 0, 1.0, -1.0) * rng.uniform(0.1, 2.0)
        elif k == 4:
            a[s] = np.linspace(-1, 1, 64) * rng.uniform(0.5, 50)
        elif k == 5:
            a[s] = rng.standard_normal(64) * 10.0 ** rng.integers(-12, 12, 64)
        elif k == 6:
            a[s] = rng.standard_normal(64) * 1e-30
        elif k == 7:
            a[s] = rng.standard_normal(64) * (rng.random(64) < 0.1)
        else:
            a[s] = np.sin(0.37 * np.arange(64) + b) * 1.5
    return a


def arbitrary_streams(words, seed):
    """uint32 streams that no encoder wrote: random bits, sparse bits, all
    ones, and random bits behind 23 zero bits after every fourth word's header
    (many empty leading planes)."""
    rng = np.random.default_rng(seed)
    dense = rng.integers(0, 2**32, words, dtype=np.uint64).astype(np.uint32)
    sparse = dense & rng.integers(0, 2**32, words, dtype=np.uint64).astype(np.uint32) & \
        rng.integers(0, 2**32, words, dtype=np.uint64).astype(np.uint32)
    ones = np.full(words, 0xFFFFFFFF, dtype=np.uint32)
    late = dense.copy()
    late[0::4] &= np.uint32(0x1FF)
    late[0::4] |= np.uint32(1)
    return [dense, sparse | np.uint32(1), ones, late]
