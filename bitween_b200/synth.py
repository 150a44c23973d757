"""Deterministic synthetic tensors for parity fixtures and benchmarks.

The generator is a counter-based splitmix64 hash evaluated with numpy integer ops and
an Irwin-Hall (sum of uniforms) normal approximation, so the same (seed, shape) gives the
same bits on every machine, numpy version and torch version -- which is what lets a
fixture store only a digest of the reference's output for a large seeded input.  It has
no transcendental function in it on purpose.
"""
import numpy as np

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def _splitmix64(x):
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def uniform01(seed, n, stream=0):
    """n float64 values in [0, 1), a pure function of (seed, stream, index)."""
    with np.errstate(over="ignore"):
        idx = np.arange(1, n + 1, dtype=np.uint64)
        base = _splitmix64(np.uint64(seed) * _GOLDEN + np.uint64(stream) * np.uint64(0xD1B54A32D192ED03))
        z = _splitmix64(base + idx * _GOLDEN)
    return (z >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal(seed, shape, std=1.0, terms=8):
    """float32 array ~ N(0, std^2) (Irwin-Hall with `terms` uniforms, exact in float64)."""
    n = int(np.prod(shape))
    acc = np.zeros(n, dtype=np.float64)
    for t in range(terms):
        acc += uniform01(seed, n, stream=t + 1)
    acc = (acc - terms / 2.0) * np.sqrt(12.0 / terms)
    return (acc * std).astype(np.float32).reshape(shape)


def randint(seed, shape, high):
    n = int(np.prod(shape))
    return (uniform01(seed, n, stream=99) * high).astype(np.int64).reshape(shape)


def uniform(seed, shape, lo=0.0, hi=1.0):
    """float32 array uniform in [lo, hi)."""
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform01(seed, n, stream=77)).astype(np.float32).reshape(shape)
