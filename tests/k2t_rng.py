"""Seeded synthetic inputs shared by tests and benchmarks (SplitMix64 + Box-Muller via numpy)."""
import numpy as np


def normal(seed, shape, std=1.0):
    return (np.random.Generator(np.random.PCG64(seed)).standard_normal(shape) * std).astype(np.float32)


def uniform_ids(seed, n, vocab):
    return np.random.Generator(np.random.PCG64(seed)).integers(0, vocab, size=n, dtype=np.int64)
