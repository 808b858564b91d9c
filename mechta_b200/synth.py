"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures on a private conversation with the real model; here K, V and Q are N(0,1) as the
configurations state, drawn from a counter-based generator keyed by (seed, stream) so that any piece can be
regenerated on its own.
"""
from __future__ import annotations

import numpy as np

# stream ids
S_K, S_V, S_Q, S_KNEW, S_VNEW, S_ACCEPT, S_LEN = range(7)


def normal(seed: int, stream: int, index: int, shape) -> np.ndarray:
    """f32 N(0,1) of `shape`, a pure function of (seed, stream, index)."""
    g = np.random.Generator(np.random.Philox(key=[int(seed), (int(stream) << 32) | (int(index) & 0xFFFFFFFF)]))
    return g.standard_normal(shape, dtype=np.float32)


def accept_counts(seed: int, steps: int) -> np.ndarray:
    """Accepted drafts per verify step, uniform in 0..3."""
    g = np.random.Generator(np.random.Philox(key=[int(seed), S_ACCEPT << 32]))
    return g.integers(0, 4, size=steps, dtype=np.int64)


def session_lengths(seed: int, n: int, lo: int = 1024, hi: int = 131072) -> np.ndarray:
    """Ragged cache lengths of the multi-session configuration, uniform in [lo, hi]."""
    g = np.random.Generator(np.random.Philox(key=[int(seed), S_LEN << 32]))
    return g.integers(lo, hi + 1, size=n, dtype=np.int64)
