"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures on a private conversation with the real model; here K, V and Q are N(0,1) as the
configurations state, drawn from a counter-based generator keyed by (seed, stream) so that any piece can be
regenerated on its own.
"""
from __future__ import annotations

import numpy as np

# stream ids
S_K, S_V, S_Q, S_KNEW, S_VNEW, S_ACCEPT, S_LEN, S_QF, S_NORM = range(9)


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


def step_inputs(seed: int, ntok: int):
    """Inputs of a fused layer step: qf [ntok][16][512] (query | gate per head), kb [ntok][2][256], vb [ntok][512],
    the two RMSNorm weights [256] (close to 1) and per-head sink logits [16]."""
    qf = normal(seed, S_QF, 0, (ntok, 16, 512)) * np.float32(1.5)
    kb = normal(seed, S_KNEW, 1, (ntok, 2, 256)) * np.float32(0.7)
    vb = normal(seed, S_VNEW, 1, (ntok, 512))
    qw = np.float32(1.0) + np.float32(0.1) * normal(seed, S_NORM, 0, (256,))
    kw = np.float32(1.0) + np.float32(0.1) * normal(seed, S_NORM, 1, (256,))
    sinks = normal(seed, S_NORM, 2, (16,)) * np.float32(2.0)
    return qf, kb, vb, qw, kw, sinks
