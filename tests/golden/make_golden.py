"""Generates tests/golden/config0.npz: known answers for the CPU-runnable configuration (one full-attention layer, f16
cache of 4,096 prior tokens, a 4-token verify step with append and rollback),
and tests/golden/step.npz: the fused layer step and the ring / window / sinks variant on the same prior cache.

The reference cannot run where this was written (Rust + wgpu/Vulkan; no graphics stack), and it holds no fixture
for this path, so these vectors come from the CPU oracle (oracle/mkv_oracle.c) — they pin the oracle against
regressions and give the GPU tests a fixed target that does not depend on the oracle being rebuilt.
Inputs are regenerated from seeds (mechta_b200/synth.py); only outputs are stored.

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from mechta_b200 import synth  # noqa: E402
from oracle import oracle  # noqa: E402

SEED, PRIOR, K = 2024, 4096, 4


def build(fmt):
    kc, vc = oracle.new_cache(fmt, PRIOR + 64), oracle.new_cache(fmt, PRIOR + 64)
    for p in range(0, PRIOR, 1024):
        oracle.append(fmt, kc, vc, p, synth.normal(SEED, synth.S_K, p, (1024, 2, 256)), synth.normal(SEED, synth.S_V, p, (1024, 2, 256)),
                      oracle.rope_tables(p, 1024))
    k = synth.normal(SEED, synth.S_KNEW, 0, (K, 2, 256))
    v = synth.normal(SEED, synth.S_VNEW, 0, (K, 2, 256))
    q = synth.normal(SEED, synth.S_Q, 0, (K, 16, 256))
    tab = oracle.rope_tables(PRIOR, K)
    oracle.append(fmt, kc, vc, PRIOR, k, v, tab)
    out = oracle.attn_ref_f32(fmt, kc, vc, 0, PRIOR, q)
    out64 = oracle.attn_ref_f64(fmt, kc, vc, 0, PRIOR, q)
    window = oracle.attn_ref_f32(fmt, kc, vc, 1, PRIOR, q[:2])  # the MTP layer's window (first_pos = 1), 2 tokens
    snap = oracle.snapshot(fmt, [kc], [vc], PRIOR + 1)          # after rolling back 3 refused drafts
    return dict(new_k=kc[PRIOR:PRIOR + K].copy(), new_v=vc[PRIOR:PRIOR + K].copy(), out=out, out64=out64.astype(np.float64),
                window=window, snap_sha256=np.frombuffer(hashlib.sha256(snap.tobytes()).digest(), np.uint8),
                prior_k_sha256=np.frombuffer(hashlib.sha256(kc[:PRIOR].tobytes()).digest(), np.uint8))


def build_step(fmt):
    """The layer step of quad.rs:113-125 at position PRIOR over config 0's cache, and a windowed step with sinks on a
    ring of 1,024 rows holding the same history (window 513 as flint.rs:22)."""
    eps, ring, win = 1e-6, 1024, 513
    kc, vc = oracle.new_cache(fmt, PRIOR + 64), oracle.new_cache(fmt, PRIOR + 64)
    kr, vr = oracle.new_cache(fmt, ring), oracle.new_cache(fmt, ring)
    for p in range(0, PRIOR, 1024):
        k, v = synth.normal(SEED, synth.S_K, p, (1024, 2, 256)), synth.normal(SEED, synth.S_V, p, (1024, 2, 256))
        tab = oracle.rope_tables(p, 1024)
        oracle.append(fmt, kc, vc, p, k, v, tab)
        oracle.append_ring(fmt, kr, vr, ring, p, k, v, tab)
    qf, kb, vb, qw, kw, sinks = synth.step_inputs(SEED, K)
    tab = oracle.rope_tables(PRIOR, K)
    qn = oracle.rmsnorm(qf, 16 * K, 256, 512, qw, eps)
    kn = oracle.rmsnorm(kb, 2 * K, 256, 256, kw, eps)
    qr = oracle.rope2(qn, 16, tab).reshape(K, 16, 256)
    oracle.append(fmt, kc, vc, PRIOR, kn.reshape(K, 2, 256), vb.reshape(K, 2, 256), tab)
    oracle.append_ring(fmt, kr, vr, ring, PRIOR, kn.reshape(K, 2, 256), vb.reshape(K, 2, 256), tab)
    ag = oracle.attn_gate(oracle.attn_ref_f32(fmt, kc, vc, 0, PRIOR, qr), qf)
    windowed = oracle.attn_window_f64(fmt, kr, vr, ring, win, sinks, PRIOR, qr)
    return dict(step_k=kc[PRIOR:PRIOR + K].copy(), step_v=vc[PRIOR:PRIOR + K].copy(), qr=qr, ag=ag, windowed=windowed,
                ring_k_sha256=np.frombuffer(hashlib.sha256(kr.tobytes()).digest(), np.uint8))


def main():
    data = {"rope_4096": oracle.rope_tables(PRIOR, K), "seed": np.array([SEED, PRIOR, K])}
    for fmt, name in ((0, "f16"), (1, "f32")):
        for key, val in build(fmt).items():
            data[f"{name}_{key}"] = val
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "config0.npz"), **data)
    print("wrote config0.npz:", {k: v.shape for k, v in data.items()})
    step = {"seed": np.array([SEED, PRIOR, K])}
    for fmt, name in ((0, "f16"), (1, "f32")):
        for key, val in build_step(fmt).items():
            step[f"{name}_{key}"] = val
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "step.npz"), **step)
    print("wrote step.npz:", {k: v.shape for k, v in step.items()})


if __name__ == "__main__":
    main()
