"""Known answers of the CPU-runnable configuration (tests/golden/config0.npz, made by tests/golden/make_golden.py):
the oracle must reproduce them bit for bit on the CPU; the CUDA path must match them on the GPU (append and
snapshot bit-exact, attention within the tolerance of the cache format)."""
import hashlib
import os

import numpy as np
import pytest

from mechta_b200 import synth

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config0.npz"))
SEED, PRIOR, K = (int(x) for x in G["seed"])
TOL = {0: 2e-3, 1: 1e-5}


def _inputs():
    return (synth.normal(SEED, synth.S_KNEW, 0, (K, 2, 256)), synth.normal(SEED, synth.S_VNEW, 0, (K, 2, 256)),
            synth.normal(SEED, synth.S_Q, 0, (K, 16, 256)))


@pytest.mark.parametrize("fmt,name", [(0, "f16"), (1, "f32")])
def test_oracle_reproduces_golden(oracle, fmt, name):
    kc, vc = oracle.new_cache(fmt, PRIOR + 64), oracle.new_cache(fmt, PRIOR + 64)
    for p in range(0, PRIOR, 1024):
        oracle.append(fmt, kc, vc, p, synth.normal(SEED, synth.S_K, p, (1024, 2, 256)), synth.normal(SEED, synth.S_V, p, (1024, 2, 256)),
                      oracle.rope_tables(p, 1024))
    k, v, q = _inputs()
    tab = oracle.rope_tables(PRIOR, K)
    assert np.array_equal(tab, G["rope_4096"])
    oracle.append(fmt, kc, vc, PRIOR, k, v, tab)
    assert np.array_equal(kc[PRIOR:PRIOR + K], G[f"{name}_new_k"]) and np.array_equal(vc[PRIOR:PRIOR + K], G[f"{name}_new_v"])
    assert hashlib.sha256(kc[:PRIOR].tobytes()).digest() == G[f"{name}_prior_k_sha256"].tobytes()
    # thread scheduling does not change the sums: each block is reduced by one thread, the merge is sequential
    assert np.array_equal(oracle.attn_ref_f32(fmt, kc, vc, 0, PRIOR, q), G[f"{name}_out"])
    assert np.array_equal(oracle.attn_ref_f32(fmt, kc, vc, 1, PRIOR, q[:2]), G[f"{name}_window"])
    assert oracle.max_rel(G[f"{name}_out"], G[f"{name}_out64"]) < 2e-6
    snap = oracle.snapshot(fmt, [kc], [vc], PRIOR + 1)
    assert hashlib.sha256(snap.tobytes()).digest() == G[f"{name}_snap_sha256"].tobytes()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,name", [(0, "f16"), (1, "f32")])
def test_gpu_matches_golden(oracle, fmt, name):
    import torch
    from mechta_b200 import kv
    torch.cuda.set_device(0)
    ctx = kv.KvContext(0, torch.cuda.current_stream())
    cache = kv.KvCache(ctx, kv.KvFormat(fmt), 1, 8192)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for p in range(0, PRIOR, 1024):
        cache.append(0, p, to(synth.normal(SEED, synth.S_K, p, (1024, 2, 256))), to(synth.normal(SEED, synth.S_V, p, (1024, 2, 256))),
                     to(kv.rope_table(p, 1024)))
    k, v, q = _inputs()
    cache.append(0, PRIOR, to(k), to(v), to(G["rope_4096"]))
    out, win = torch.empty(K, 16, 256, device="cuda"), torch.empty(2, 16, 256, device="cuda")
    cache.attn_verify(0, 0, PRIOR, to(q), out)
    cache.attn_verify(0, 1, PRIOR, to(q[:2]), win)
    cache.truncate(PRIOR + 1)  # 3 refused drafts rolled back
    root = cache.read_root(PRIOR + 1)
    ctx.sync()
    gk, gv = cache.buffer_tensors(0)
    view = (lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)) if fmt == 0 else (lambda t: t.cpu().numpy())
    assert np.array_equal(view(gk)[PRIOR:PRIOR + K], G[f"{name}_new_k"]) and np.array_equal(view(gv)[PRIOR:PRIOR + K], G[f"{name}_new_v"])
    assert hashlib.sha256(view(gk)[:PRIOR].tobytes()).digest() == G[f"{name}_prior_k_sha256"].tobytes()
    assert hashlib.sha256(root.payload.numpy().tobytes()).digest() == G[f"{name}_snap_sha256"].tobytes()
    assert oracle.max_rel(out.cpu().numpy(), G[f"{name}_out64"]) < TOL[fmt]
    assert oracle.max_rel(win.cpu().numpy(), G[f"{name}_window"]) < TOL[fmt]
    cache.close()
    ctx.close()


# ---- tests/golden/step.npz: the fused layer step and the ring / window / sinks variant over the same history ----
S = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "step.npz"))
RING, WIN, EPS = 1024, 513, 1e-6


@pytest.mark.parametrize("fmt,name", [(0, "f16"), (1, "f32")])
def test_oracle_reproduces_step_golden(oracle, fmt, name):
    kc, vc = oracle.new_cache(fmt, PRIOR + 64), oracle.new_cache(fmt, PRIOR + 64)
    kr, vr = oracle.new_cache(fmt, RING), oracle.new_cache(fmt, RING)
    for p in range(0, PRIOR, 1024):
        k, v = synth.normal(SEED, synth.S_K, p, (1024, 2, 256)), synth.normal(SEED, synth.S_V, p, (1024, 2, 256))
        tab = oracle.rope_tables(p, 1024)
        oracle.append(fmt, kc, vc, p, k, v, tab)
        oracle.append_ring(fmt, kr, vr, RING, p, k, v, tab)
    qf, kb, vb, qw, kw, sinks = synth.step_inputs(SEED, K)
    tab = oracle.rope_tables(PRIOR, K)
    kn = oracle.rmsnorm(kb, 2 * K, 256, 256, kw, EPS).reshape(K, 2, 256)
    qr = oracle.rope2(oracle.rmsnorm(qf, 16 * K, 256, 512, qw, EPS), 16, tab).reshape(K, 16, 256)
    assert np.array_equal(qr, S[f"{name}_qr"])
    oracle.append(fmt, kc, vc, PRIOR, kn, vb.reshape(K, 2, 256), tab)
    oracle.append_ring(fmt, kr, vr, RING, PRIOR, kn, vb.reshape(K, 2, 256), tab)
    assert np.array_equal(kc[PRIOR:PRIOR + K], S[f"{name}_step_k"]) and np.array_equal(vc[PRIOR:PRIOR + K], S[f"{name}_step_v"])
    assert hashlib.sha256(kr.tobytes()).digest() == S[f"{name}_ring_k_sha256"].tobytes()
    ag = oracle.attn_gate(oracle.attn_ref_f32(fmt, kc, vc, 0, PRIOR, qr), qf)
    assert oracle.max_rel(ag, S[f"{name}_ag"]) < 1e-6  # expf of the C library may differ in the last place between hosts
    assert oracle.max_rel(oracle.attn_window_f64(fmt, kr, vr, RING, WIN, sinks, PRIOR, qr), S[f"{name}_windowed"]) < 1e-12


@pytest.mark.gpu
@pytest.mark.parametrize("fmt,name", [(0, "f16"), (1, "f32")])
def test_gpu_step_matches_golden(oracle, fmt, name):
    import torch
    from mechta_b200 import kv
    torch.cuda.set_device(0)
    ctx = kv.KvContext(0, torch.cuda.current_stream())
    cache = kv.KvCache(ctx, kv.KvFormat(fmt), 1, 8192)
    ring = kv.KvCache(ctx, kv.KvFormat(fmt), 1, 8192, ring=RING)
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for p in range(0, PRIOR, 1024):
        k, v = to(synth.normal(SEED, synth.S_K, p, (1024, 2, 256))), to(synth.normal(SEED, synth.S_V, p, (1024, 2, 256)))
        tab = to(kv.rope_table(p, 1024))
        cache.append(0, p, k, v, tab)
        ring.append(0, p, k, v, tab)
    qf, kb, vb, qw, kw, sinks = synth.step_inputs(SEED, K)
    tab = to(kv.rope_table(PRIOR, K))
    ag = torch.empty(K, 16, 256, device="cuda")
    cache.attn_step(0, 0, PRIOR, to(qf), to(kb), to(vb), to(qw), to(kw), tab, ag, None, EPS)
    # the step's rows into the ring as they are stored (already normalised and rotated: no table)
    stored_k = S[f"{name}_step_k"] if fmt == 1 else S[f"{name}_step_k"].view(np.float16).astype(np.float32)
    ring.append(0, PRIOR, to(stored_k), to(vb.reshape(K, 2, 256)), None)
    win = torch.empty(K, 16, 256, device="cuda")
    ring.attn_verify_window(0, WIN, to(sinks), PRIOR, to(S[f"{name}_qr"]), win)
    ctx.sync()
    view = (lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16)) if fmt == 0 else (lambda t: t.cpu().numpy())
    gk, gv = cache.buffer_tensors(0)
    assert np.array_equal(view(gk)[PRIOR:PRIOR + K], S[f"{name}_step_k"]) and np.array_equal(view(gv)[PRIOR:PRIOR + K], S[f"{name}_step_v"])
    rk, _ = ring.buffer_tensors(0)
    assert hashlib.sha256(view(rk).tobytes()).digest() == S[f"{name}_ring_k_sha256"].tobytes()
    assert oracle.max_rel(ag.cpu().numpy(), S[f"{name}_ag"]) < TOL[fmt]
    assert oracle.max_rel(win.cpu().numpy(), S[f"{name}_windowed"]) < TOL[fmt]
    cache.close()
    ring.close()
    ctx.close()
