"""ctypes front end of the CPU oracle (oracle/mkv_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke run and by the CPU-baseline leg of the benchmark.
The product path (mechta_b200) never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libmkv_oracle.so")
F16, F32 = 0, 1
REC = 258
NEG_BIG = np.float32(-3.0e38)


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (gcc, OpenMP, -ffp-contract=off)."""
    src = os.path.join(_HERE, "mkv_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libmkv_oracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        vp, u32, i32, u64, sz = C.c_void_p, C.c_uint32, C.c_int, C.c_uint64, C.c_size_t
        L.mko_rope_table.argtypes = [C.c_int32, vp]
        L.mko_f32_to_f16.argtypes = [C.c_float]; L.mko_f32_to_f16.restype = C.c_uint16
        L.mko_f16_to_f32.argtypes = [C.c_uint16]; L.mko_f16_to_f32.restype = C.c_float
        L.mko_f32_to_f16_n.argtypes = [vp, vp, sz]
        L.mko_buffer_bytes_for.argtypes = [i32, u64]; L.mko_buffer_bytes_for.restype = u64
        L.mko_need_bytes_kv.argtypes = [u64, i32, u64]; L.mko_need_bytes_kv.restype = u64
        L.mko_append_k.argtypes = [i32, vp, u32, u32, vp, vp]
        L.mko_append_v.argtypes = [i32, vp, u32, u32, vp]
        L.mko_attn_fd.argtypes = [i32, vp, vp, u32, u32, u32, vp, vp, u32]
        L.mko_attn_fd_combine.argtypes = [vp, u32, u32, u32, u32, u32, vp]
        L.mko_attn_ref_f32.argtypes = [i32, vp, vp, u32, u32, u32, vp, vp]; L.mko_attn_ref_f32.restype = i32
        L.mko_attn_ref_f64.argtypes = [i32, vp, vp, u32, u32, u32, vp, vp]
        L.mko_attn_ref_f32_sel.argtypes = [i32, vp, vp, u32, u32, vp, u32, vp, vp]; L.mko_attn_ref_f32_sel.restype = i32
        L.mko_attn_shard_partial.argtypes = [i32, vp, vp, u32, u32, u32, u32, u32, u32, vp, vp]
        L.mko_attn_shard_partial.restype = i32
        L.mko_combine_shards.argtypes = [vp, u32, u32, vp]
        L.mko_attn_dmx_emul.argtypes = [vp, vp, u32, u32, u32, vp, vp]; L.mko_attn_dmx_emul.restype = i32
        L.mko_snapshot.argtypes = [i32, vp, vp, u32, u32, vp]; L.mko_snapshot.restype = sz
        L.mko_restore.argtypes = [i32, vp, vp, u32, u32, vp]; L.mko_restore.restype = sz
        L.mko_root_key.argtypes = [vp, sz]; L.mko_root_key.restype = u64
        L.mko_rmsnorm.argtypes = [vp, u32, u32, u32, vp, C.c_float, vp]
        L.mko_rope2.argtypes = [vp, u32, u32, vp, vp]
        L.mko_attn_gate.argtypes = [vp, vp, u32, vp]
        L.mko_attn_window_f64.argtypes = [i32, vp, vp, u32, u32, vp, u32, u32, vp, vp]
        L.mko_threads.restype = i32
        L.mko_set_threads.argtypes = [i32]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def cache_dtype(fmt: int):
    return np.float32 if fmt == F32 else np.uint16


def new_cache(fmt: int, rows: int) -> np.ndarray:
    """One K or V buffer of `rows` positions, zeroed: [rows][2][256] of f32 or of f16 bit patterns."""
    return np.zeros((rows, 2, 256), dtype=cache_dtype(fmt))


def rope_table(pos: int) -> np.ndarray:
    out = np.empty(64, np.float32)
    lib().mko_rope_table(int(pos), _p(out))
    return out


def rope_tables(pos: int, ntok: int) -> np.ndarray:
    return np.stack([rope_table(pos + t) for t in range(ntok)])


def f32_to_f16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    h = np.empty(x.shape, np.uint16)
    lib().mko_f32_to_f16_n(_p(x), _p(h), x.size)
    return h


def append(fmt, kc, vc, pos, k, v, tab):
    """k = [ntok][2][256] f32, v = [ntok][2][256] f32, tab = [ntok][64] f32 or None."""
    k = np.ascontiguousarray(k, np.float32); v = np.ascontiguousarray(v, np.float32)
    ntok = k.shape[0]
    if pos < 0 or pos + ntok > kc.shape[0] or pos + ntok > vc.shape[0]:
        raise ValueError(f"rows [{pos}, {pos + ntok}) do not fit a cache of {min(kc.shape[0], vc.shape[0])} rows")
    t = None if tab is None else _p(np.ascontiguousarray(tab, np.float32))
    lib().mko_append_k(fmt, _p(kc), pos, ntok, _p(k), t)
    lib().mko_append_v(fmt, _p(vc), pos, ntok, _p(v))


def attn_ref_f32(fmt, kc, vc, first_pos, pos, q) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    ntok = q.shape[0]
    out = np.empty((ntok, 16, 256), np.float32)
    rc = lib().mko_attn_ref_f32(fmt, _p(kc), _p(vc), first_pos, pos, ntok, _p(q), _p(out))
    assert rc == 0
    return out


def attn_ref_f64(fmt, kc, vc, first_pos, pos, q) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    ntok = q.shape[0]
    out = np.empty((ntok, 16, 256), np.float64)
    lib().mko_attn_ref_f64(fmt, _p(kc), _p(vc), first_pos, pos, ntok, _p(q), _p(out))
    return out


def attn_ref_f32_sel(fmt, kc, vc, first_pos, pos, toks, q) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    toks = np.ascontiguousarray(toks, np.uint32)
    out = np.empty((toks.size, 16, 256), np.float32)
    rc = lib().mko_attn_ref_f32_sel(fmt, _p(kc), _p(vc), first_pos, pos, _p(toks), toks.size, _p(q), _p(out))
    assert rc == 0
    return out


def attn_shard_partial(fmt, kc, vc, cache_first_pos, lo, hi, first_pos, pos, q) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    ntok = q.shape[0]
    rec = np.empty((64, REC), np.float32)
    lib().mko_attn_shard_partial(fmt, _p(kc), _p(vc), cache_first_pos, lo, hi, first_pos, pos, ntok, _p(q), _p(rec))
    return rec


def combine_shards(recs: np.ndarray) -> np.ndarray:
    recs = np.ascontiguousarray(recs, np.float32)
    g, nrow, _ = recs.shape
    out = np.empty((nrow, 256), np.float32)
    lib().mko_combine_shards(_p(recs), g, nrow, _p(out))
    return out


def attn_dmx_emul(kc, vc, pos, q, chunk=2048) -> np.ndarray:
    q = np.ascontiguousarray(q, np.float32)
    ntok = q.shape[0]
    out = np.empty((ntok, 16, 256), np.float32)
    rc = lib().mko_attn_dmx_emul(_p(kc), _p(vc), pos, ntok, chunk, _p(q), _p(out))
    assert rc == 0
    return out


def snapshot(fmt, kcs, vcs, p) -> np.ndarray:
    n = len(kcs)
    nbytes = 2 * n * p * 512 * (4 if fmt == F32 else 2)
    dst = np.empty(nbytes, np.uint8)
    ka = (C.c_void_p * n)(*[k.ctypes.data for k in kcs])
    va = (C.c_void_p * n)(*[v.ctypes.data for v in vcs])
    w = lib().mko_snapshot(fmt, ka, va, n, p, _p(dst))
    assert w == nbytes
    return dst


def restore(fmt, kcs, vcs, p, src: np.ndarray) -> None:
    n = len(kcs)
    ka = (C.c_void_p * n)(*[k.ctypes.data for k in kcs])
    va = (C.c_void_p * n)(*[v.ctypes.data for v in vcs])
    r = lib().mko_restore(fmt, ka, va, n, p, _p(np.ascontiguousarray(src, np.uint8)))
    assert r == src.size


def rmsnorm(x: np.ndarray, rows: int, n: int, step_x: int, w: np.ndarray, eps: float) -> np.ndarray:
    """Rows of n values at stride step_x of the flat f32 array x, normalised and weighted (W/ops.wgsl:27-56)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1); w = np.ascontiguousarray(w, dtype=np.float32)
    y = np.empty((rows, n), dtype=np.float32)
    lib().mko_rmsnorm(_p(x), rows, n, step_x, _p(w), float(eps), _p(y))
    return y


def rope2(x: np.ndarray, rows_per_tok: int, tab: np.ndarray) -> np.ndarray:
    """Rows of 256 values, dims 0..63 rotated with the table of token row // rows_per_tok (W/ops.wgsl:275-286)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 256); tab = np.ascontiguousarray(tab, dtype=np.float32)
    y = np.empty_like(x)
    lib().mko_rope2(_p(x), x.shape[0], rows_per_tok, _p(tab), _p(y))
    return y


def attn_gate(att: np.ndarray, qf: np.ndarray) -> np.ndarray:
    """att [ntok][16][256] times the sigmoid of the gate half of qf [ntok][16][512] (W/ops.wgsl:171-177)."""
    att = np.ascontiguousarray(att, dtype=np.float32); qf = np.ascontiguousarray(qf, dtype=np.float32)
    out = np.empty_like(att)
    lib().mko_attn_gate(_p(att), _p(qf), att.shape[0], _p(out))
    return out


def append_ring(fmt, kc, vc, ring, pos, k, v, tab):
    """Rows pos.. of a step into a ring cache: row = position % ring (flint_attn.wgsl:54), one row at a time."""
    k = np.ascontiguousarray(k, dtype=np.float32); v = np.ascontiguousarray(v, dtype=np.float32)
    for t in range(k.shape[0]):
        append(fmt, kc, vc, (pos + t) % ring, k[t:t + 1], v[t:t + 1], None if tab is None else tab[t:t + 1])


def attn_window_f64(fmt, kc, vc, ring, win, sinks, pos, q) -> np.ndarray:
    """Attention with ring rows, a sliding window and per-head sinks, accumulated in f64."""
    q = np.ascontiguousarray(q, dtype=np.float32)
    out = np.empty(q.shape, dtype=np.float64)
    sk = None if sinks is None else np.ascontiguousarray(sinks, dtype=np.float32)
    lib().mko_attn_window_f64(fmt, _p(kc), _p(vc), ring, win, None if sk is None else _p(sk), pos, q.shape[0], _p(q), _p(out))
    return out


def root_key(tokens) -> int:
    t = np.ascontiguousarray(tokens, np.uint32)
    return int(lib().mko_root_key(_p(t), t.size))


def threads() -> int:
    return int(lib().mko_threads())


def use_all_cores() -> int:
    """Sets the OpenMP thread count to the cores this process may run on (a launcher may have exported
    OMP_NUM_THREADS=1) and returns it."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().mko_set_threads(int(n))
    return threads()


def max_rel(a: np.ndarray, b: np.ndarray) -> float:
    """The reference's error metric, max|a-b| / max|b| (engine/reference/strato/README.md:6)."""
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / np.max(np.abs(b)))
