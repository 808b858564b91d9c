"""Parity of the CUDA path (through the C ABI) against the CPU oracle. Needs a B200.

Bars: append / truncate / snapshot bit-exact; attention max|a-b|/max|b| <= 2e-3 on the f16 cache and <= 1e-5 on
the f32 cache (the reference's error metric, engine/reference/strato/README.md:6).
"""
import numpy as np
import pytest
import torch

from mechta_b200 import _lib, kv, synth

pytestmark = pytest.mark.gpu

TOL = {kv.KvFormat.F16: 2e-3, kv.KvFormat.F32: 1e-5}
FMTS = [kv.KvFormat.F16, kv.KvFormat.F32]


@pytest.fixture(scope="module")
def ctx():
    assert torch.cuda.is_available(), "these tests need the GPU"
    torch.cuda.set_device(0)
    c = kv.KvContext(0, torch.cuda.current_stream())
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host_bits(cache, layer):
    """K and V of a layer as the oracle's arrays (f16 bit patterns or f32)."""
    k, v = cache.buffer_tensors(layer)
    torch.cuda.synchronize()
    if cache.fmt == kv.KvFormat.F16:
        return k.view(torch.int16).cpu().numpy().view(np.uint16), v.view(torch.int16).cpu().numpy().view(np.uint16)
    return k.cpu().numpy(), v.cpu().numpy()


def fill_both(oracle, cache, layer, rows, seed, first=0, chunk=2048):
    """Appends `rows` seeded rows from `first` to the device cache and to fresh oracle arrays."""
    fmt = int(cache.fmt)
    kc, vc = oracle.new_cache(fmt, cache.capacity), oracle.new_cache(fmt, cache.capacity)
    for p in range(first, first + rows, chunk):
        n = min(chunk, first + rows - p)
        k = synth.normal(seed, synth.S_K, p, (n, 2, 256))
        v = synth.normal(seed, synth.S_V, p, (n, 2, 256))
        tab = kv.rope_table(p, n)
        cache.append(layer, p, dev(k), dev(v), dev(tab))
        oracle.append(fmt, kc, vc, p, k, v, tab)
    return kc, vc


# ---------------------------------------------------------------- append / rollback ----------------------------

@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("ntok", [1, 2, 3, 4, 64, 2048])
def test_append_bit_exact(ctx, oracle, fmt, ntok):
    cache = kv.KvCache(ctx, fmt, 2, 4096)
    pos = 4096 - ntok if ntok > 4 else 1029
    k = synth.normal(21, synth.S_KNEW, ntok, (ntok, 2, 256)) * 4.0
    v = synth.normal(21, synth.S_VNEW, ntok, (ntok, 2, 256)) * 4.0
    k[0, 0, :6] = [70000.0, -70000.0, 1e-7, 6e-8, 2.0**-24, 65519.0]  # overflow, subnormals, ties
    tab = kv.rope_table(pos, ntok)
    with pytest.raises(_lib.MkvError) as e:  # rows [0, pos) were never written: an append there would make them 'valid'
        cache.append(1, pos, dev(k), dev(v), dev(tab))
    assert e.value.status == _lib.ERR_STATE and len(cache) == 0
    cache.set_len(pos)  # the host vouches for the (zero) rows below
    cache.append(1, pos, dev(k), dev(v), dev(tab))
    kc, vc = oracle.new_cache(int(fmt), 4096), oracle.new_cache(int(fmt), 4096)
    oracle.append(int(fmt), kc, vc, pos, k, v, tab)
    gk, gv = host_bits(cache, 1)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    assert len(cache) == pos + ntok
    zk, zv = host_bits(cache, 0)  # the other layer is untouched and zero-initialised
    assert not zk.any() and not zv.any()
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_append_without_table_and_all_layers(ctx, oracle, fmt):
    n_layers, ntok, pos = 3, 4, 200
    cache = kv.KvCache(ctx, fmt, n_layers, 4096)
    k = synth.normal(22, synth.S_KNEW, 0, (n_layers, ntok, 2, 256))
    v = synth.normal(22, synth.S_VNEW, 0, (n_layers, ntok, 2, 256))
    tab = kv.rope_table(pos, ntok)
    cache.set_len(pos)
    cache.append_layers(pos, dev(k), dev(v), dev(tab))
    for l in range(n_layers):
        kc, vc = oracle.new_cache(int(fmt), 4096), oracle.new_cache(int(fmt), 4096)
        oracle.append(int(fmt), kc, vc, pos, k[l], v[l], tab)
        gk, gv = host_bits(cache, l)
        assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    cache.append(0, pos, dev(k[0]), dev(v[0]), None)  # K already rotated
    kc, vc = oracle.new_cache(int(fmt), 4096), oracle.new_cache(int(fmt), 4096)
    oracle.append(int(fmt), kc, vc, pos, k[0], v[0], None)
    gk, _ = host_bits(cache, 0)
    assert np.array_equal(gk, kc)
    cache.close()


def test_capacity_and_argument_errors(ctx):
    for bad in (4000, 1024, 262144 + 1024):
        with pytest.raises(_lib.MkvError) as e:
            kv.KvCache(ctx, kv.KvFormat.F16, 1, bad)
        assert e.value.status == _lib.ERR_INVALID
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, 4096)
    k = torch.zeros(4, 2, 256, device="cuda")
    with pytest.raises(_lib.MkvError) as e:
        cache.append(0, 4093, k, k, None)  # rows 4093..4096 do not fit
    assert e.value.status == _lib.ERR_CAPACITY
    with pytest.raises(_lib.MkvError) as e:
        cache.append(1, 0, k, k, None)
    assert e.value.status == _lib.ERR_INVALID
    q = torch.zeros(4, 16, 256, device="cuda")
    out = torch.empty_like(q)
    with pytest.raises(_lib.MkvError) as e:
        cache.attn_verify(0, 0, 10, q, out)  # nothing appended yet
    assert e.value.status == _lib.ERR_STATE
    cache.append(0, 0, k, k, None)
    with pytest.raises(_lib.MkvError) as e:
        cache.attn_verify(0, 0, 0, torch.zeros(5, 16, 256, device="cuda"), torch.zeros(5, 16, 256, device="cuda"))
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.MkvError) as e:
        cache.truncate(9)
    assert e.value.status == _lib.ERR_STATE
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_truncate_rollback(ctx, oracle, fmt):
    """Rows [0, new_len) unchanged and visible; rows beyond never observed; scrub zeroes them."""
    cache = kv.KvCache(ctx, fmt, 1, 4096)
    pos = 500
    kc, vc = fill_both(oracle, cache, 0, pos + 4, 23)
    q = synth.normal(23, synth.S_Q, 0, (4, 16, 256))
    qd, out = dev(q), torch.empty(4, 16, 256, device="cuda")
    before = host_bits(cache, 0)
    cache.truncate(pos + 2)  # 1 draft accepted, 2 refused
    assert len(cache) == pos + 2
    after = host_bits(cache, 0)
    assert np.array_equal(before[0], after[0]) and np.array_equal(before[1], after[1])  # refused rows stay in memory
    with pytest.raises(_lib.MkvError) as e:
        cache.attn_verify(0, 0, pos, qd, out)  # would read the refused rows
    assert e.value.status == _lib.ERR_STATE
    # the next step starts at the new length and overwrites them
    k2 = synth.normal(24, synth.S_KNEW, 0, (4, 2, 256))
    v2 = synth.normal(24, synth.S_VNEW, 0, (4, 2, 256))
    tab = kv.rope_table(pos + 2, 4)
    cache.append(0, pos + 2, dev(k2), dev(v2), dev(tab))
    oracle.append(int(fmt), kc, vc, pos + 2, k2, v2, tab)
    cache.attn_verify(0, 0, pos + 2, qd, out)
    want = oracle.attn_ref_f32(int(fmt), kc, vc, 0, pos + 2, q)
    assert oracle.max_rel(out.cpu().numpy(), want) < TOL[fmt]
    cache.truncate(pos + 3, scrub=True)
    gk, gv = host_bits(cache, 0)
    assert np.array_equal(gk[:pos + 3], kc[:pos + 3]) and not gk[pos + 3:].any() and not gv[pos + 3:].any()
    cache.close()


# ---------------------------------------------------------------- verify attention ------------------------------

@pytest.mark.parametrize("fmt", FMTS)
def test_config0_verify_step(ctx, oracle, fmt):
    """4,096 prior tokens, append 4, causal verify, roll back 3 (the CPU-runnable configuration)."""
    cache = kv.KvCache(ctx, fmt, 1, 8192)
    pos = 4096
    kc, vc = fill_both(oracle, cache, 0, pos, 31)
    k = synth.normal(31, synth.S_KNEW, 0, (4, 2, 256))
    v = synth.normal(31, synth.S_VNEW, 0, (4, 2, 256))
    q = synth.normal(31, synth.S_Q, 0, (4, 16, 256))
    tab = kv.rope_table(pos, 4)
    cache.append(0, pos, dev(k), dev(v), dev(tab))
    oracle.append(int(fmt), kc, vc, pos, k, v, tab)
    out = torch.empty(4, 16, 256, device="cuda")
    cache.attn_verify(0, 0, pos, dev(q), out)
    cache.truncate(pos + 1)
    ctx.sync()
    gk, gv = host_bits(cache, 0)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    want = oracle.attn_ref_f32(int(fmt), kc, vc, 0, pos, q)
    err = oracle.max_rel(out.cpu().numpy(), want)
    assert err < TOL[fmt], err
    assert len(cache) == pos + 1
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("pos,ntok,first", [(0, 1, 0), (0, 4, 0), (3, 4, 0), (59, 4, 0), (60, 4, 0), (61, 4, 0), (63, 2, 0),
                                            (64, 4, 0), (127, 3, 0), (1000, 4, 0), (1000, 1, 0), (1000, 2, 1), (1000, 4, 333),
                                            (2047, 4, 2040), (4091, 4, 0), (4092, 4, 64)])
def test_verify_edges(ctx, oracle, fmt, pos, ntok, first):
    """Empty prefix, ragged tails around tile edges, windows (the MTP layer's first_pos), end of capacity."""
    cache = kv.KvCache(ctx, fmt, 1, 4096)
    kc, vc = fill_both(oracle, cache, 0, pos + ntok, 41 + pos)
    q = synth.normal(41, synth.S_Q, pos, (ntok, 16, 256))
    out = torch.full((ntok, 16, 256), float("nan"), device="cuda")
    cache.attn_verify(0, first, pos, dev(q), out)
    ctx.sync()
    want = oracle.attn_ref_f32(int(fmt), kc, vc, first, pos, q)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    err = oracle.max_rel(got, want)
    assert err < TOL[fmt], err
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_stale_rows_beyond_the_length_do_not_leak(ctx, oracle, fmt):
    """The tail tile reads rows past the visible range; whatever they hold must not change the result."""
    cache = kv.KvCache(ctx, fmt, 1, 4096)
    pos = 700
    kc, vc = fill_both(oracle, cache, 0, pos + 64, 43)  # 60 rows of 'refused drafts' beyond the step
    cache.truncate(pos)
    k = synth.normal(43, synth.S_KNEW, 0, (4, 2, 256))
    v = synth.normal(43, synth.S_VNEW, 0, (4, 2, 256))
    q = synth.normal(43, synth.S_Q, 0, (4, 16, 256))
    tab = kv.rope_table(pos, 4)
    cache.append(0, pos, dev(k), dev(v), dev(tab))
    oracle.append(int(fmt), kc, vc, pos, k, v, tab)
    out = torch.empty(4, 16, 256, device="cuda")
    cache.attn_verify(0, 0, pos, dev(q), out)
    want = oracle.attn_ref_f32(int(fmt), kc, vc, 0, pos, q)
    assert oracle.max_rel(out.cpu().numpy(), want) < TOL[fmt]
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_verify_is_deterministic(ctx, oracle, fmt):
    cache = kv.KvCache(ctx, fmt, 1, 8192)
    pos = 5000
    fill_both(oracle, cache, 0, pos + 4, 45)
    q = dev(synth.normal(45, synth.S_Q, 0, (4, 16, 256)))
    a, b = torch.empty(4, 16, 256, device="cuda"), torch.empty(4, 16, 256, device="cuda")
    cache.attn_verify(0, 0, pos, q, a)
    cache.attn_verify(0, 0, pos, q, b)
    ctx.sync()
    assert torch.equal(a, b)
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_steady_state_steps_with_random_accepts(ctx, oracle, fmt):
    """The loop of the steady-state configuration, short: append 4, verify, accept 0..3, roll back the rest."""
    n_layers, steps, pos = 2, 12, 1500
    cache = kv.KvCache(ctx, fmt, n_layers, 4096)
    ocs = [fill_both(oracle, cache, l, pos, 50 + l) for l in range(n_layers)]
    acc = synth.accept_counts(51, steps)
    out = torch.empty(4, 16, 256, device="cuda")
    for s in range(steps):
        k = synth.normal(52, synth.S_KNEW, s, (n_layers, 4, 2, 256))
        v = synth.normal(52, synth.S_VNEW, s, (n_layers, 4, 2, 256))
        q = synth.normal(52, synth.S_Q, s, (n_layers, 4, 16, 256))
        tab = kv.rope_table(pos, 4)
        cache.append_layers(pos, dev(k), dev(v), dev(tab))
        for l in range(n_layers):
            oracle.append(int(fmt), ocs[l][0], ocs[l][1], pos, k[l], v[l], tab)
            cache.attn_verify(l, 0, pos, dev(q[l]), out)
            want = oracle.attn_ref_f32(int(fmt), ocs[l][0], ocs[l][1], 0, pos, q[l])
            assert oracle.max_rel(out.cpu().numpy(), want) < TOL[fmt]
        pos += 1 + int(acc[s])
        cache.truncate(pos)
    for l in range(n_layers):
        gk, gv = host_bits(cache, l)
        assert np.array_equal(gk[:pos], ocs[l][0][:pos]) and np.array_equal(gv[:pos], ocs[l][1][:pos])
    cache.close()


@pytest.mark.parametrize("fmt,ctx_len", [(kv.KvFormat.F16, 65536), (kv.KvFormat.F32, 32768), (kv.KvFormat.F32, 131072),
                                         (kv.KvFormat.F32, 261120), (kv.KvFormat.F16, 261120)])
def test_verify_full_size_against_oracle(ctx, oracle, fmt, ctx_len):
    """One layer at the benchmark's context lengths (65,536 tokens; the last rows of a 262,144-token context) against the
    oracle, plus linearity in V."""
    cache = kv.KvCache(ctx, fmt, 1, ctx_len + 1024)
    pos = ctx_len
    kc, vc = fill_both(oracle, cache, 0, pos + 4, 61, chunk=4096)
    q = synth.normal(61, synth.S_Q, 0, (4, 16, 256))
    out = torch.empty(4, 16, 256, device="cuda")
    cache.attn_verify(0, 0, pos, dev(q), out)
    ctx.sync()
    want = oracle.attn_ref_f32(int(fmt), kc, vc, 0, pos, q)
    err = oracle.max_rel(out.cpu().numpy(), want)
    assert err < TOL[fmt], err
    # linearity in V: scaling V by 2 (exact in both formats) scales the output by 2 — bit for bit on the f16
    # cache; on the f32 cache the low halves of the f16 split can be subnormal, so only to f32 rounding
    _, v = cache.buffer_tensors(0)
    v.mul_(2.0)
    out2 = torch.empty_like(out)
    cache.attn_verify(0, 0, pos, dev(q), out2)
    ctx.sync()
    if fmt == kv.KvFormat.F16:
        assert torch.equal(out2, out * 2.0)
    else:
        assert oracle.max_rel(out2.cpu().numpy(), (out * 2.0).cpu().numpy()) < 1e-6
    cache.close()


def test_chained_launches_equal_synchronised_launches(ctx):
    """The benchmark's launch pattern (several layers at 65,536 tokens, append + verify per step, nothing between the
    launches) must give bit for bit what the same launches give one at a time: the kernels overlap their neighbours
    in the stream (early tile loads, L2 prefetch, the merge by the last CTAs), and nothing of that may change a result."""
    n_layers, n, steps = 4, 65536, 6
    cache = kv.KvCache(ctx, kv.KvFormat.F16, n_layers, n + 3072)
    g = torch.Generator(device="cuda"); g.manual_seed(71)
    for l in range(n_layers):
        k, v = cache.buffer_tensors(l)
        k[:n].normal_(generator=g); v[:n].normal_(generator=g)
    q = torch.randn(steps, n_layers, 4, 16, 256, device="cuda", generator=g)
    kn = torch.randn(steps, n_layers, 4, 2, 256, device="cuda", generator=g)
    vn = torch.randn(steps, n_layers, 4, 2, 256, device="cuda", generator=g)
    acc = synth.accept_counts(72, steps)

    cache.set_len(n)
    ctx.sync()

    def run(sync_each):
        cache.truncate(n)
        pos, outs = n, torch.empty(steps, n_layers, 4, 16, 256, device="cuda")
        for s in range(steps):
            cache.append_layers(pos, kn[s], vn[s], dev(kv.rope_table(pos, 4)))
            for l in range(n_layers):
                cache.attn_verify(l, 0, pos, q[s, l], outs[s, l])
                if sync_each:
                    ctx.sync()
            pos += 1 + int(acc[s])
            cache.truncate(pos)
        ctx.sync()
        return outs

    a = run(False)
    b = run(True)
    c = run(False)
    assert torch.isfinite(a).all()
    assert torch.equal(a, b) and torch.equal(a, c)
    cache.close()


# ---------------------------------------------------------------- the step either side of the path ---------------

@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("ntok,first", [(4, 0), (1, 0), (2, 700)])
def test_fused_step_against_the_reference_dispatch_list(ctx, oracle, fmt, ntok, first):
    """mkv_attn_step against the oracle run as the reference's dispatch list (quad.rs:113-125): rmsnorm of q and k
    heads, rope2, kv_rope2 + kv_copy, attention, attn_gate. Cache rows bit for bit; output to the attention bar."""
    pos, eps = 3000, 1e-6
    cache = kv.KvCache(ctx, fmt, 2, 4096)
    kc, vc = fill_both(oracle, cache, 1, pos, 81)
    rng = np.random.default_rng(82 + ntok)
    qf = (rng.standard_normal((ntok, 16, 512)) * 1.5).astype(np.float32)
    kb = (rng.standard_normal((ntok, 2, 256)) * 0.7).astype(np.float32)
    vb = rng.standard_normal((ntok, 512)).astype(np.float32)
    qw = (1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    kw = (1.0 + 0.1 * rng.standard_normal(256)).astype(np.float32)
    tab = kv.rope_table(pos, ntok)
    # the reference's order of operations on the CPU
    qn = oracle.rmsnorm(qf, 16 * ntok, 256, 512, qw, eps)
    kn = oracle.rmsnorm(kb, 2 * ntok, 256, 256, kw, eps)
    qr = oracle.rope2(qn, 16, tab).reshape(ntok, 16, 256)
    oracle.append(int(fmt), kc, vc, pos, kn.reshape(ntok, 2, 256), vb.reshape(ntok, 2, 256), tab)
    att = oracle.attn_ref_f32(int(fmt), kc, vc, first, pos, qr)
    want = oracle.attn_gate(att, qf)

    out = torch.empty(ntok, 16, 256, device="cuda")
    out16 = torch.empty(ntok, 16, 256, device="cuda", dtype=torch.float16)
    n0 = ctx.launches
    cache.attn_step(1, first, pos, dev(qf), dev(kb), dev(vb), dev(qw), dev(kw), dev(tab), out, out16, eps)
    ctx.sync()
    assert ctx.launches - n0 == 2  # nine dispatches of the reference in two launches
    gk, gv = host_bits(cache, 1)
    assert np.array_equal(gk[: pos + ntok], kc[: pos + ntok]) and np.array_equal(gv[: pos + ntok], vc[: pos + ntok])
    assert len(cache) == pos + ntok
    assert oracle.max_rel(out.cpu().numpy(), want) < TOL[fmt]
    assert torch.equal(out16, out.half())
    # the same through the separate operators: append of the normalised keys, then verify, must agree with the fused call
    cache.truncate(pos)
    cache.append(1, pos, dev(kn.reshape(ntok, 2, 256)), dev(vb.reshape(ntok, 2, 256)), dev(tab))
    plain = torch.empty(ntok, 16, 256, device="cuda")
    cache.attn_verify(1, first, pos, dev(qr), plain)
    ctx.sync()
    gated = oracle.attn_gate(plain.cpu().numpy(), qf)
    assert oracle.max_rel(out.cpu().numpy(), gated) < 1e-6
    # only one of the outputs
    only16 = torch.empty_like(out16)
    cache.truncate(pos)
    cache.attn_step(1, first, pos, dev(qf), dev(kb), dev(vb), dev(qw), dev(kw), dev(tab), None, only16, eps)
    ctx.sync()
    assert torch.equal(only16, out16)
    cache.close()


def test_fused_step_argument_errors(ctx):
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, 4096)
    z = lambda *s: torch.zeros(*s, device="cuda")
    args = (z(4, 16, 512), z(4, 2, 256), z(4, 512), z(256), z(256), z(4, 64))
    with pytest.raises(kv.MkvError):  # no output at all
        cache.attn_step(0, 0, 0, *args, None, None)
    with pytest.raises(kv.MkvError):  # a gap before the rows
        cache.attn_step(0, 0, 10, *args, z(4, 16, 256))
    with pytest.raises(kv.MkvError):  # past the context
        cache.attn_step(0, 0, 4094, *args, z(4, 16, 256))
    shard = kv.KvCache(ctx, kv.KvFormat.F16, 1, 8192, 4096, 4096)
    with pytest.raises(kv.MkvError):  # shards have no gate of their own
        shard.attn_step(0, 0, 0, *args, z(4, 16, 256))
    shard.close()
    cache.close()


# ---------------------------------------------------------------- ring rows, window, sinks ---------------------

WTOL = {kv.KvFormat.F16: 2e-3, kv.KvFormat.F32: 1e-5}


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("pos,ntok,win,use_sinks", [(2500, 4, 513, True), (900, 1, 513, False), (5000, 3, 1000, True),
                                                    (600, 4, 0, True), (1023, 4, 513, True)])
def test_ring_cache_window_and_sinks(ctx, oracle, fmt, pos, ntok, win, use_sinks):
    """Rows at position % ring, a sliding window per token and per-head sinks, against the oracle's f64 reference;
    the positions run several times round the ring before the step that is checked."""
    ring = 1024 if win else 1024
    if win == 0 and pos + ntok > ring:
        pytest.skip("without a window the whole history must fit the ring")
    cache = kv.KvCache(ctx, fmt, 2, 8192, ring=ring)
    f = int(fmt)
    kc, vc = oracle.new_cache(f, ring), oracle.new_cache(f, ring)
    for p in range(0, pos, 256):  # the history, through the library's own writer and the oracle's
        n = min(256, pos - p)
        k = synth.normal(91, synth.S_K, p, (n, 2, 256)); v = synth.normal(91, synth.S_V, p, (n, 2, 256))
        tab = kv.rope_table(p, n)
        cache.append(1, p, dev(k), dev(v), dev(tab))
        oracle.append_ring(f, kc, vc, ring, p, k, v, tab)
    k = synth.normal(92, synth.S_KNEW, 0, (ntok, 2, 256)); v = synth.normal(92, synth.S_VNEW, 0, (ntok, 2, 256))
    tab = kv.rope_table(pos, ntok)
    cache.append(1, pos, dev(k), dev(v), dev(tab))
    oracle.append_ring(f, kc, vc, ring, pos, k, v, tab)
    gk, gv = host_bits(cache, 1)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)  # every ring row, bit for bit
    q = synth.normal(92, synth.S_Q, 0, (ntok, 16, 256))
    sinks = (np.linspace(-2.0, 3.0, 16)).astype(np.float32) if use_sinks else None
    out = torch.empty(ntok, 16, 256, device="cuda")
    cache.attn_verify_window(1, win, None if sinks is None else dev(sinks), pos, dev(q), out)
    ctx.sync()
    want = oracle.attn_window_f64(f, kc, vc, ring, win, sinks, pos, q)
    assert oracle.max_rel(out.cpu().numpy(), want) < WTOL[fmt]
    if use_sinks:  # the sinks must matter: without them the result differs
        out2 = torch.empty_like(out)
        cache.attn_verify_window(1, win, None, pos, dev(q), out2)
        ctx.sync()
        assert oracle.max_rel(out2.cpu().numpy(), want) > 2 * WTOL[fmt]
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_window_and_sinks_on_an_ordinary_cache(ctx, oracle, fmt):
    """The same options on a contiguous cache; window 0 and no sinks is the plain verify."""
    pos, ntok = 3000, 4
    cache = kv.KvCache(ctx, fmt, 1, 4096)
    kc, vc = fill_both(oracle, cache, 0, pos + ntok, 95)
    q = synth.normal(95, synth.S_Q, 0, (ntok, 16, 256))
    sinks = np.linspace(1.0, -1.0, 16).astype(np.float32)
    out = torch.empty(ntok, 16, 256, device="cuda")
    for win, sk in ((700, sinks), (0, sinks), (64, None), (1, None)):
        cache.attn_verify_window(0, win, None if sk is None else dev(sk), pos, dev(q), out)
        ctx.sync()
        want = oracle.attn_window_f64(int(fmt), kc, vc, 0, win, sk, pos, q)
        assert oracle.max_rel(out.cpu().numpy(), want) < WTOL[fmt], (win, sk is None)
    plain = torch.empty_like(out)
    cache.attn_verify(0, 0, pos, dev(q), plain)
    cache.attn_verify_window(0, 0, None, pos, dev(q), out)
    ctx.sync()
    assert torch.equal(plain, out)
    cache.close()


def test_ring_cache_limits(ctx):
    with pytest.raises(kv.MkvError):
        kv.KvCache(ctx, kv.KvFormat.F16, 1, 8192, ring=1000)  # not a multiple of 128
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, 8192, ring=1024)
    z = lambda *s: torch.zeros(*s, device="cuda")
    for p in range(0, 2048, 512):
        cache.append(0, p, z(512, 2, 256), z(512, 2, 256), None)
    assert len(cache) == 2048
    with pytest.raises(kv.MkvError):  # 2048 keys do not fit 1024 rows
        cache.attn_verify(0, 0, 2044, z(4, 16, 256), z(4, 16, 256))
    with pytest.raises(kv.MkvError):  # window + step larger than the ring
        cache.attn_verify_window(0, 1022, None, 2044, z(4, 16, 256), z(4, 16, 256))
    cache.attn_verify_window(0, 1021, None, 2044, z(4, 16, 256), z(4, 16, 256))
    with pytest.raises(kv.MkvError):
        cache.attn_prefill(0, 0, 2044, z(4, 16, 256), z(4, 16, 256))
    with pytest.raises(kv.MkvError):
        cache.truncate(2040, scrub=True)
    cache.truncate(2040)
    ctx.sync()
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_fused_step_on_a_ring_cache_that_has_wrapped(ctx, oracle, fmt):
    """mkv_attn_step on a ring cache: once the positions have gone round the ring, a step whose keys no longer fit it is
    refused (and leaves the length alone); one that fits gives the attention over the ring's rows."""
    ring, eps = 1024, 1e-6
    cache = kv.KvCache(ctx, fmt, 1, 8192, ring=ring)
    kc, vc = oracle.new_cache(int(fmt), ring), oracle.new_cache(int(fmt), ring)
    pos = 2500  # two and a half turns
    for p in range(0, pos, 500):
        k = synth.normal(171, synth.S_K, p, (500, 2, 256)); v = synth.normal(171, synth.S_V, p, (500, 2, 256))
        tab = kv.rope_table(p, 500)
        cache.append(0, p, dev(k), dev(v), dev(tab))
        oracle.append_ring(int(fmt), kc, vc, ring, p, k, v, tab)
    ntok = 4
    qf, kb, vb, qw, kw, _ = synth.step_inputs(172, ntok)
    tab = kv.rope_table(pos, ntok)
    out = torch.full((ntok, 16, 256), 5.0, device="cuda")
    with pytest.raises(_lib.MkvError) as e:  # first_pos 0: 2,504 keys do not fit 1,024 rows
        cache.attn_step(0, 0, pos, dev(qf), dev(kb), dev(vb), dev(qw), dev(kw), dev(tab), out, None, eps)
    assert e.value.status == _lib.ERR_CAPACITY and len(cache) == pos
    first = pos + ntok - ring  # the oldest position the ring still holds once the step's rows are in
    cache.attn_step(0, first, pos, dev(qf), dev(kb), dev(vb), dev(qw), dev(kw), dev(tab), out, None, eps)
    ctx.sync()
    assert len(cache) == pos + ntok
    qn = oracle.rmsnorm(qf, 16 * ntok, 256, 512, qw, eps)
    kn = oracle.rmsnorm(kb, 2 * ntok, 256, 256, kw, eps)
    qr = oracle.rope2(qn, 16, tab).reshape(ntok, 16, 256)
    oracle.append_ring(int(fmt), kc, vc, ring, pos, kn.reshape(ntok, 2, 256), vb.reshape(ntok, 2, 256), tab)
    gk, gv = host_bits(cache, 0)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    # token t sees keys first..pos + t: a window of pos + t - first + 1 positions that moves with the token, so compare
    # token by token against the windowed f64 reference
    got = out.cpu().numpy()
    for t in range(ntok):
        want = oracle.attn_window_f64(int(fmt), kc, vc, ring, pos + t - first + 1, None, pos + t, qr[t:t + 1])
        assert oracle.max_rel(got[t:t + 1], oracle.attn_gate(want.astype(np.float32), qf[t:t + 1])) < TOL[fmt]
    cache.close()


# ---------------------------------------------------------------- shards and batches ----------------------------

@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_sequence_shards_on_one_gpu(ctx, oracle, fmt, n_shards):
    """Each shard holds a contiguous range; records merged by combine_shards equal the unsharded result."""
    total, pos, ntok = 8192, 8192 - 4, 4
    per = total // n_shards
    whole = kv.KvCache(ctx, fmt, 1, total)
    kc, vc = fill_both(oracle, whole, 0, total, 71)
    shards = [kv.KvCache(ctx, fmt, 1, total, shard_first=g * per, shard_tokens=per) for g in range(n_shards)]
    for p in range(0, total, 2048):  # every shard sees every append and keeps its own rows
        k = dev(synth.normal(71, synth.S_K, p, (2048, 2, 256)))
        v = dev(synth.normal(71, synth.S_V, p, (2048, 2, 256)))
        tab = dev(kv.rope_table(p, 2048))
        for s in shards:
            s.append(0, p, k, v, tab)
    hk, hv = host_bits(whole, 0)
    for g, s in enumerate(shards):
        gk, gv = host_bits(s, 0)
        assert np.array_equal(gk, hk[g * per:(g + 1) * per]) and np.array_equal(gv, hv[g * per:(g + 1) * per])
    q = synth.normal(71, synth.S_Q, 0, (ntok, 16, 256))
    recs = torch.empty(n_shards, 64, 258, device="cuda")
    for g, s in enumerate(shards):
        s.attn_verify_partial(0, 0, pos, dev(q), recs[g])
    out = torch.empty(ntok, 16, 256, device="cuda")
    ctx.combine_shards(recs, ntok, out)
    ctx.sync()
    want = oracle.attn_ref_f32(int(fmt), kc, vc, 0, pos, q)
    assert oracle.max_rel(out.cpu().numpy(), want) < TOL[fmt]
    # each record against the oracle's shard record (same un-normalised format)
    r = recs.cpu().numpy()
    for g in range(n_shards):
        wr = oracle.attn_shard_partial(int(fmt), kc[g * per:], vc[g * per:], g * per, g * per, (g + 1) * per, 0, pos, q)
        e = np.exp(wr[:, 0] - r[g][:, 0])  # the two may use different reference maxima
        assert np.allclose(r[g][:, 1], wr[:, 1] * e, rtol=TOL[fmt] * 5, atol=0)
    # a window that starts inside shard 1: shard 0 contributes the empty record
    first = per + 100
    for g, s in enumerate(shards):
        s.attn_verify_partial(0, first, pos, dev(q[:2]), recs[g])
    ctx.combine_shards(recs, 2, out[:2])
    ctx.sync()
    r0 = recs[0].cpu().numpy()
    assert (r0[:32, 0] == np.float32(-3.0e38)).all() and not r0[:32, 1:].any()
    want = oracle.attn_ref_f32(int(fmt), kc, vc, first, pos, q[:2])
    assert oracle.max_rel(out[:2].cpu().numpy(), want) < TOL[fmt]
    for s in shards:
        s.close()
    whole.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_ragged_batch_of_sessions(ctx, oracle, fmt):
    """Several sessions of different lengths in one launch pair; each equals its own single call."""
    lens = [64, 1024, 1500, 3000, 4000, 129, 2048]
    caches, ocs, qs, outs, singles = [], [], [], [], []
    for i, n in enumerate(lens):
        c = kv.KvCache(ctx, fmt, 2, 4096)
        ocs.append(fill_both(oracle, c, 1, n + 4, 80 + i))
        caches.append(c)
        ntok = 4 if i % 3 else 2
        q = synth.normal(80 + i, synth.S_Q, 0, (ntok, 16, 256))
        qs.append(q)
        outs.append(torch.empty(ntok, 16, 256, device="cuda"))
        singles.append(torch.empty(ntok, 16, 256, device="cuda"))
    dq = [dev(q) for q in qs]
    ctx.attn_verify_batch([(caches[i], 1, 0, lens[i], dq[i], outs[i]) for i in range(len(lens))])
    for i in range(len(lens)):
        caches[i].attn_verify(1, 0, lens[i], dq[i], singles[i])
    ctx.sync()
    for i in range(len(lens)):
        want = oracle.attn_ref_f32(int(fmt), ocs[i][0], ocs[i][1], 0, lens[i], qs[i])
        assert oracle.max_rel(outs[i].cpu().numpy(), want) < TOL[fmt]
        assert oracle.max_rel(outs[i].cpu().numpy(), singles[i].cpu().numpy()) < TOL[fmt]
    for c in caches:
        c.close()


def test_ragged_batch_at_full_lengths(ctx, oracle):
    """Eight sessions with lengths up to 131,072 (the multi-session configuration's range) in one launch per layer, each
    against the oracle."""
    fmt = kv.KvFormat.F16
    lens = [131072 - 8, 1024, 100000, 65536, 7777, 32768 + 5, 2048, 50001]
    caches, ocs, qs, outs = [], [], [], []
    for i, n in enumerate(lens):
        c = kv.KvCache(ctx, fmt, 1, max(kv.CTX_MIN, min(kv.CTX_MAX, (n + 4 + 1023) // 1024 * 1024 + 1024)))
        ocs.append(fill_both(oracle, c, 0, n + 4, 180 + i, chunk=8192))
        caches.append(c)
        qs.append(synth.normal(180 + i, synth.S_Q, 0, (4, 16, 256)))
        outs.append(torch.full((4, 16, 256), float("nan"), device="cuda"))
    dq = [dev(q) for q in qs]
    ctx.attn_verify_batch([(caches[i], 0, 0, lens[i], dq[i], outs[i]) for i in range(len(lens))])
    ctx.sync()
    for i in range(len(lens)):
        want = oracle.attn_ref_f32(int(fmt), ocs[i][0], ocs[i][1], 0, lens[i], qs[i])
        err = oracle.max_rel(outs[i].cpu().numpy(), want)
        assert err < TOL[fmt], (lens[i], err)
    for c in caches:
        c.close()


# ---------------------------------------------------------------- prefill ------------------------------------

def test_prefix_restore_prefill_snapshot_at_full_size(ctx, oracle):
    """The prefix-cache configuration at its own size: a 32,768-row f16 snapshot is restored, a 2,048-token block is
    appended and attends to the prefix and to itself (544 key tiles for the last tokens), and the 34,816 rows are
    snapshotted back. Order of the reference: write_root (engine.rs:804-823), writers of the whole block, attention
    (engine.rs:1213-1226), read_root (engine.rs:784-802). Attention against the oracle on tokens at the block's ends,
    group borders and middle, with f32 and with f16 queries; the snapshot bytes against the oracle's."""
    fmt = kv.KvFormat.F16
    n_layers, prefix, block = 2, 32768, 2048
    kcs = [oracle.new_cache(int(fmt), prefix + block) for _ in range(n_layers)]
    vcs = [oracle.new_cache(int(fmt), prefix + block) for _ in range(n_layers)]
    for l in range(n_layers):
        for p in range(0, prefix, 8192):
            oracle.append(int(fmt), kcs[l], vcs[l], p, synth.normal(190 + l, synth.S_K, p, (8192, 2, 256)),
                          synth.normal(190 + l, synth.S_V, p, (8192, 2, 256)), kv.rope_table(p, 8192))
    snap = oracle.snapshot(int(fmt), kcs, vcs, prefix)
    cache = kv.KvCache(ctx, fmt, n_layers, prefix + block)
    payload = torch.from_numpy(snap).pin_memory()
    cache.write_root(kv.Root(prefix, fmt, n_layers, payload))
    assert len(cache) == prefix
    kn = synth.normal(192, synth.S_KNEW, 0, (n_layers, block, 2, 256))
    vn = synth.normal(192, synth.S_VNEW, 0, (n_layers, block, 2, 256))
    tab = kv.rope_table(prefix, block)
    cache.append_layers(prefix, dev(kn), dev(vn), dev(tab))
    for l in range(n_layers):
        oracle.append(int(fmt), kcs[l], vcs[l], prefix, kn[l], vn[l], tab)
    toks = [0, 1, 15, 16, 1023, 2046, 2047]
    for l in range(n_layers):
        q = synth.normal(193 + l, synth.S_Q, 0, (block, 16, 256))
        out = torch.full((block, 16, 256), float("nan"), device="cuda")
        cache.attn_prefill(l, 0, prefix, dev(q), out)
        out16 = torch.full((block, 16, 256), float("nan"), device="cuda")
        cache.attn_prefill(l, 0, prefix, dev(q).half(), out16)
        ctx.sync()
        got, got16 = out.cpu().numpy(), out16.cpu().numpy()
        assert np.isfinite(got).all() and np.isfinite(got16).all()
        want = oracle.attn_ref_f32_sel(int(fmt), kcs[l], vcs[l], 0, prefix, toks, q)
        err = oracle.max_rel(got[toks], want)
        assert err < TOL[fmt], err
        # the kernel rounds f32 queries to f16 itself (the reference's q_f16 pass): the f16 input gives the same bits
        assert np.array_equal(got, got16)
    root = cache.read_root(prefix + block)
    assert np.array_equal(root.payload.numpy(), oracle.snapshot(int(fmt), kcs, vcs, prefix + block))
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("prefix,ntok,first", [(0, 64, 0), (0, 17, 0), (100, 8, 0), (1000, 512, 0), (1000, 128, 300),
                                                (2048, 2048, 0), (0, 4096, 0), (700, 3001, 130), (3000, 2400, 2999),
                                                (3000, 512, 0), (7000, 128, 100), (5000, 700, 4990)])
def test_prefill_over_cache(ctx, oracle, fmt, prefix, ntok, first):
    """Token T of the block sees [first, prefix + T]; rows are appended first, as the reference does. Blocks of up to about
    880 tokens over a long enough prefix are the ones the f16 kernel cuts into equal tile ranges over all SMs (items split
    over CTAs and merged); the largest have more work items than the GPU has SMs."""
    cache = kv.KvCache(ctx, fmt, 1, 4096 if prefix + ntok <= 4096 else 8192)
    kc, vc = fill_both(oracle, cache, 0, prefix + ntok, 90 + ntok)
    q = synth.normal(90, synth.S_Q, ntok, (ntok, 16, 256))
    out = torch.full((ntok, 16, 256), float("nan"), device="cuda")
    cache.attn_prefill(0, first, prefix, dev(q), out)
    ctx.sync()
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    toks = (sorted(set([0, 1, 15, 16, 17, ntok // 3, ntok // 2, ntok // 2 + 1, (2 * ntok) // 3, ntok - 17, ntok - 2, ntok - 1])
                   & set(range(ntok))) if ntok > 64 else list(range(ntok)))
    want = oracle.attn_ref_f32_sel(int(fmt), kc, vc, first, prefix, toks, q)
    err = oracle.max_rel(got[toks], want)
    assert err < TOL[fmt], err
    cache.close()


# ---------------------------------------------------------------- snapshot / restore ---------------------------

@pytest.mark.parametrize("fmt", FMTS)
def test_snapshot_restore_bit_exact(ctx, oracle, fmt, tmp_path):
    n_layers, rows, p = 3, 1500, 1300
    a = kv.KvCache(ctx, fmt, n_layers, 4096)
    ocs = [fill_both(oracle, a, l, rows, 100 + l) for l in range(n_layers)]
    root = a.read_root(p)
    want = oracle.snapshot(int(fmt), [o[0] for o in ocs], [o[1] for o in ocs], p)
    assert root.payload.numel() == a.snapshot_bytes(p) == want.size
    assert np.array_equal(root.payload.numpy(), want)  # layout: per layer K rows then V rows (engine.rs:790-795)
    with pytest.raises(_lib.MkvError) as e:
        a.read_root(rows + 1)
    assert e.value.status == _lib.ERR_STATE
    # through a root file into a fresh cache
    toks = np.arange(p, dtype=np.uint32)
    path = str(tmp_path / f"root-{fmt.name.lower()}-{kv.root_key(toks)}.bin")
    kv.write_root_file(path, toks, root)
    t2, r2 = kv.read_root_file(path, fmt, n_layers)
    assert np.array_equal(t2, toks)
    b = kv.KvCache(ctx, fmt, n_layers, 4096)
    b.write_root(r2)
    assert len(b) == p
    for l in range(n_layers):
        gk, gv = host_bits(b, l)
        assert np.array_equal(gk[:p], ocs[l][0][:p]) and np.array_equal(gv[:p], ocs[l][1][:p])
        assert not gk[p:].any() and not gv[p:].any()
    # continuing at pos = p is indistinguishable from having computed the prefix here
    k = synth.normal(105, synth.S_KNEW, 0, (4, 2, 256))
    v = synth.normal(105, synth.S_VNEW, 0, (4, 2, 256))
    q = dev(synth.normal(105, synth.S_Q, 0, (4, 16, 256)))
    tab = dev(kv.rope_table(p, 4))
    oa, ob = torch.empty(4, 16, 256, device="cuda"), torch.empty(4, 16, 256, device="cuda")
    a.truncate(p)
    for c, o in ((a, oa), (b, ob)):
        c.append(2, p, dev(k), dev(v), tab)
        c.attn_verify(2, 0, p, q, o)
    ctx.sync()
    assert torch.equal(oa, ob)
    with pytest.raises(_lib.MkvError) as e:
        b.write_root(kv.Root(p, fmt, n_layers, root.payload[:-2]))
    assert e.value.status == _lib.ERR_FORMAT
    a.close()
    b.close()


def test_snapshot_of_shards_concatenates_to_the_whole(ctx, oracle):
    fmt, total, per = kv.KvFormat.F16, 4096, 1024
    whole = kv.KvCache(ctx, fmt, 1, total)
    fill_both(oracle, whole, 0, 3000, 110)
    shards = [kv.KvCache(ctx, fmt, 1, total, shard_first=g * per, shard_tokens=per) for g in range(4)]
    p = 2500
    hk, hv = host_bits(whole, 0)
    for g, s in enumerate(shards):
        kt, vt = s.buffer_tensors(0)
        wk, wv = whole.buffer_tensors(0)
        kt.copy_(wk[g * per:(g + 1) * per])
        vt.copy_(wv[g * per:(g + 1) * per])
        s.set_len(min(3000, (g + 1) * per))
    rows = 0
    for g, s in enumerate(shards):
        r = s.read_root(p)
        n = max(0, min(p, (g + 1) * per) - g * per)
        assert r.payload.numel() == 2 * n * 512 * 2
        if n:
            got = r.payload.numpy().view(np.uint16).reshape(2, n, 2, 256)
            assert np.array_equal(got[0], hk[g * per:g * per + n]) and np.array_equal(got[1], hv[g * per:g * per + n])
        rows += n
    assert rows == p
    for s in shards:
        s.close()
    whole.close()


# ---------------------------------------------------------------- the reference's dispatch form ---------------

def test_dispatch_with_reference_uniforms(ctx, oracle):
    """kv_rope2 / kv_copy / attn_dmx2 with the uniforms of quad.rs:284-286."""
    import struct
    fmt = kv.KvFormat.F16
    cache = kv.KvCache(ctx, fmt, 1, 4096)
    pos, K = 900, 4
    kc, vc = fill_both(oracle, cache, 0, pos, 120)
    k = synth.normal(120, synth.S_KNEW, 0, (K, 2, 256))
    v = synth.normal(120, synth.S_VNEW, 0, (K, 2, 256))
    q = synth.normal(120, synth.S_Q, 0, (K, 16, 256))
    tab = kv.rope_table(pos, K)
    scale_bits = struct.unpack("<I", struct.pack("<f", 1.0 / 16.0))[0]
    cache.dispatch(0, "kv_rope2", [256, 2 * K, 0, 0, 256, 256, 2, pos * 512], dev(k), dev(tab))
    cache.dispatch(0, "kv_copy", [512 * K, 0, 0, 0, 0, 0, 0, pos * 512], dev(v))
    out = torch.empty(K, 16, 256, device="cuda")
    cache.dispatch(0, "q_dmx", [0, 32, 0, 4, 0, 0, 0, 0])
    cache.dispatch(0, "attn_dmx2", [pos + 1, 2, scale_bits, K, 0, 0, 2048, 0], dev(q), None, out)
    cache.dispatch(0, "attn_fd_combine", [pos + 1, 2, scale_bits, K, 0, 0, 2048, 0])
    ctx.sync()
    oracle.append(int(fmt), kc, vc, pos, k, v, tab)
    gk, gv = host_bits(cache, 0)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    want = oracle.attn_ref_f32(int(fmt), kc, vc, 0, pos, q)
    assert oracle.max_rel(out.cpu().numpy(), want) < TOL[fmt]
    with pytest.raises(_lib.MkvError) as e:
        cache.dispatch(0, "rope2", [256, 8, 0, 0, 256, 256, 2, pos * 512], dev(k), dev(tab))  # the f32 cache's writer
    assert e.value.status == _lib.ERR_INVALID
    with pytest.raises(_lib.MkvError) as e:
        cache.dispatch(0, "delta_q", [0] * 8)
    assert e.value.status == _lib.ERR_UNSUPPORTED
    cache.close()


@pytest.mark.parametrize("fmt", FMTS)
def test_dispatch_of_the_prefill_list(ctx, oracle, fmt):
    """The attention branch of block_n (engine.rs:1213-1241) with the uniforms of inputs_n (engine.rs:915-927): writers of
    the whole block, q_f16 + attn_fa_mx (f16 cache) or attn_fa (f32 cache) per group of 64 tokens and split of chunks with
    the attn_fd_combine after each group; then a block of 8 through attn_fd4."""
    import struct
    scale_bits = struct.unpack("<I", struct.pack("<f", 1.0 / 16.0))[0]
    f16 = fmt == kv.KvFormat.F16
    context, pos, nb = 4096, 1000, 128
    cache = kv.KvCache(ctx, fmt, 1, context)
    kc, vc = fill_both(oracle, cache, 0, pos, 160)
    k = synth.normal(160, synth.S_KNEW, 0, (nb, 2, 256)); v = synth.normal(160, synth.S_VNEW, 0, (nb, 2, 256))
    q = synth.normal(160, synth.S_Q, 0, (nb, 16, 256))
    tab = kv.rope_table(pos, nb)
    cache.dispatch(0, "kv_rope2" if f16 else "rope2", [256, 2 * nb, 0, 0, 256, 256, 2, pos * 512], dev(k), dev(tab))
    assert len(cache) == pos  # the rows count once their V half is written
    cache.dispatch(0, "kv_copy" if f16 else "copy", [nb * 512, 0, 0, 0, 0, 0, 0, pos * 512], dev(v))
    assert len(cache) == pos + nb
    oracle.append(int(fmt), kc, vc, pos, k, v, tab)
    gk, gv = host_bits(cache, 0)
    assert np.array_equal(gk, kc) and np.array_equal(gv, vc)
    att = torch.full((nb, 16, 256), float("nan"), device="cuda")
    qr = dev(q)
    fa_ch, fa_split = 2048, 8
    n_splits = -(-(context // fa_ch) // fa_split)
    if f16:
        qh = torch.empty(nb, 16, 256, device="cuda", dtype=torch.float16)
        cache.dispatch(0, "q_f16", [nb * 2048, 0, 0, 0, 0, 0, 0, 0], qr, None, qh)
        assert torch.equal(qh, qr.half())
    for g in range(nb // 64):
        u0 = None
        for sp in range(n_splits):
            u = [pos + 1, context // fa_ch, scale_bits, 0, g * 64, sp * fa_split, fa_ch, 0]
            u0 = u0 or u
            cache.dispatch(0, "attn_fa_mx" if f16 else "attn_fa", u, qh if f16 else qr, None, att)
        cache.dispatch(0, "attn_fd_combine", u0, None, None, att)
    ctx.sync()
    got = att.cpu().numpy()
    assert np.isfinite(got).all()
    toks = [0, 1, 63, 64, 100, 127]
    assert oracle.max_rel(got[toks], oracle.attn_ref_f32_sel(int(fmt), kc, vc, 0, pos, toks, q)) < TOL[fmt]
    # a block of 8 tokens after it: attn_fd4, one dispatch per 8 tokens (engine.rs:1237-1241, uniform engine.rs:920-922)
    pos2, nb2 = pos + nb, 8
    k2 = synth.normal(161, synth.S_KNEW, 0, (nb2, 2, 256)); v2 = synth.normal(161, synth.S_VNEW, 0, (nb2, 2, 256))
    q2 = synth.normal(161, synth.S_Q, 0, (nb2, 16, 256))
    tab2 = kv.rope_table(pos2, nb2)
    cache.dispatch(0, "kv_rope2" if f16 else "rope2", [256, 2 * nb2, 0, 0, 256, 256, 2, pos2 * 512], dev(k2), dev(tab2))
    cache.dispatch(0, "kv_copy" if f16 else "copy", [nb2 * 512, 0, 0, 0, 0, 0, 0, pos2 * 512], dev(v2))
    oracle.append(int(fmt), kc, vc, pos2, k2, v2, tab2)
    att2 = torch.full((nb2, 16, 256), float("nan"), device="cuda")
    u4 = [pos2 + 1, context // 64, scale_bits, 0, 0, 0, 64, 0]
    cache.dispatch(0, "attn_fd4", u4, dev(q2), None, att2)
    cache.dispatch(0, "attn_fd_combine", u4, None, None, att2)
    ctx.sync()
    want2 = oracle.attn_ref_f32_sel(int(fmt), kc, vc, 0, pos2, list(range(nb2)), q2)
    assert oracle.max_rel(att2.cpu().numpy(), want2) < TOL[fmt]
    # a writer whose rows would leave a gap is refused like mkv_append
    with pytest.raises(_lib.MkvError) as e:
        cache.dispatch(0, "kv_rope2" if f16 else "rope2", [256, 8, 0, 0, 256, 256, 2, (pos2 + 100) * 512], dev(k2), dev(tab2))
    assert e.value.status == _lib.ERR_STATE
    cache.close()


def test_launch_count_and_profiling(ctx, oracle):
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, 4096)
    fill_both(oracle, cache, 0, 1000, 130)
    q = dev(synth.normal(130, synth.S_Q, 0, (4, 16, 256)))
    out = torch.empty(4, 16, 256, device="cuda")
    n0 = ctx.launches
    ctx.prof_enable(True)
    for _ in range(3):
        cache.attn_verify(0, 0, 996, q, out)
    ms, n = ctx.prof_read()
    ctx.prof_enable(False)
    assert n == 3 and 0.0 < ms < 100.0
    assert ctx.launches - n0 == 3  # one kernel per call: the last CTAs merge the pieces
    cache.close()


# ---------------------------------------------------------------- peer exchange ----------------------------------

@pytest.mark.parametrize("fmt", FMTS)
def test_exchange_with_one_rank_equals_plain_verify(ctx, oracle, fmt):
    """world = 1: the record goes through the mailbox and the flag, the result must equal mkv_attn_verify."""
    cache = kv.KvCache(ctx, fmt, 1, 4096)
    kc, vc = fill_both(oracle, cache, 0, 2004, 140)
    ex = kv.KvExchange(ctx, 0, 1)
    for i, (first, pos, ntok) in enumerate([(0, 2000, 4), (50, 1500, 2), (0, 2000, 4)]):
        q = synth.normal(140, synth.S_Q, i, (ntok, 16, 256))
        a, b = torch.empty(ntok, 16, 256, device="cuda"), torch.full((ntok, 16, 256), float("nan"), device="cuda")
        cache.attn_verify(0, first, pos, dev(q), a)
        ex.attn_verify(cache, 0, first, pos, dev(q), b)
        ctx.sync()
        want = oracle.attn_ref_f32(int(fmt), kc, vc, first, pos, q)
        assert oracle.max_rel(b.cpu().numpy(), want) < TOL[fmt]
        assert oracle.max_rel(b.cpu().numpy(), a.cpu().numpy()) < TOL[fmt]
    ex.close()
    cache.close()


def _exchange_rank(rank, world, port, ret):
    import os
    import torch.distributed as dist
    from mechta_b200.sharded import ShardedKvCache
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    st = torch.cuda.Stream()
    total, pos = 8192, 8192 - 4
    with torch.cuda.stream(st):
        c = kv.KvContext(rank, st)
        outs = {}
        for mode in ("p2p", "nccl"):
            sh = ShardedKvCache(c, kv.KvFormat.F16, 1, total, None, exchange=mode)
            for p in range(0, total, 2048):
                k = torch.from_numpy(synth.normal(71, synth.S_K, p, (2048, 2, 256))).cuda()
                v = torch.from_numpy(synth.normal(71, synth.S_V, p, (2048, 2, 256))).cuda()
                sh.append(0, p, k, v, torch.from_numpy(kv.rope_table(p, 2048)).cuda())
            out = torch.empty(4, 16, 256, device="cuda")
            for rep in range(3):  # several calls: the parity slots and epochs are reused
                q = torch.from_numpy(synth.normal(71, synth.S_Q, rep, (4, 16, 256))).cuda()
                sh.attn_verify(0, 0, pos, q, out)
            torch.cuda.synchronize()
            outs[mode] = out.cpu().numpy()
            dist.barrier()
            sh.close()
        c.sync()
    if rank == 0:
        np.savez(ret, **outs)
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_exchange_two_ranks_matches_nccl_and_oracle(oracle, tmp_path):
    import os
    import torch.multiprocessing as mp
    ret = str(tmp_path / "ex.npz")
    mp.spawn(_exchange_rank, args=(2, 29600 + os.getpid() % 300, ret), nprocs=2, join=True)
    got = np.load(ret)
    total, pos = 8192, 8192 - 4
    kc, vc = oracle.new_cache(0, total), oracle.new_cache(0, total)
    for p in range(0, total, 2048):
        oracle.append(0, kc, vc, p, synth.normal(71, synth.S_K, p, (2048, 2, 256)), synth.normal(71, synth.S_V, p, (2048, 2, 256)),
                      kv.rope_table(p, 2048))
    want = oracle.attn_ref_f32(0, kc, vc, 0, pos, synth.normal(71, synth.S_Q, 2, (4, 16, 256)))
    assert oracle.max_rel(got["p2p"], want) < 2e-3 and oracle.max_rel(got["nccl"], want) < 2e-3
    assert oracle.max_rel(got["p2p"], got["nccl"]) < 1e-6


def test_exchange_with_an_absent_rank_times_out_and_the_context_survives(ctx, oracle):
    """Failure made on the host: rank 1 of 2 never joins. The merge's bounded wait runs out (about two seconds), the
    status is reported by sync, nothing hangs, and the context keeps working."""
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, 4096)
    kc, vc = fill_both(oracle, cache, 0, 1004, 150)
    ex = kv.KvExchange(ctx, 0, 2, gather_handles=lambda mine: [mine, None])
    q = synth.normal(150, synth.S_Q, 0, (4, 16, 256))
    out = torch.full((4, 16, 256), 7.0, device="cuda")
    ex.attn_verify(cache, 0, 0, 1000, dev(q), out)
    with pytest.raises(_lib.MkvError) as e:
        ctx.sync()
    assert e.value.status == _lib.ERR_CUDA and "wait ran out" in str(e.value)
    assert bool((out == 7.0).all())  # the merge did not run on incomplete data
    cache.attn_verify(0, 0, 1000, dev(q), out)  # the context is still usable
    ctx.sync()
    want = oracle.attn_ref_f32(0, kc, vc, 0, 1000, q)
    assert oracle.max_rel(out.cpu().numpy(), want) < 2e-3
    ex.close()
    cache.close()
