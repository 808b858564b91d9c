"""The CPU oracle against what can be pinned without the reference running: numpy float16 for the RTE
conversion, a numpy restatement of the K writer, its own f64 arbiter, and the sizes the reference's tests hold."""
import numpy as np
import pytest

from mechta_b200 import synth


def test_f16_rte_matches_numpy_on_random_bit_patterns(oracle):
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 2**32, size=2_000_000, dtype=np.uint64).astype(np.uint32)
    x = bits.view(np.float32)
    x = x[~np.isnan(x)]
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = oracle.f32_to_f16(x)
    assert np.array_equal(got, want)


def test_f16_rte_boundaries(oracle):
    cases = np.array([0.0, -0.0, 65504.0, 65519.99, 65520.0, 1e9, -1e9, np.inf, -np.inf, 2.0**-24, 2.0**-25,
                      np.nextafter(np.float32(2.0**-25), np.float32(1)), 2.0**-14, 2.0**-14 - 2.0**-26, 1.0 + 2.0**-11,
                      1.0 + 2.0**-11 + 2.0**-20, 1.0 + 3 * 2.0**-11, 5.9604645e-08, 6.1035156e-05, 0.1, -0.3, 1e-10],
                     np.float32)
    with np.errstate(over="ignore"):
        want = cases.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16(cases), want)
    # every half value survives a round trip
    allh = np.arange(0, 0x7c01, dtype=np.uint16)
    back = oracle.f32_to_f16(allh.view(np.float16).astype(np.float32))
    assert np.array_equal(back, allh)
    assert np.isnan(np.array([oracle.lib().mko_f16_to_f32(int(oracle.lib().mko_f32_to_f16(float("nan"))))]))[0]


def test_f16_to_f32_all_values(oracle):
    allh = np.arange(0, 0x10000, dtype=np.uint32).astype(np.uint16)
    want = allh.view(np.float16).astype(np.float32)
    got = np.array([oracle.lib().mko_f16_to_f32(int(h)) for h in allh[::7]], np.float32)
    w = want[::7]
    ok = (got == w) | (np.isnan(got) & np.isnan(w))
    assert ok.all()


def test_rope_table(oracle):
    t0 = oracle.rope_table(0)
    assert np.array_equal(t0[:32], np.ones(32, np.float32)) and np.array_equal(t0[32:], np.zeros(32, np.float32))
    # the iterative theta of engine.rs:108-114, restated in numpy f32
    pos = 4097
    scale = np.float32(np.float32(1e7) ** np.float32(-2.0 / 64.0))
    th = np.float32(pos)
    for i in range(32):
        t = oracle.rope_table(pos)
        assert abs(t[i] - np.cos(np.float64(th))) < 2e-7 and abs(t[32 + i] - np.sin(np.float64(th))) < 2e-7
        th = np.float32(th * scale)


def _append_numpy(fmt, k, v, tab):
    """kv.wgsl:13-28 in numpy f32 (separate roundings of products and sums)."""
    k = k.astype(np.float32).copy()
    out = k.copy()
    for t in range(k.shape[0]):
        c, s = tab[t, :32], tab[t, 32:]
        a, b = k[t, :, :32], k[t, :, 32:64]
        out[t, :, :32] = (a * c).astype(np.float32) - (b * s).astype(np.float32)
        out[t, :, 32:64] = (a * s).astype(np.float32) + (b * c).astype(np.float32)
    if fmt == 0:
        with np.errstate(over="ignore"):
            return out.astype(np.float16).view(np.uint16), v.astype(np.float16).view(np.uint16)
    return out, v.astype(np.float32)


@pytest.mark.parametrize("fmt", [0, 1])
def test_append_matches_numpy(oracle, fmt):
    ntok, pos = 4, 37
    k = synth.normal(3, synth.S_KNEW, 0, (ntok, 2, 256)) * 3.0
    v = synth.normal(3, synth.S_VNEW, 0, (ntok, 2, 256)) * 3.0
    tab = oracle.rope_tables(pos, ntok)
    kc, vc = oracle.new_cache(fmt, 64), oracle.new_cache(fmt, 64)
    oracle.append(fmt, kc, vc, pos, k, v, tab)
    wk, wv = _append_numpy(fmt, k, v, tab)
    assert np.array_equal(kc[pos:pos + ntok], wk) and np.array_equal(vc[pos:pos + ntok], wv)
    assert not kc[:pos].any() and not kc[pos + ntok:].any() and not vc[:pos].any() and not vc[pos + ntok:].any()
    # no table: K copied as is
    kc2, vc2 = oracle.new_cache(fmt, 64), oracle.new_cache(fmt, 64)
    oracle.append(fmt, kc2, vc2, pos, k, v, None)
    wk2, _ = _append_numpy(fmt, k, v, np.tile(np.concatenate([np.ones(32), np.zeros(32)]).astype(np.float32), (ntok, 1)))
    assert np.array_equal(kc2[pos:pos + ntok], wk2)


def _filled(oracle, fmt, rows, seed):
    kc, vc = oracle.new_cache(fmt, rows + 64), oracle.new_cache(fmt, rows + 64)
    step = 256
    for p in range(0, rows, step):
        n = min(step, rows - p)
        oracle.append(fmt, kc, vc, p, synth.normal(seed, synth.S_K, p, (n, 2, 256)), synth.normal(seed, synth.S_V, p, (n, 2, 256)),
                      oracle.rope_tables(p, n))
    return kc, vc


@pytest.mark.parametrize("fmt,tol", [(0, 2e-6), (1, 2e-6)])
def test_attn_f32_against_f64_arbiter(oracle, fmt, tol):
    pos = 1000
    kc, vc = _filled(oracle, fmt, pos + 4, 5)
    q = synth.normal(5, synth.S_Q, 0, (4, 16, 256))
    a = oracle.attn_ref_f32(fmt, kc, vc, 0, pos, q)
    b = oracle.attn_ref_f64(fmt, kc, vc, 0, pos, q)
    assert oracle.max_rel(a, b) < tol
    # a window that does not start at 0 (the MTP layer's first_pos, quad.rs:295)
    a = oracle.attn_ref_f32(fmt, kc, vc, 130, pos, q[:2])
    b = oracle.attn_ref_f64(fmt, kc, vc, 130, pos, q[:2])
    assert oracle.max_rel(a, b) < tol


def test_visibility_is_causal_inside_the_step(oracle):
    """Token t sees keys < pos + 1 + t: changing the row at pos + 2 must not move tokens 0 and 1."""
    pos = 300
    kc, vc = _filled(oracle, 1, pos + 4, 7)
    q = synth.normal(7, synth.S_Q, 0, (4, 16, 256))
    a = oracle.attn_ref_f32(1, kc, vc, 0, pos, q)
    vc[pos + 2] += 5.0
    b = oracle.attn_ref_f32(1, kc, vc, 0, pos, q)
    assert np.array_equal(a[:2], b[:2]) and not np.array_equal(a[2], b[2]) and not np.array_equal(a[3], b[3])


def test_token_t_equals_single_token_call(oracle):
    pos = 777
    kc, vc = _filled(oracle, 0, pos + 4, 9)
    q = synth.normal(9, synth.S_Q, 0, (4, 16, 256))
    a = oracle.attn_ref_f32(0, kc, vc, 0, pos, q)
    sel = oracle.attn_ref_f32_sel(0, kc, vc, 0, pos, [3, 1], q)
    assert np.array_equal(sel[0], a[3]) and np.array_equal(sel[1], a[1])


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("n_shards", [2, 4, 8])
def test_sharded_combine_equals_unsharded(oracle, fmt, n_shards):
    total = 2048
    pos = total - 4
    kc, vc = _filled(oracle, fmt, total, 11)
    q = synth.normal(11, synth.S_Q, 0, (4, 16, 256))
    want = oracle.attn_ref_f32(fmt, kc, vc, 0, pos, q)
    per = total // n_shards
    recs = np.stack([oracle.attn_shard_partial(fmt, kc[g * per:], vc[g * per:], g * per, g * per, (g + 1) * per, 0, pos, q)
                     for g in range(n_shards)])
    got = oracle.combine_shards(recs).reshape(4, 16, 256)
    assert oracle.max_rel(got, want) < 2e-6
    # a shard that sees nothing contributes the empty record
    empty = oracle.attn_shard_partial(fmt, kc, vc, 0, 0, per, per, pos, q)
    assert (empty[:, 0] == np.float32(-3.0e38)).all() and not empty[:, 1:].any()


def test_dmx_emulation_within_f16_tolerance(oracle):
    """The reference's production f16 path (dmx.rs: Q and P in f16, lazy max) against its f32 path."""
    pos = 4096
    kc, vc = _filled(oracle, 0, pos + 4, 13)
    q = synth.normal(13, synth.S_Q, 0, (4, 16, 256))
    a = oracle.attn_dmx_emul(kc, vc, pos, q)
    b = oracle.attn_ref_f32(0, kc, vc, 0, pos, q)
    assert oracle.max_rel(a, b) < 2e-3


def test_sizes_pinned_by_the_reference(oracle):
    L = oracle.lib()
    # memcheck.rs:111
    assert 2 * 11 * L.mko_buffer_bytes_for(1, 65536) == 2_952_790_016
    assert L.mko_buffer_bytes_for(0, 65536) * 2 == L.mko_buffer_bytes_for(1, 65536)
    # memcheck.rs:15-18 with 11 KV layers
    ctx = 131072
    partials = 4 * 258 * 16 * (2 * (ctx // 128) + max(8 * (ctx // 64), 64 * (ctx // 2048)))
    assert L.mko_need_bytes_kv(ctx, 0, 11) == 2 * 11 * 4 * (ctx * 512 // 2) + partials
    # model.md:34: 20 KB per token in f16 over 10 layers
    assert 10 * 2 * 512 * 2 == 20480


def test_root_key_is_fnv1a64(oracle):
    def fnv(data: bytes) -> int:
        h = 0xCBF29CE484222325
        for b in data:
            h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
        return h
    assert fnv(b"") == 0xCBF29CE484222325 and fnv(b"a") == 0xAF63DC4C8601EC8C  # published FNV-1a vectors
    toks = np.array([1, 2, 3, 151643, 4_000_000_000], np.uint32)
    assert oracle.root_key(toks) == fnv(toks.tobytes())
    assert oracle.root_key(np.zeros(0, np.uint32)) == 0xCBF29CE484222325


@pytest.mark.parametrize("fmt", [0, 1])
def test_snapshot_roundtrip_and_layout(oracle, fmt):
    n_layers, p, rows = 3, 100, 128
    kcs = [oracle.new_cache(fmt, rows) for _ in range(n_layers)]
    vcs = [oracle.new_cache(fmt, rows) for _ in range(n_layers)]
    for l in range(n_layers):
        oracle.append(fmt, kcs[l], vcs[l], 0, synth.normal(17, synth.S_K, l, (rows, 2, 256)),
                      synth.normal(17, synth.S_V, l, (rows, 2, 256)), None)
    snap = oracle.snapshot(fmt, kcs, vcs, p)
    eb = 2 if fmt == 0 else 4
    per = p * 512 * eb
    assert snap.size == 2 * n_layers * per
    # K of layer 1 starts after K and V of layer 0 (engine.rs:790-795)
    assert np.array_equal(snap[2 * per:3 * per], kcs[1][:p].view(np.uint8).reshape(-1))
    assert np.array_equal(snap[3 * per:4 * per], vcs[1][:p].view(np.uint8).reshape(-1))
    k2 = [oracle.new_cache(fmt, rows) for _ in range(n_layers)]
    v2 = [oracle.new_cache(fmt, rows) for _ in range(n_layers)]
    oracle.restore(fmt, k2, v2, p, snap)
    for l in range(n_layers):
        assert np.array_equal(k2[l][:p], kcs[l][:p]) and not k2[l][p:].any()
        assert np.array_equal(v2[l][:p], vcs[l][:p]) and not v2[l][p:].any()


def test_step_operators_around_the_path(oracle):
    """rmsnorm / rope2 / attn_gate of the reference's dispatch list (quad.rs:113-116,125) as restated by the oracle."""
    rng = np.random.default_rng(23)
    ntok = 3
    qf = (rng.standard_normal((ntok, 16, 512)) * 2.0).astype(np.float32)
    w = (1.0 + 0.2 * rng.standard_normal(256)).astype(np.float32)
    y = oracle.rmsnorm(qf, 16 * ntok, 256, 512, w, 1e-6)  # rows at stride 512: the query half of every head
    x = qf[:, :, :256].reshape(-1, 256).astype(np.float64)
    ref = x / np.sqrt((x * x).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.abs(y - ref).max() < 2e-6 * np.abs(ref).max()
    assert not np.array_equal(y, oracle.rmsnorm(qf[:, :, 256:].copy(), 16 * ntok, 256, 256, w, 1e-6))  # the stride matters
    # rope2 on [rows][256] = the rotation the K writer applies before it converts (kv.wgsl:19-23)
    tab = oracle.rope_tables(77, ntok)
    kn = rng.standard_normal((ntok, 2, 256)).astype(np.float32)
    rot = oracle.rope2(kn, 2, tab)
    assert np.array_equal(rot[:, 64:], kn.reshape(-1, 256)[:, 64:])
    kc, vc = oracle.new_cache(1, 128), oracle.new_cache(1, 128)
    oracle.append(1, kc, vc, 5, kn, kn, tab)
    assert np.array_equal(kc[5:5 + ntok].reshape(-1, 256), rot)
    for t in range(ntok):  # a rotation keeps the norm of every (i, i + 32) pair
        a, b = kn[t].reshape(2, 256), rot.reshape(ntok, 2, 256)[t]
        assert np.allclose(a[:, :32] ** 2 + a[:, 32:64] ** 2, b[:, :32] ** 2 + b[:, 32:64] ** 2, rtol=1e-5)
    # the gate reads the second half of each head's 512 values
    att = rng.standard_normal((ntok, 16, 256)).astype(np.float32)
    g = oracle.attn_gate(att, qf)
    ref = att / (1.0 + np.exp(-qf[:, :, 256:].astype(np.float64)))
    assert np.abs(g - ref).max() < 1e-6


@pytest.mark.parametrize("fmt", [0, 1])
def test_window_reference_reduces_to_the_plain_one(oracle, fmt):
    """Ring rows, window and sinks of the second model (flint_attn.wgsl:79-82,243-255): with none of them the f64
    reference is the plain one; a ring only renames rows; the window drops old keys; a sink only scales rows down."""
    pos, ntok, ring = 300, 3, 256
    k = synth.normal(31, synth.S_K, 0, (pos + ntok, 2, 256)); v = synth.normal(31, synth.S_V, 0, (pos + ntok, 2, 256))
    kc, vc = oracle.new_cache(fmt, 512), oracle.new_cache(fmt, 512)
    oracle.append(fmt, kc, vc, 0, k, v, None)
    q = synth.normal(31, synth.S_Q, 0, (ntok, 16, 256))
    plain = oracle.attn_ref_f64(fmt, kc, vc, 0, pos, q)
    assert np.array_equal(oracle.attn_window_f64(fmt, kc, vc, 0, 0, None, pos, q), plain)
    # window 100 on the contiguous cache = the same rows placed in a ring of 256 (only the last 256 positions survive)
    kr, vr = oracle.new_cache(fmt, ring), oracle.new_cache(fmt, ring)
    oracle.append_ring(fmt, kr, vr, ring, 0, k, v, None)
    a = oracle.attn_window_f64(fmt, kc, vc, 0, 100, None, pos, q)
    b = oracle.attn_window_f64(fmt, kr, vr, ring, 100, None, pos, q)
    assert np.array_equal(a, b) and not np.array_equal(a, plain)
    # token t with window w = a one-token call whose first position is pos + t + 1 - w
    for t in range(ntok):
        one = oracle.attn_ref_f64(fmt, kc, vc, pos + t + 1 - 100, pos + t, q[t:t + 1])
        assert np.allclose(a[t], one[0], rtol=1e-12, atol=1e-15)
    # a sink adds exp(sink - max) to every denominator: outputs shrink by a common factor per row
    s = oracle.attn_window_f64(fmt, kc, vc, 0, 0, np.full(16, 2.0, np.float32), pos, q)
    ratio = s / plain
    assert np.all(ratio > 0) and np.all(ratio < 1) and np.allclose(ratio, ratio[..., :1], rtol=1e-9)
