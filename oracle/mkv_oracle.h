/* CPU oracle for the KV-cache / attention path of ssomenzi/mechta.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing here is part of the product: the shipped
 * path is the CUDA library declared in include/mechta_kv.h. This file is a
 * plain-C restatement of the arithmetic of the reference's WGSL kernels and of
 * the few host routines around them, used as the checker in the tests, in the
 * smoke run and as the timed CPU baseline of the benchmark.
 *
 * PARITY UNPINNED at bit level for attention: the reference holds no golden
 * vector, known-answer test or fixture for append, attention or snapshot (its
 * shaders are only parsed in its tests) and it cannot be compiled or run where
 * this was written (Rust + wgpu + Vulkan). What the reference does pin is
 * checked in tests/test_oracle.py: the KV sizing of memcheck.rs:111
 * (2,952,790,016 bytes) and need_bytes' formula. The f32->f16 conversion is
 * pinned to round-to-nearest-even against numpy's float16.
 *
 * Each function names the reference file:line it follows
 * (M/ = engine/crates/mechta/src/, W/ = M/wgsl/).
 */
#ifndef MKV_ORACLE_H
#define MKV_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MKO_F16 = 0, MKO_F32 = 1 };
enum { MKO_HQ = 16, MKO_HKV = 2, MKO_D = 256, MKO_G = 8, MKO_ROW = 512, MKO_REC = 258 };

/* M/engine.rs:108-114 rope_table */
void mko_rope_table(int32_t pos, float out[64]);

/* WGSL pack2x16float / unpack2x16float with round-to-nearest-even */
uint16_t mko_f32_to_f16(float x);
float mko_f16_to_f32(uint16_t h);
void mko_f32_to_f16_n(const float *x, uint16_t *h, size_t n);

/* bytes of one element / of one cache buffer (M/engine.rs:63-67) */
size_t mko_elem_bytes(int fmt);
uint64_t mko_buffer_bytes_for(int fmt, uint64_t ctx);
/* M/memcheck.rs:14-20 without the fixed part */
uint64_t mko_need_bytes_kv(uint64_t ctx, int fmt, uint64_t n_layer);

/* W/kv.wgsl:13-28,39-42 (f16) and W/ops.wgsl:275-286 (f32): K rows with RoPE
 * on dims 0..63. kn = [ntok*2][256] f32, tab = [ntok][64] f32 (NULL: no
 * rotation), cache element (pos,kvh,d) at pos*512+kvh*256+d. */
void mko_append_k(int fmt, void *kcache, uint32_t pos, uint32_t ntok, const float *kn, const float *tab);
/* W/kv.wgsl:29-33 and W/ops.wgsl:141-145: V rows, convert and store */
void mko_append_v(int fmt, void *vcache, uint32_t pos, uint32_t ntok, const float *vb);

/* Cache variants of the reference's second model, on this path's geometry (W/flint_attn.wgsl:1-8,79-82,243-255;
 * M/flint.rs:22-26): position p in row p % ring (ring = 0: row p), token T sees keys pos + T - win < key <= pos + T
 * (win = 0: all from 0), sinks[16] = per-head logits that join the maximum and the sum of the softmax and never the
 * output (NULL: none). Accumulation in f64, as mko_attn_ref_f64. */
void mko_attn_window_f64(int fmt, const void *kcache, const void *vcache, uint32_t ring, uint32_t win, const float *sinks,
                         uint32_t pos, uint32_t ntok, const float *q, double *out);

/* The step either side of the KV path (M/quad.rs:113-116,125,131):
 * W/ops.wgsl:27-56 rmsnorm with flag 1 (weight) and scale 1: `rows` rows of n values, row r at x[r*step_x],
 * y[r*n + i] = x * (1 / sqrt(sum(x^2)/n + eps)) * w[i]; the sum of squares in the shader's order (thread t adds
 * elements t, t+256, ..., then the 256 partial sums are folded by halving strides). */
void mko_rmsnorm(const float *x, uint32_t rows, uint32_t n, uint32_t step_x, const float *w, float eps, float *y);
/* W/ops.wgsl:275-286 rope2: rows of 256 values, dims 0..63 rotated with the table of token r / rows_per_tok */
void mko_rope2(const float *x, uint32_t rows, uint32_t rows_per_tok, const float *tab, float *y);
/* W/ops.wgsl:171-177 attn_gate: out[i] = att[i] * sigmoid(qf[h*512 + 256 + d]), i = h*256 + d over ntok*16 heads */
void mko_attn_gate(const float *att, const float *qf, uint32_t ntok, float *out);

/* W/ops.wgsl:333-394 attn_fd_one for tokens 0..ntok-1 of a call at `pos`
 * (n = pos + 1), blocks of 128 positions from first_pos; partial records
 * [m, l, acc[256]] at ((tok*16+head)*nb+block)*258. nb = blocks allocated.
 * Blocks past the visible range of a token are not written. */
void mko_attn_fd(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos,
                 uint32_t ntok, const float *q, float *partials, uint32_t nb);
/* W/ops.wgsl:523-538 attn_fd_combine with block size bb; out = [ntok][16][256] */
void mko_attn_fd_combine(const float *partials, uint32_t nb, uint32_t bb, uint32_t first_pos, uint32_t pos,
                         uint32_t ntok, float *out);
/* both of the above; returns 0, or -1 if the scratch could not be allocated */
int mko_attn_ref_f32(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos,
                     uint32_t ntok, const float *q, float *out);
/* the same result computed in double precision in one pass (the arbiter) */
void mko_attn_ref_f64(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos,
                      uint32_t ntok, const float *q, double *out);
/* as mko_attn_ref_f32 for selected tokens only: token index list `toks` of a
 * call of many tokens (prefill: token T sees [first_pos, pos+T]); q is the
 * full [ntok_total][16][256] array; out = [n_sel][16][256]. */
int mko_attn_ref_f32_sel(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos,
                         const uint32_t *toks, uint32_t n_sel, const float *q, float *out);

/* Sequence-sharded form: positions [lo, hi) only, merged over 128-blocks as
 * W/ops.wgsl:529-536 but WITHOUT the final divide: rec = [64 rows][258] with
 * row = tok*16+head, [M, tot, acc[256]]; a row that sees nothing in [lo,hi)
 * gets M = -3e38, tot = 0, acc = 0. */
int mko_attn_shard_partial(int fmt, const void *kcache, const void *vcache, uint32_t cache_first_pos,
                           uint32_t lo, uint32_t hi, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                           const float *q, float *rec);
/* W/ops.wgsl:529-537 over n_shards records of [nrow][258]; out = [nrow][256] */
void mko_combine_shards(const float *recs, uint32_t n_shards, uint32_t nrow, float *out);

/* M/dmx.rs:47-112 attn_dmx2 arithmetic (Q and P rounded to f16, lazy
 * reference max with threshold 8, chunks of `chunk` positions, tiles of 64
 * keys) + the combine: shows the deviation the reference's production f16
 * path has from the f32 path. f16 cache only. */
int mko_attn_dmx_emul(const void *kcache, const void *vcache, uint32_t pos, uint32_t ntok, uint32_t chunk,
                      const float *q, float *out);

/* M/engine.rs:784-823: raw rows [0,p) of K then V per layer, layer order.
 * kc/vc = arrays of n_layers cache pointers. Returns bytes written/read. */
size_t mko_snapshot(int fmt, void *const *kc, void *const *vc, uint32_t n_layers, uint32_t p, uint8_t *dst);
size_t mko_restore(int fmt, void *const *kc, void *const *vc, uint32_t n_layers, uint32_t p, const uint8_t *src);

/* M/session.rs:61-66 root_key: FNV-1a 64 over the little-endian token bytes */
uint64_t mko_root_key(const uint32_t *tok, size_t n);

/* number of OpenMP threads the attention routines use (1 if built without) */
int mko_threads(void);
void mko_set_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
