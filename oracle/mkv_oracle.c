/* CPU oracle: see mkv_oracle.h. TEST INFRASTRUCTURE ONLY, never the product path.
 * PARITY UNPINNED at bit level for attention (the reference has no golden vectors for this path).
 * Build with -ffp-contract=off so that a*b+c keeps two roundings, as the contract for the K writer says.
 */
#include "mkv_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define NEG_BIG (-3.0e38f)
#define NEG_TEST (-1.0e38f)
#define FD_B 128u

int mko_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Threads of the parallel regions that follow, whatever OMP_NUM_THREADS said when the library was loaded (launchers such
 * as torch.distributed.run export OMP_NUM_THREADS=1 to every rank). n < 1 leaves the setting alone. */
void mko_set_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ---- M/engine.rs:108-114 ------------------------------------------------------------------------ */
void mko_rope_table(int32_t pos, float out[64]) {
    const float scale = powf(1e7f, -2.0f / 64.0f);
    float th = (float)pos;
    for (int i = 0; i < 32; i++) {
        out[i] = cosf(th);
        out[32 + i] = sinf(th);
        th *= scale;
    }
}

/* ---- f16 conversion, round to nearest even -------------------------------------------------------- */
uint16_t mko_f32_to_f16(float x) {
    uint32_t u;
    memcpy(&u, &x, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7fffffffu;
    if (a >= 0x7f800000u) /* inf or NaN (NaN kept quiet, payload top bits kept) */
        return (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? (0x0200u | ((a >> 13) & 0x03ffu)) : 0u));
    if (a >= 0x477ff000u) /* >= 65520: rounds to infinity */
        return (uint16_t)(sign | 0x7c00u);
    if (a >= 0x38800000u) { /* normal half: 2^-14 <= |x| */
        uint32_t m = a - 0x38000000u; /* rebias exponent 127 -> 15 */
        uint32_t r = m >> 13;
        uint32_t rest = m & 0x1fffu;
        if (rest > 0x1000u || (rest == 0x1000u && (r & 1u))) r++;
        return (uint16_t)(sign | r);
    }
    if (a < 0x33000000u) /* < 2^-25: rounds to zero (2^-25 itself is a tie to even = 0) */
        return (uint16_t)sign;
    /* subnormal half: value = mant24 * 2^(e-150), unit 2^-24 */
    uint32_t e = a >> 23;
    uint32_t mant = (a & 0x7fffffu) | 0x800000u;
    uint32_t shift = 126u - e; /* e in [102,112] -> shift in [14,24] */
    uint32_t r = mant >> shift;
    uint32_t rest = mant & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1u);
    if (rest > half || (rest == half && (r & 1u))) r++;
    return (uint16_t)(sign | r);
}

float mko_f16_to_f32(uint16_t h) {
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1fu;
    uint32_t m = h & 0x3ffu;
    uint32_t u;
    if (e == 0) {
        if (m == 0) u = sign;
        else {
            int s = 0;
            while (!(m & 0x400u)) { m <<= 1; s++; }
            m &= 0x3ffu;
            u = sign | ((uint32_t)(113 - s) << 23) | (m << 13);
        }
    } else if (e == 31) u = sign | 0x7f800000u | (m << 13);
    else u = sign | ((e + 112u) << 23) | (m << 13);
    float f;
    memcpy(&f, &u, 4);
    return f;
}

void mko_f32_to_f16_n(const float *x, uint16_t *h, size_t n) {
    for (size_t i = 0; i < n; i++) h[i] = mko_f32_to_f16(x[i]);
}

size_t mko_elem_bytes(int fmt) { return fmt == MKO_F32 ? 4 : 2; }
/* M/engine.rs:63-67: 4 * data_words(ctx * 512) */
uint64_t mko_buffer_bytes_for(int fmt, uint64_t ctx) { return 4u * (fmt == MKO_F32 ? ctx * 512u : ctx * 512u / 2u); }
/* M/memcheck.rs:15-18: K and V of every layer + the flash-decoding partials */
uint64_t mko_need_bytes_kv(uint64_t ctx, int fmt, uint64_t n_layer) {
    uint64_t kv = 2u * n_layer * mko_buffer_bytes_for(fmt, ctx);
    uint64_t a = 8u * (ctx / 64u), b = 64u * (ctx / 2048u);
    uint64_t partials = 4u * 258u * 16u * (2u * (ctx / 128u) + (a > b ? a : b));
    return kv + partials;
}

static inline float cache_get(int fmt, const void *c, size_t e) {
    return fmt == MKO_F32 ? ((const float *)c)[e] : mko_f16_to_f32(((const uint16_t *)c)[e]);
}
static inline void cache_put(int fmt, void *c, size_t e, float v) {
    if (fmt == MKO_F32) ((float *)c)[e] = v;
    else ((uint16_t *)c)[e] = mko_f32_to_f16(v);
}

/* ---- W/kv.wgsl:13-17 kv_src; W/ops.wgsl:278-285 ---------------------------------------------------- */
static inline float k_src(const float *a, const float *tab, uint32_t d) {
    if (tab && d < 32u) {
        float p0 = a[d] * tab[d];
        float p1 = a[d + 32u] * tab[32u + d];
        return p0 - p1;
    }
    if (tab && d < 64u) {
        uint32_t i = d - 32u;
        float p0 = a[i] * tab[32u + i];
        float p1 = a[d] * tab[i];
        return p0 + p1;
    }
    return a[d];
}

void mko_append_k(int fmt, void *kcache, uint32_t pos, uint32_t ntok, const float *kn, const float *tab) {
    for (uint32_t r = 0; r < 2u * ntok; r++) { /* row r = token r/2, KV head r%2 (flag = 2) */
        const float *a = kn + (size_t)r * 256u;
        const float *tb = tab ? tab + (size_t)(r / 2u) * 64u : NULL;
        size_t o0 = (size_t)pos * 512u + (size_t)r * 256u;
        for (uint32_t d = 0; d < 256u; d++) cache_put(fmt, kcache, o0 + d, k_src(a, tb, d));
    }
}

void mko_append_v(int fmt, void *vcache, uint32_t pos, uint32_t ntok, const float *vb) {
    size_t n = 512u * (size_t)ntok, o0 = (size_t)pos * 512u;
    for (size_t e = 0; e < n; e++) cache_put(fmt, vcache, o0 + e, vb[e]);
}

/* ---- one block of attn_fd_one (W/ops.wgsl:340-393): positions [start, start+128) of KV head kvh,
 * visible while s < n; q8 = the 8 query rows of this KV head (each 256 f32). Cache row of position s is at
 * (s - cfirst) * 512. Results: m[8], l[8], acc[8][256]. ------------------------------------------------ */
static inline float dot4(const float *x, const float *y) {
    float s = x[0] * y[0];
    s = s + x[1] * y[1];
    s = s + x[2] * y[2];
    s = s + x[3] * y[3];
    return s;
}

static void fd_block(int fmt, const void *kc, const void *vc, uint32_t cfirst, uint32_t kvh, uint32_t start, uint32_t n,
                     const float *const q8[8], float scale, float *m, float *l, float (*acc)[256]) {
    float fs[8][FD_B];
    float krow[256];
    for (uint32_t p = 0; p < FD_B; p++) {
        uint32_t s = start + p;
        int valid = s < n;
        if (valid) {
            size_t kb = (size_t)(s - cfirst) * 512u + kvh * 256u;
            for (uint32_t d = 0; d < 256u; d++) krow[d] = cache_get(fmt, kc, kb + d);
            for (uint32_t h = 0; h < 8u; h++) {
                float side0 = 0.0f, side1 = 0.0f; /* the two half-row threads of phase 1 */
                for (uint32_t i = 0; i < 32u; i++) side0 += dot4(q8[h] + 4u * i, krow + 4u * i);
                for (uint32_t i = 32u; i < 64u; i++) side1 += dot4(q8[h] + 4u * i, krow + 4u * i);
                fs[h][p] = (side0 + side1) * scale;
            }
        } else {
            for (uint32_t h = 0; h < 8u; h++) fs[h][p] = NEG_BIG;
        }
    }
    for (uint32_t h = 0; h < 8u; h++) {
        float mx = NEG_BIG;
        for (uint32_t i = 0; i < FD_B; i++) mx = fmaxf(mx, fs[h][i]);
        float sm = 0.0f;
        for (uint32_t i = 0; i < FD_B; i++) {
            float w = fs[h][i] > NEG_TEST ? expf(fs[h][i] - mx) : 0.0f;
            fs[h][i] = w;
            sm += w;
        }
        m[h] = mx;
        l[h] = sm;
    }
    /* phase 2: 4 lanes of positions (sp = start + lane, +4, ...), summed lane0 + lane1 + lane2 + lane3 */
    uint32_t end = n < start + FD_B ? n : start + FD_B;
    static _Thread_local float lane_acc[4][8][256];
    memset(lane_acc, 0, sizeof lane_acc);
    for (uint32_t sp = start; sp < end; sp++) {
        uint32_t i = sp - start, lane = i & 3u;
        size_t vb = (size_t)(sp - cfirst) * 512u + kvh * 256u;
        for (uint32_t d = 0; d < 256u; d++) krow[d] = cache_get(fmt, vc, vb + d);
        for (uint32_t h = 0; h < 8u; h++) {
            float w = fs[h][i];
            float *a = lane_acc[lane][h];
            for (uint32_t d = 0; d < 256u; d++) a[d] += w * krow[d];
        }
    }
    for (uint32_t h = 0; h < 8u; h++)
        for (uint32_t d = 0; d < 256u; d++)
            acc[h][d] = lane_acc[0][h][d] + lane_acc[1][h][d] + lane_acc[2][h][d] + lane_acc[3][h][d];
}

void mko_attn_fd(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                 const float *q, float *partials, uint32_t nb) {
    const float scale = 1.0f / 16.0f;
    uint32_t nblk_max = (pos + ntok - first_pos + FD_B - 1u) / FD_B;
    long total = (long)ntok * 2 * nblk_max;
#pragma omp parallel for schedule(dynamic, 4)
    for (long w = 0; w < total; w++) {
        uint32_t block = (uint32_t)(w % nblk_max);
        uint32_t kvh = (uint32_t)((w / nblk_max) % 2);
        uint32_t tl = (uint32_t)(w / (2 * (long)nblk_max));
        uint32_t n = pos + 1u + tl;
        uint32_t start = first_pos + block * FD_B;
        if (start >= n) continue; /* W/ops.wgsl:339 */
        const float *q8[8];
        for (uint32_t h = 0; h < 8u; h++) q8[h] = q + (size_t)tl * 4096u + (size_t)(8u * kvh + h) * 256u;
        float m[8], l[8];
        float acc[8][256];
        fd_block(fmt, kcache, vcache, 0, kvh, start, n, q8, scale, m, l, acc);
        for (uint32_t h = 0; h < 8u; h++) {
            float *rec = partials + ((size_t)(tl * 16u + 8u * kvh + h) * nb + block) * MKO_REC;
            rec[0] = m[h];
            rec[1] = l[h];
            memcpy(rec + 2, acc[h], 256 * sizeof(float));
        }
    }
}

void mko_attn_fd_combine(const float *partials, uint32_t nb, uint32_t bb, uint32_t first_pos, uint32_t pos,
                         uint32_t ntok, float *out) {
    for (uint32_t tl = 0; tl < ntok; tl++)
        for (uint32_t h = 0; h < 16u; h++) {
            uint32_t nbv = (pos + 1u + tl - first_pos + bb - 1u) / bb;
            const float *base = partials + (size_t)(tl * 16u + h) * nb * MKO_REC;
            float M = NEG_BIG;
            for (uint32_t b = 0; b < nbv; b++) M = fmaxf(M, base[(size_t)b * MKO_REC]);
            float tot = 0.0f;
            float acc[256];
            memset(acc, 0, sizeof acc);
            for (uint32_t b = 0; b < nbv; b++) {
                const float *rec = base + (size_t)b * MKO_REC;
                float e = expf(rec[0] - M);
                tot += e * rec[1];
                for (uint32_t d = 0; d < 256u; d++) acc[d] += e * rec[2 + d];
            }
            float *o = out + (size_t)tl * 4096u + (size_t)h * 256u;
            for (uint32_t d = 0; d < 256u; d++) o[d] = acc[d] / tot;
        }
}

int mko_attn_ref_f32(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                     const float *q, float *out) {
    uint32_t nb = (pos + ntok - first_pos + FD_B - 1u) / FD_B;
    float *part = (float *)malloc((size_t)ntok * 16u * nb * MKO_REC * sizeof(float));
    if (!part) return -1;
    mko_attn_fd(fmt, kcache, vcache, first_pos, pos, ntok, q, part, nb);
    mko_attn_fd_combine(part, nb, FD_B, first_pos, pos, ntok, out);
    free(part);
    return 0;
}

int mko_attn_ref_f32_sel(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos,
                         const uint32_t *toks, uint32_t n_sel, const float *q, float *out) {
    for (uint32_t i = 0; i < n_sel; i++) {
        /* token T of the call at pos behaves as a 1-token call at pos+T (W/ops.wgsl:334-336) */
        int rc = mko_attn_ref_f32(fmt, kcache, vcache, first_pos, pos + toks[i], 1, q + (size_t)toks[i] * 4096u,
                                  out + (size_t)i * 4096u);
        if (rc) return rc;
    }
    return 0;
}

void mko_attn_ref_f64(int fmt, const void *kcache, const void *vcache, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                      const float *q, double *out) {
    for (uint32_t tl = 0; tl < ntok; tl++) {
        uint32_t n = pos + 1u + tl;
        uint32_t cnt = n > first_pos ? n - first_pos : 0;
#pragma omp parallel for schedule(static)
        for (int h = 0; h < 16; h++) {
            uint32_t kvh = (uint32_t)h / 8u;
            const float *qr = q + (size_t)tl * 4096u + (size_t)h * 256u;
            double *sc = (double *)malloc((size_t)(cnt ? cnt : 1) * sizeof(double));
            double mx = -INFINITY;
            for (uint32_t s = first_pos; s < n; s++) {
                size_t kb = (size_t)s * 512u + kvh * 256u;
                double a = 0.0;
                for (uint32_t d = 0; d < 256u; d++) a += (double)qr[d] * (double)cache_get(fmt, kcache, kb + d);
                a *= 1.0 / 16.0;
                sc[s - first_pos] = a;
                if (a > mx) mx = a;
            }
            double tot = 0.0, acc[256];
            memset(acc, 0, sizeof acc);
            for (uint32_t s = first_pos; s < n; s++) {
                double w = exp(sc[s - first_pos] - mx);
                tot += w;
                size_t vb = (size_t)s * 512u + kvh * 256u;
                for (uint32_t d = 0; d < 256u; d++) acc[d] += w * (double)cache_get(fmt, vcache, vb + d);
            }
            double *o = out + (size_t)tl * 4096u + (size_t)h * 256u;
            for (uint32_t d = 0; d < 256u; d++) o[d] = acc[d] / tot;
            free(sc);
        }
    }
}

/* ---- sequence shards -------------------------------------------------------------------------------- */
int mko_attn_shard_partial(int fmt, const void *kcache, const void *vcache, uint32_t cache_first_pos, uint32_t lo,
                           uint32_t hi, uint32_t first_pos, uint32_t pos, uint32_t ntok, const float *q, float *rec) {
    const float scale = 1.0f / 16.0f;
    uint32_t s0 = first_pos > lo ? first_pos : lo;
    for (uint32_t r = 0; r < 64u; r++) {
        float *x = rec + (size_t)r * MKO_REC;
        x[0] = NEG_BIG;
        for (uint32_t i = 1; i < MKO_REC; i++) x[i] = 0.0f;
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int w = 0; w < (int)(ntok * 2u); w++) {
        uint32_t tl = (uint32_t)w / 2u, kvh = (uint32_t)w % 2u;
        uint32_t n = pos + 1u + tl;
        if (n > hi) n = hi;
        if (s0 >= n) continue;
        uint32_t nblk = (n - s0 + FD_B - 1u) / FD_B;
        const float *q8[8];
        for (uint32_t h = 0; h < 8u; h++) q8[h] = q + (size_t)tl * 4096u + (size_t)(8u * kvh + h) * 256u;
        float *bm = (float *)malloc((size_t)nblk * 8u * sizeof(float));
        float *bl = (float *)malloc((size_t)nblk * 8u * sizeof(float));
        float(*ba)[8][256] = (float(*)[8][256])malloc((size_t)nblk * sizeof(*ba));
        for (uint32_t b = 0; b < nblk; b++)
            fd_block(fmt, kcache, vcache, cache_first_pos, kvh, s0 + b * FD_B, n, q8, scale, bm + 8u * b, bl + 8u * b, ba[b]);
        for (uint32_t h = 0; h < 8u; h++) {
            float M = NEG_BIG;
            for (uint32_t b = 0; b < nblk; b++) M = fmaxf(M, bm[8u * b + h]);
            float tot = 0.0f;
            float *x = rec + (size_t)(tl * 16u + 8u * kvh + h) * MKO_REC;
            for (uint32_t b = 0; b < nblk; b++) {
                float e = expf(bm[8u * b + h] - M);
                tot += e * bl[8u * b + h];
                for (uint32_t d = 0; d < 256u; d++) x[2 + d] += e * ba[b][h][d];
            }
            x[0] = M;
            x[1] = tot;
        }
        free(bm);
        free(bl);
        free(ba);
    }
    return 0;
}

void mko_combine_shards(const float *recs, uint32_t n_shards, uint32_t nrow, float *out) {
    for (uint32_t r = 0; r < nrow; r++) {
        float M = NEG_BIG;
        for (uint32_t g = 0; g < n_shards; g++) M = fmaxf(M, recs[((size_t)g * nrow + r) * MKO_REC]);
        float tot = 0.0f;
        float acc[256];
        memset(acc, 0, sizeof acc);
        for (uint32_t g = 0; g < n_shards; g++) {
            const float *x = recs + ((size_t)g * nrow + r) * MKO_REC;
            float e = expf(x[0] - M);
            tot += e * x[1];
            for (uint32_t d = 0; d < 256u; d++) acc[d] += e * x[2 + d];
        }
        for (uint32_t d = 0; d < 256u; d++) out[(size_t)r * 256u + d] = acc[d] / tot;
    }
}

/* ---- M/dmx.rs:47-112 in scalar form ------------------------------------------------------------------ */
int mko_attn_dmx_emul(const void *kcache, const void *vcache, uint32_t pos, uint32_t ntok, uint32_t chunk,
                      const float *q, float *out) {
    const float scale = 1.0f / 16.0f, lazy = 8.0f;
    const uint16_t *kh = (const uint16_t *)kcache, *vh = (const uint16_t *)vcache;
    uint32_t lim = pos + ntok; /* p.n + kk - 1 */
    uint32_t nb = (lim + chunk - 1u) / chunk;
    uint32_t nrow = 8u * ntok;
    float *part = (float *)calloc((size_t)ntok * 16u * nb * MKO_REC, sizeof(float));
    if (!part) return -1;
#pragma omp parallel for schedule(dynamic, 1)
    for (int w = 0; w < (int)(2u * nb); w++) {
        uint32_t kvh = (uint32_t)w % 2u, ch = (uint32_t)w / 2u;
        uint32_t cs = ch * chunk;
        if (cs >= lim) continue;
        uint32_t ntile = (lim - cs + 63u) / 64u;
        if (ntile > chunk / 64u) ntile = chunk / 64u;
        float qh[32][256];
        float mrow[32], lrow[32];
        float(*O)[256] = (float(*)[256])calloc(32, sizeof(*O));
        for (uint32_t r = 0; r < nrow; r++) { /* q_dmx: row = token*8 + head%8 */
            const float *src = q + (size_t)(r / 8u) * 4096u + (size_t)(8u * kvh + r % 8u) * 256u;
            for (uint32_t d = 0; d < 256u; d++) qh[r][d] = mko_f16_to_f32(mko_f32_to_f16(src[d]));
            mrow[r] = NEG_BIG;
            lrow[r] = 0.0f;
        }
        for (uint32_t tile = 0; tile < ntile; tile++) {
            uint32_t k0 = cs + tile * 64u;
            for (uint32_t r = 0; r < nrow; r++) {
                uint32_t vis = pos + 1u + r / 8u;
                float sv[64], mt = NEG_BIG;
                for (uint32_t c = 0; c < 64u; c++) {
                    float a = 0.0f;
                    const uint16_t *kr = kh + (size_t)(k0 + c) * 512u + kvh * 256u;
                    for (uint32_t d = 0; d < 256u; d++) a += qh[r][d] * mko_f16_to_f32(kr[d]);
                    sv[c] = (k0 + c < vis) ? a * scale : NEG_BIG;
                    mt = fmaxf(mt, sv[c]);
                }
                float mo = mrow[r], mr = mo;
                if (mo < NEG_TEST || mt > mo + lazy) mr = fmaxf(mo, mt);
                float ph[64], sm = 0.0f;
                for (uint32_t c = 0; c < 64u; c++) {
                    float wgt = sv[c] > NEG_TEST ? expf(sv[c] - mr) : 0.0f;
                    ph[c] = mko_f16_to_f32(mko_f32_to_f16(wgt));
                    sm += ph[c];
                }
                float cf = mo > NEG_TEST ? expf(mo - mr) : 1.0f;
                mrow[r] = mr;
                lrow[r] = lrow[r] * cf + sm;
                if (cf != 1.0f)
                    for (uint32_t d = 0; d < 256u; d++) O[r][d] *= cf;
                for (uint32_t c = 0; c < 64u; c++) {
                    if (ph[c] == 0.0f) continue;
                    const uint16_t *vr = vh + (size_t)(k0 + c) * 512u + kvh * 256u;
                    for (uint32_t d = 0; d < 256u; d++) O[r][d] += ph[c] * mko_f16_to_f32(vr[d]);
                }
            }
        }
        for (uint32_t r = 0; r < nrow; r++) {
            float *rec = part + ((size_t)((r / 8u) * 16u + 8u * kvh + r % 8u) * nb + ch) * MKO_REC;
            rec[0] = mrow[r];
            rec[1] = lrow[r];
            memcpy(rec + 2, O[r], 256 * sizeof(float));
        }
        free(O);
    }
    mko_attn_fd_combine(part, nb, chunk, 0, pos, ntok, out);
    free(part);
    return 0;
}

/* ---- M/engine.rs:790-795, 808-816 --------------------------------------------------------------------- */
size_t mko_snapshot(int fmt, void *const *kc, void *const *vc, uint32_t n_layers, uint32_t p, uint8_t *dst) {
    size_t nb = (size_t)p * 512u * mko_elem_bytes(fmt), o = 0;
    for (uint32_t l = 0; l < n_layers; l++) {
        memcpy(dst + o, kc[l], nb); o += nb;
        memcpy(dst + o, vc[l], nb); o += nb;
    }
    return o;
}

size_t mko_restore(int fmt, void *const *kc, void *const *vc, uint32_t n_layers, uint32_t p, const uint8_t *src) {
    size_t nb = (size_t)p * 512u * mko_elem_bytes(fmt), o = 0;
    for (uint32_t l = 0; l < n_layers; l++) {
        memcpy(kc[l], src + o, nb); o += nb;
        memcpy(vc[l], src + o, nb); o += nb;
    }
    return o;
}

/* ---- M/session.rs:61-66 -------------------------------------------------------------------------------- */
uint64_t mko_root_key(const uint32_t *tok, size_t n) {
    uint64_t h = 0xcbf29ce484222325ull;
    for (size_t i = 0; i < n; i++)
        for (int b = 0; b < 4; b++) {
            h ^= (uint64_t)((tok[i] >> (8 * b)) & 0xffu);
            h *= 0x100000001b3ull;
        }
    return h;
}

/* ---- the step either side of the KV path ------------------------------------------------------------------ */

/* W/ops.wgsl:27-56 (rmsnorm, flag = 1, f1 = 1.0) */
void mko_rmsnorm(const float *x, uint32_t rows, uint32_t n, uint32_t step_x, const float *w, float eps, float *y) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *a = x + (size_t)r * step_x;
        float partial[256];
        for (uint32_t t = 0; t < 256; t++) { /* W/ops.wgsl:33-34 */
            float s = 0.0f;
            for (uint32_t i = t; i < n; i += 256u) { const float v = a[i]; s += v * v; }
            partial[t] = s;
        }
        for (uint32_t m = 128u; m > 0u; m >>= 1) /* W/ops.wgsl:37-40 */
            for (uint32_t t = 0; t < m; t++) partial[t] += partial[t + m];
        const float scale = 1.0f / sqrtf(partial[0] / (float)n + eps); /* W/ops.wgsl:41 */
        for (uint32_t i = 0; i < n; i++) { /* W/ops.wgsl:51-55 rms_val */
            float v = a[i] * scale * 1.0f;
            v = v * w[i];
            y[(size_t)r * n + i] = v;
        }
    }
}

/* W/ops.wgsl:275-286 (rope2) */
void mko_rope2(const float *x, uint32_t rows, uint32_t rows_per_tok, const float *tab, float *y) {
    for (uint32_t r = 0; r < rows; r++) {
        const float *a = x + (size_t)r * 256u, *tb = tab + (size_t)(r / rows_per_tok) * 64u;
        float *o = y + (size_t)r * 256u;
        for (uint32_t t = 0; t < 32u; t++) {
            const float x1 = a[t], x2 = a[t + 32u], co = tb[t], si = tb[32u + t];
            o[t] = x1 * co - x2 * si;
            o[t + 32u] = x1 * si + x2 * co;
        }
        for (uint32_t t = 64u; t < 256u; t++) o[t] = a[t];
    }
}

/* W/ops.wgsl:27 sigm and 171-177 attn_gate */
void mko_attn_gate(const float *att, const float *qf, uint32_t ntok, float *out) {
    const uint32_t n = ntok * 4096u;
    for (uint32_t i = 0; i < n; i++) {
        const uint32_t h = i / 256u, dd = i % 256u;
        const float v = qf[(size_t)h * 512u + 256u + dd];
        out[i] = att[i] * (1.0f / (1.0f + expf(-v)));
    }
}

/* ---- ring rows, sliding window, sinks (W/flint_attn.wgsl:79-82 kv4 and lo_di, 243-255 attn_fd_merge) ---------- */
void mko_attn_window_f64(int fmt, const void *kcache, const void *vcache, uint32_t ring, uint32_t win, const float *sinks,
                         uint32_t pos, uint32_t ntok, const float *q, double *out) {
    for (uint32_t tl = 0; tl < ntok; tl++) {
        const uint32_t n = pos + 1u + tl;
        const uint32_t lo = (win > 0u && n > win) ? n - win : 0u; /* lo_di */
#pragma omp parallel for schedule(static)
        for (int h = 0; h < 16; h++) {
            const uint32_t kvh = (uint32_t)h / 8u;
            const float *qr = q + (size_t)tl * 4096u + (size_t)h * 256u;
            double *sc = (double *)malloc((size_t)(n - lo) * sizeof(double));
            double mx = sinks ? (double)sinks[h] : -INFINITY;
            for (uint32_t s = lo; s < n; s++) {
                const size_t kb = (size_t)(ring ? s % ring : s) * 512u + kvh * 256u;
                double a = 0.0;
                for (uint32_t d = 0; d < 256u; d++) a += (double)qr[d] * (double)cache_get(fmt, kcache, kb + d);
                a *= 1.0 / 16.0;
                sc[s - lo] = a;
                if (a > mx) mx = a;
            }
            double tot = sinks ? exp((double)sinks[h] - mx) : 0.0, acc[256];
            memset(acc, 0, sizeof acc);
            for (uint32_t s = lo; s < n; s++) {
                const double w = exp(sc[s - lo] - mx);
                tot += w;
                const size_t vb = (size_t)(ring ? s % ring : s) * 512u + kvh * 256u;
                for (uint32_t d = 0; d < 256u; d++) acc[d] += w * (double)cache_get(fmt, vcache, vb + d);
            }
            double *o = out + (size_t)tl * 4096u + (size_t)h * 256u;
            for (uint32_t d = 0; d < 256u; d++) o[d] = acc[d] / tot;
            free(sc);
        }
    }
}
