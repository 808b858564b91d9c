// Prefill attention over the f16 cache on the 5th-generation tensor cores: tcgen05.mma with the S and O
// accumulators in tensor memory, K/V tiles staged by TMA.
//
// Stands in for q_f16 + attn_fa_mx + attn_fd_combine (W/fa_mx.wgsl:19-115,313-319; M/engine.rs:1215-1226): token T
// of the block (at pos0 + T) sees first_pos <= key < pos0 + 1 + T; the block's K/V rows were appended before
// (M/engine.rs:1213-1214). A CTA owns 16 tokens x the 8 query heads of one KV head = 128 rows (row = head * 16 +
// token, the reference's row order, W/fa_mx.wgsl:4), i.e. one 128-lane TMEM accumulator; every K/V tile feeds all
// 8 heads. No split over keys: the output is final.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one thread) and TMEM owner, warps 2..5 = one
// softmax thread per row. Per 64-key tile: S = Q K^T (16 MMAs 128x64x16 into one of two S buffers in TMEM);
// the row's thread reads S, scales, masks, exponentiates against a reference maximum that only moves when the
// tile maximum exceeds it by more than 8 (the reference's lazy maximum, M/dmx.rs:80 and W/fa_mx.wgsl:120: a
// matrix accumulator cannot be rescaled per row cheaply), writes P as f16 to shared memory; O += P V (4 MMAs
// 128x256x16, V used N-major straight from its TMA tile). S of tile j+1 is computed while tile j is in softmax.
// TMEM: O = columns 0..255, S buffers = 256..319 and 320..383, Q (f16, the A operand of Q K^T) = 384..511, which
// leaves shared memory to a 3-deep K/V ring. Every wait is bounded; TMEM is freed on every path.
#include <stdlib.h>

#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int TC_NST = 3;                              // K/V ring depth
constexpr uint32_t TC_TILE = 64;                       // keys per tile (= PF_TILE, the tensor map's box)
constexpr uint32_t TC_KV_STAGE = 65536;                // K 32 KB + V 32 KB
constexpr uint32_t TC_SUB = 8192;                      // [64 keys][64 dims] f16
constexpr uint32_t TC_OFF_P = TC_NST * TC_KV_STAGE;    // [128 rows][64 keys] f16
constexpr uint32_t TC_OFF_BAR = TC_OFF_P + 16384;
// barriers: kv_full[NST], kv_empty[NST], s_full[2], p_full, pv_done
constexpr uint32_t TC_NBAR = 2 * TC_NST + 4;
constexpr uint32_t TC_OFF_MISC = TC_OFF_BAR + TC_NBAR * 8; // tmem base, abort flag
constexpr uint32_t TC_SMEM = TC_OFF_MISC + 16 + 1024;
constexpr uint32_t TC_COL_O = 0, TC_COL_S = 256, TC_COL_Q = 384, TC_COLS = 512;
constexpr long long TC_WAIT_LIMIT = 2000000000ll;
constexpr float TC_LAZY = 8.0f;

struct TcShared {
    uint32_t tmem_base;
    volatile uint32_t abort;
};

// Bounded wait shared by all roles: returns false (and raises the CTA's abort flag) when it runs out or when
// another thread already gave up.
__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity, TcShared *sh, uint32_t *status) {
    if (sh->abort) return false;
    if (mbar_wait_bounded(bar, parity, TC_WAIT_LIMIT)) return true;
    sh->abort = 1;
    atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
    return false;
}

// QF16: the queries come as f16 [ntok][16][256] (the output of the reference's q_f16 pass) instead of f32.
template <bool QF16>
__global__ void __launch_bounds__(192, 1)
prefill_f16_tc_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      const void *__restrict__ q, float *__restrict__ out, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                      uint32_t row0, uint32_t *__restrict__ status, uint32_t phase_arg) {
    // phase (builds with -DMKV_MEASURE only): 0 = everything, 1 = tile loads only, 2 = loads and MMAs without the softmax math
#ifdef MKV_MEASURE
    const uint32_t phase = phase_arg;
#else
    constexpr uint32_t phase = 0u;
    (void)phase_arg;
#endif
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t grp = gridDim.x - 1u - blockIdx.x; // longest key ranges first
    const uint32_t kvh = blockIdx.y;
    const uint32_t tok0 = grp * 16u;
    const uint32_t last_tok = min(tok0 + 15u, ntok - 1u);
    const uint32_t lim = pos0 + 1u + last_tok; // keys seen by the group: [first_pos, lim)
    const uint32_t t0 = first_pos / TC_TILE, nt = (lim + TC_TILE - 1u) / TC_TILE - t0;
    const uint32_t bar0 = smem_base + TC_OFF_BAR;
    const uint32_t bar_kv_full = bar0, bar_kv_empty = bar0 + 8u * TC_NST, bar_s_full = bar0 + 16u * TC_NST;
    const uint32_t bar_p_full = bar_s_full + 16u, bar_pv_done = bar_p_full + 8u;
    TcShared *sh = reinterpret_cast<TcShared *>(smem + TC_OFF_MISC);

    if (tid == 0) {
        for (int s = 0; s < TC_NST; s++) {
            mbar_init(bar_kv_full + 8u * s, 1);
            mbar_init(bar_kv_empty + 8u * s, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_full + 8u, 1);
        mbar_init(bar_p_full, 128);
        mbar_init(bar_pv_done, 1);
        sh->abort = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_base + TC_OFF_MISC, TC_COLS); // writes sh->tmem_base

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    // Q of the group goes to tensor memory as the A operand of S = Q K^T (q_f16 of the reference, W/fa_mx.wgsl:313-319):
    // the thread that owns a row converts it to f16 and stores it in its lane, two values per 32-bit column.
    // Q in TMEM instead of shared memory leaves room for a third K/V stage.
    if (warp >= 2) {
        const uint32_t row = 32u * (warp & 3u) + lane, lane_addr = (32u * (warp & 3u)) << 16;
        const uint32_t tok = tok0 + (row & 15u), head = 8u * kvh + (row >> 4);
        const size_t qoff = (size_t)min(tok, ntok - 1u) * 4096u + (size_t)head * 256u;
#pragma unroll 1
        for (uint32_t c0 = 0; c0 < 4u; c0++) { // 64 dims = 32 columns per store
            uint32_t w[32];
            if constexpr (QF16) { // already f16: eight 16-byte loads per 64 dims
                const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const __half *>(q) + qoff + c0 * 64u);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const uint4 a = src[i];
                    w[4 * i] = a.x; w[4 * i + 1] = a.y; w[4 * i + 2] = a.z; w[4 * i + 3] = a.w;
                }
            } else {
                const float *src = static_cast<const float *>(q) + qoff + c0 * 64u;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float4 a = *reinterpret_cast<const float4 *>(src + 4 * i);
                    const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
                    w[2 * i] = *reinterpret_cast<const uint32_t *>(&h0);
                    w[2 * i + 1] = *reinterpret_cast<const uint32_t *>(&h1);
                }
            }
            if (tok >= ntok) {
#pragma unroll
                for (int i = 0; i < 32; i++) w[i] = 0u;
            }
            tmem_st32(tmem + lane_addr + TC_COL_Q + 32u * c0, w);
        }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (uint32_t j = 0; j < nt; j++) {
                const uint32_t s = j % TC_NST;
                if (j >= (uint32_t)TC_NST && !tc_wait(bar_kv_empty + 8u * s, ((j / TC_NST) - 1u) & 1u, sh, status)) break;
                const uint32_t dst = smem_base + s * TC_KV_STAGE, bar = bar_kv_full + 8u * s;
                const int y = (int)((t0 + j) * TC_TILE - row0), x = (int)(kvh * 256u);
                mbar_expect_tx(bar, TC_KV_STAGE);
#pragma unroll
                for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + sb * TC_SUB, &kmap, x + 64 * sb, y, bar);
#pragma unroll
                for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + 4 * TC_SUB + sb * TC_SUB, &vmap, x + 64 * sb, y, bar);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t IDESC_QK = tc_idesc_f16(128, 64, false);
            constexpr uint32_t IDESC_PV = tc_idesc_f16(128, 256, true);
            auto qk = [&](uint32_t j) -> bool { // S[j & 1] = Q K_j^T
                const uint32_t s = j % TC_NST;
                if (!tc_wait(bar_kv_full + 8u * s, (j / TC_NST) & 1u, sh, status)) return false;
                tc_fence_after();
                const uint32_t kb = smem_base + s * TC_KV_STAGE;
                const uint32_t d = tmem + TC_COL_S + 64u * (j & 1u);
#pragma unroll
                for (uint32_t ks = 0; ks < 16u; ks++) { // 16 dims per MMA; 4 per 64-dim sub-box
                    const uint64_t b = tc_desc_sw128(kb + (ks >> 2) * TC_SUB + (ks & 3u) * 32u, 16, 1024);
                    if (phase != 1u) tc_mma_f16_ta(d, tmem + TC_COL_Q + 8u * ks, b, IDESC_QK, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full + 8u * (j & 1u));
                return true;
            };
            bool ok = nt > 0 && qk(0);
            for (uint32_t j = 0; ok && j < nt; j++) {
                if (j + 1u < nt && !(ok = qk(j + 1u))) break; // tile j+1's scores while tile j is in softmax
                if (!(ok = tc_wait(bar_p_full, j & 1u, sh, status))) break;
                tc_fence_after();
                const uint32_t vb = smem_base + (j % TC_NST) * TC_KV_STAGE + 4 * TC_SUB, pb = smem_base + TC_OFF_P;
#pragma unroll
                for (uint32_t ks = 0; ks < 4u; ks++) { // 16 keys per MMA
                    const uint64_t a = tc_desc_sw128(pb + ks * 32u, 16, 1024);
                    // V tile [64 keys][64 dims] x 4 sub-boxes, N-major: next 64 dims 8192 bytes on, next 8 keys 1024
                    const uint64_t b = tc_desc_sw128(vb + ks * 2048u, TC_SUB, 1024);
                    if (phase != 1u) tc_mma_f16(tmem + TC_COL_O, a, b, IDESC_PV, (j > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(bar_kv_empty + 8u * (j % TC_NST)); // K and V of the stage are free
                tc_commit(bar_pv_done);                      // O holds tiles 0..j; P may be overwritten
            }
        }
    } else {
        // ---------------- softmax: one thread per row (TMEM lane) ----------------
        const uint32_t row = 32u * (warp & 3u) + lane; // the TMEM lanes this warp may access
        const uint32_t lane_addr = (32u * (warp & 3u)) << 16;
        const uint32_t tok = tok0 + (row & 15u), head = 8u * kvh + (row >> 4);
        const uint32_t vis = pos0 + 1u + tok;              // the row's token sees keys < vis
        const uint32_t full_below = pos0 + 1u + tok0;      // keys below this are visible to every row
        float m_ref = NEG_BIG, l_run = 0.0f;
        bool ok = true;
        for (uint32_t j = 0; j < nt; j++) {
            // the warp takes every wait's outcome together: the TMEM loads below are warp-collective
            if (!(ok = __all_sync(0xffffffffu, tc_wait(bar_s_full + 8u * (j & 1u), (j >> 1) & 1u, sh, status)))) break;
            tc_fence_after();
            if (phase != 0u) { // measurement: no softmax math, P left as it is
                if (j > 0 && !(ok = __all_sync(0xffffffffu, tc_wait(bar_pv_done, (j - 1u) & 1u, sh, status)))) break;
                tc_fence_before();
                mbar_arrive(bar_p_full);
                continue;
            }
            uint32_t sr[2][32];
            tmem_ld32(tmem + lane_addr + TC_COL_S + 64u * (j & 1u), sr[0]);
            tmem_ld32(tmem + lane_addr + TC_COL_S + 64u * (j & 1u) + 32u, sr[1]);
            tmem_wait_ld();
            const uint32_t key_base = (t0 + j) * TC_TILE;
            const bool need_mask = key_base + TC_TILE > full_below || key_base < first_pos;
            // work in base-2 exponents: exp(s / 16 - m) = 2^(s * C - m2), C = log2(e) / 16, one FFMA + one ex2 per score
            constexpr float C2 = SCALE * 1.4426950408889634f;
            float mt = NEG_BIG;
            if (need_mask) { // tiles that touch the causal diagonal or the window start: scale, then mask (W/fa_mx.wgsl:62)
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        const uint32_t key = key_base + 32u * h + c;
                        const float v = (key >= first_pos && key < vis) ? __uint_as_float(sr[h][c]) : NEG_BIG;
                        sr[h][c] = __float_as_uint(v);
                        mt = fmaxf(mt, v);
                    }
            } else {
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int c = 0; c < 32; c++) mt = fmaxf(mt, __uint_as_float(sr[h][c]));
            }
            mt = mt > NEG_TEST ? mt * C2 : NEG_BIG; // the tile maximum as a base-2 exponent
            // lazy reference maximum: move it only for the first valid tile or when the tile exceeds it by more than 8
            // (in natural units, as the reference; 8 * log2(e) here)
            float cf = 1.0f;
            if (mt > NEG_TEST && (m_ref < NEG_TEST || mt > m_ref + TC_LAZY * 1.4426950408889634f)) {
                const float m_new = fmaxf(m_ref, mt);
                cf = m_ref > NEG_TEST ? exp2f(m_ref - m_new) : 1.0f;
                m_ref = m_new;
            }
            const float neg_m = m_ref > NEG_TEST ? -m_ref : 0.0f; // masked scores stay at -3e38 * C: 2^that = 0
            float sum = 0.0f;
            uint32_t ph[32]; // 64 weights as f16 pairs
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    float w0, w1;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w0) : "f"(fmaf(__uint_as_float(sr[h][c]), C2, neg_m)));
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w1) : "f"(fmaf(__uint_as_float(sr[h][c + 1]), C2, neg_m)));
                    sum += w0 + w1;
                    const __half2 hp = __floats2half2_rn(w0, w1);
                    ph[16 * h + (c >> 1)] = *reinterpret_cast<const uint32_t *>(&hp);
                }
            l_run = l_run * cf + sum;
            // P and O belong to the MMAs of tile j-1 until those have completed
            if (j > 0 && !(ok = __all_sync(0xffffffffu, tc_wait(bar_pv_done, (j - 1u) & 1u, sh, status)))) break;
            tc_fence_after();
            if (j > 0 && __any_sync(0xffffffffu, cf != 1.0f)) { // rescale this warp's rows of O (rare)
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < 256u; c0 += 32u) {
                    uint32_t orow[32];
                    tmem_ld32(tmem + lane_addr + TC_COL_O + c0, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; c++) orow[c] = __float_as_uint(__uint_as_float(orow[c]) * cf);
                    tmem_st32(tmem + lane_addr + TC_COL_O + c0, orow);
                }
                tmem_wait_st();
            }
            uint8_t *prow = smem + TC_OFF_P;
#pragma unroll
            for (uint32_t c = 0; c < 8u; c++) // 8 chunks of 8 keys
                *reinterpret_cast<uint4 *>(prow + swz128(row, c)) = make_uint4(ph[4 * c], ph[4 * c + 1], ph[4 * c + 2], ph[4 * c + 3]);
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar_p_full);
        }
        // ---------------- epilogue: out[tok][head][:] = O / l ----------------
        if (ok && nt > 0) ok = __all_sync(0xffffffffu, tc_wait(bar_pv_done, (nt - 1u) & 1u, sh, status));
        tc_fence_after();
        if (ok && nt > 0) {
            const float inv = 1.0f / l_run;
            float *dst = out + (size_t)tok * 4096u + (size_t)head * 256u;
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < 256u; c0 += 32u) {
                uint32_t orow[32];
                tmem_ld32(tmem + lane_addr + TC_COL_O + c0, orow);
                tmem_wait_ld();
                if (tok < ntok) {
#pragma unroll
                    for (int c = 0; c < 32; c += 4)
                        *reinterpret_cast<float4 *>(dst + c0 + c) =
                            make_float4(__uint_as_float(orow[c]) * inv, __uint_as_float(orow[c + 1]) * inv,
                                        __uint_as_float(orow[c + 2]) * inv, __uint_as_float(orow[c + 3]) * inv);
                }
            }
        }
    }

    // ---------------- teardown: nothing of this CTA may still be in flight, then free the tensor memory ----------------
    tc_fence_before();
    __syncthreads();
    if (sh->abort && tid == 0) {
        // a wait ran out somewhere: give copies already issued into this CTA's shared memory a bounded time to land
        for (int s = 0; s < TC_NST; s++) mbar_wait_bounded(bar_kv_full + 8u * s, 0, 200000000ll);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TC_COLS);
    }
}

mkv_status prefill_tc_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(prefill_f16_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(prefill_f16_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    return MKV_OK;
}

mkv_status launch_prefill_f16_tc(Ctx *ctx, Cache *c, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                                 const void *q, bool q_is_f16, float *out) {
#ifdef MKV_MEASURE
    static const uint32_t phase = [] { const char *e = getenv("MKV_PHASE"); return e ? (uint32_t)atoi(e) : 0u; }();
#else
    const uint32_t phase = 0u;
#endif
    const dim3 grid((ntok + 15u) / 16u, 2);
    const CUtensorMap &km = c->maps_host[2 * (c->n_layers + layer)], &vm = c->maps_host[2 * (c->n_layers + layer) + 1];
    if (q_is_f16)
        prefill_f16_tc_kernel<true><<<grid, 192, TC_SMEM, ctx->stream>>>(km, vm, q, out, first_pos, pos0, ntok, c->shard_first,
                                                                         ctx->dev_status, phase);
    else
        prefill_f16_tc_kernel<false><<<grid, 192, TC_SMEM, ctx->stream>>>(km, vm, q, out, first_pos, pos0, ntok, c->shard_first,
                                                                          ctx->dev_status, phase);
    ctx->launches++;
    MKV_CUDA(cudaGetLastError());
    return MKV_OK;
}

} // namespace mkv
