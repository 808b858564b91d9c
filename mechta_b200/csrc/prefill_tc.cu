// Prefill attention over the f16 cache on the 5th-generation tensor cores: tcgen05.mma with the S and O
// accumulators in tensor memory, K/V tiles staged by TMA.
//
// Stands in for q_f16 + attn_fa_mx + attn_fd_combine (W/fa_mx.wgsl:19-115,313-319; M/engine.rs:1215-1226): token T
// of the block (at pos0 + T) sees first_pos <= key < pos0 + 1 + T; the block's K/V rows were appended before
// (M/engine.rs:1213-1214). A work item is 16 tokens x the 8 query heads of one KV head = 128 rows (row = head * 16
// + token, the reference's row order, W/fa_mx.wgsl:4), i.e. one 128-lane TMEM accumulator; every K/V tile feeds all
// 8 heads.
//
// Scheduling. The reference prefills in blocks of 512, 128, 32 and 8 tokens (M/engine.rs:869-885): a 512-token block
// is 64 items, which as one CTA per item leaves 84 of 148 SMs idle. For launches with fewer items than three
// quarters of the SMs the grid is therefore one CTA per SM, and the 64-key tiles of all items, laid end to end
// (longest items first), are cut into equal ranges, one per CTA. A CTA walks its range segment by segment; a
// segment that covers its whole item writes the output, a part of an item writes its un-normalised partial
// (reference maximum, sum, O) to scratch memory, and whichever part of the item finishes last merges the parts in
// index order (the reference splits long prefills over chunks and merges with attn_fd_combine in the same way,
// M/engine.rs:1219-1225). Measured over a 32,768-token prefix: 128 tokens 0.51 -> 0.41 ms, 512 tokens 0.52 -> 0.40 ms.
// Larger launches run one CTA per item: with most SMs busy the kernel is bound by the L2 -> SM traffic of the K/V
// tiles (64 KB per 128 rows and tile, about 8 TB/s), so evening out the waves buys nothing there and the partials
// cost (1,024 tokens 0.52 -> 0.60 ms, 2,048 tokens 1.06 -> 1.10 ms when split).
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer (one thread) and TMEM owner, warps 2..5 = one
// softmax thread per row. Per 64-key tile: S = Q K^T (16 MMAs 128x64x16 into one of two S buffers in TMEM);
// the row's thread reads S, scales, masks, exponentiates against a reference maximum that only moves when the
// tile maximum exceeds it by more than 8 (the reference's lazy maximum, M/dmx.rs:80 and W/fa_mx.wgsl:120: a
// matrix accumulator cannot be rescaled per row cheaply), writes P as f16 to shared memory; O += P V (4 MMAs
// 128x256x16, V used N-major straight from its TMA tile). S of tile j+1 is computed while tile j is in softmax.
// TMEM: O = columns 0..255, S buffers = 256..319 and 320..383, Q (f16, the A operand of Q K^T) = 384..511, which
// leaves shared memory to a 3-deep K/V ring; the producer runs ahead across segment borders. Every wait is
// bounded; TMEM is freed on every path.
#include <stdlib.h>

#include <algorithm>

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
// barriers: kv_full[NST], kv_empty[NST], s_full[2], p_full, pv_done, q_full
constexpr uint32_t TC_NBAR = 2 * TC_NST + 5;
constexpr uint32_t TC_OFF_MISC = TC_OFF_BAR + TC_NBAR * 8; // TcShared
constexpr uint32_t TC_SMEM = TC_OFF_MISC + 32 + 1024;
constexpr uint32_t TC_COL_O = 0, TC_COL_S = 256, TC_COL_Q = 384, TC_COLS = 512;
constexpr long long TC_WAIT_LIMIT = 2000000000ll;
constexpr float TC_LAZY = 8.0f;
constexpr uint32_t TC_PART = 128 * REC;   // floats of one partial: [128 rows][m, l, O[256]]
constexpr uint32_t TC_MAX_ITEMS = 512;    // 4,096 tokens / 16 x 2 KV heads

struct TcShared {
    uint32_t tmem_base;
    volatile uint32_t abort;
    uint32_t ticket;
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
// named barrier 1: the 128 softmax threads
__device__ __forceinline__ void tc_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// The work of one launch and this CTA's share of it. Items are numbered longest first: item i = (token group
// ngroups - 1 - i / 2, KV head i % 2); its tiles are the 64-key tiles from first_pos / 64 up to the last key its
// last token sees. Every thread computes the same plan (a few hundred integer operations against a kernel of about
// a millisecond).
struct PfWork {
    uint32_t first_pos, pos0, ntok, ngroups, nitems, t0;
    uint32_t lo, hi, len; // this CTA's range [lo, hi) of the tiles laid end to end, the length of every CTA's range
    bool split;
    __device__ __forceinline__ uint32_t tiles_of(uint32_t item) const {
        const uint32_t grp = ngroups - 1u - (item >> 1);
        const uint32_t last_tok = min(grp * 16u + 15u, ntok - 1u);
        return (pos0 + 1u + last_tok + TC_TILE - 1u) / TC_TILE - t0;
    }
};
struct PfSegment {
    uint32_t item, a, b;     // tiles [a, b) of the item
    uint32_t piece, npieces; // which part of the item this is, of how many
    uint32_t cta0;           // the CTA that holds the item's first part
};
__device__ __forceinline__ PfWork pf_work(uint32_t first_pos, uint32_t pos0, uint32_t ntok, bool split) {
    PfWork w;
    w.first_pos = first_pos; w.pos0 = pos0; w.ntok = ntok;
    w.ngroups = (ntok + 15u) / 16u;
    w.nitems = 2u * w.ngroups;
    w.t0 = first_pos / TC_TILE;
    w.split = split;
    if (w.split) {
        uint32_t total = 0;
        for (uint32_t i = 0; i < w.nitems; i += 2u) total += 2u * w.tiles_of(i);
        w.len = (total + gridDim.x - 1u) / gridDim.x;
        w.lo = blockIdx.x * w.len;
        w.hi = min(w.lo + w.len, total);
    } else {
        w.len = w.lo = w.hi = 0;
    }
    return w;
}
// Calls f(segment) for this CTA's segments in order; f returns false to stop. Returns false if f did.
template <typename F>
__device__ __forceinline__ bool pf_segments(const PfWork &w, F &&f) {
    if (!w.split) { // one whole item per CTA
        PfSegment sg = {blockIdx.x, 0u, w.tiles_of(blockIdx.x), 0u, 1u, blockIdx.x};
        return f(sg);
    }
    uint32_t base = 0;
    for (uint32_t i = 0; i < w.nitems && base < w.hi; i++) {
        const uint32_t n = w.tiles_of(i);
        const uint32_t lo = max(base, w.lo), hi = min(base + n, w.hi);
        if (hi > lo) {
            const uint32_t c0 = base / w.len;
            PfSegment sg = {i, lo - base, hi - base, blockIdx.x - c0, (base + n - 1u) / w.len - c0 + 1u, c0};
            if (!f(sg)) return false;
        }
        base += n;
    }
    return true;
}
// Where part `piece` of an item whose first part lies in CTA cta0 keeps its partial: a CTA has at most one segment
// that continues an item begun by the CTA before it (slot 0) and at most one that begins an item it does not finish (slot 1).
__device__ __forceinline__ size_t pf_slot(uint32_t cta0, uint32_t piece) { return 2u * (size_t)(cta0 + piece) + (piece == 0u ? 1u : 0u); }

// QF16: the queries come as f16 [ntok][16][256] (the output of the reference's q_f16 pass) instead of f32.
template <bool QF16>
__global__ void __launch_bounds__(192, 1)
prefill_f16_tc_kernel(const __grid_constant__ CUtensorMap kmap, const __grid_constant__ CUtensorMap vmap,
                      const void *__restrict__ q, float *__restrict__ out, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                      uint32_t row0, float *__restrict__ scratch, uint32_t *__restrict__ counters, uint32_t split,
                      uint32_t *__restrict__ status, uint32_t phase_arg) {
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
    const uint32_t bar0 = smem_base + TC_OFF_BAR;
    const uint32_t bar_kv_full = bar0, bar_kv_empty = bar0 + 8u * TC_NST, bar_s_full = bar0 + 16u * TC_NST;
    const uint32_t bar_p_full = bar_s_full + 16u, bar_pv_done = bar_p_full + 8u, bar_q_full = bar_pv_done + 8u;
    TcShared *sh = reinterpret_cast<TcShared *>(smem + TC_OFF_MISC);
    const PfWork work = pf_work(first_pos, pos0, ntok, split != 0u);

    if (tid == 0) {
        for (int s = 0; s < TC_NST; s++) {
            mbar_init(bar_kv_full + 8u * s, 1);
            mbar_init(bar_kv_empty + 8u * s, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_full + 8u, 1);
        mbar_init(bar_p_full, 128);
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_q_full, 128);
        sh->abort = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_base + TC_OFF_MISC, TC_COLS); // writes sh->tmem_base

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    // Every role walks the same segments; g counts the tiles this CTA has dealt with so far, across segments: ring
    // stage g % NST, S buffer g & 1, and the parities of the barriers follow from it.
    if (warp == 0) {
        // ---------------- TMA producer: runs ahead of the other roles, also across segment borders ----------------
        if (lane == 0) {
            uint32_t g = 0;
            pf_segments(work, [&](const PfSegment &sg) {
                const int x = (int)((sg.item & 1u) * 256u);
                for (uint32_t j = sg.a; j < sg.b; j++, g++) {
                    const uint32_t s = g % TC_NST;
                    if (g >= (uint32_t)TC_NST && !tc_wait(bar_kv_empty + 8u * s, ((g / TC_NST) - 1u) & 1u, sh, status)) return false;
                    const uint32_t dst = smem_base + s * TC_KV_STAGE, bar = bar_kv_full + 8u * s;
                    const int y = (int)((work.t0 + j) * TC_TILE - row0);
                    mbar_expect_tx(bar, TC_KV_STAGE);
#pragma unroll
                    for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + sb * TC_SUB, &kmap, x + 64 * sb, y, bar);
#pragma unroll
                    for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + 4 * TC_SUB + sb * TC_SUB, &vmap, x + 64 * sb, y, bar);
                }
                return true;
            });
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t IDESC_QK = tc_idesc_f16(128, 64, false);
            constexpr uint32_t IDESC_PV = tc_idesc_f16(128, 256, true);
            uint32_t g = 0, nseg = 0;
            auto qk = [&](uint32_t gg) -> bool { // S[gg & 1] = Q K^T for the tile in ring stage gg % NST
                const uint32_t s = gg % TC_NST;
                if (!tc_wait(bar_kv_full + 8u * s, (gg / TC_NST) & 1u, sh, status)) return false;
                tc_fence_after();
                const uint32_t kb = smem_base + s * TC_KV_STAGE;
                const uint32_t d = tmem + TC_COL_S + 64u * (gg & 1u);
#pragma unroll
                for (uint32_t ks = 0; ks < 16u; ks++) { // 16 dims per MMA; 4 per 64-dim sub-box
                    const uint64_t b = tc_desc_sw128(kb + (ks >> 2) * TC_SUB + (ks & 3u) * 32u, 16, 1024);
                    if (phase != 1u) tc_mma_f16_ta(d, tmem + TC_COL_Q + 8u * ks, b, IDESC_QK, ks > 0 ? 1u : 0u);
                }
                tc_commit(bar_s_full + 8u * (gg & 1u));
                return true;
            };
            pf_segments(work, [&](const PfSegment &sg) {
                // the segment's Q is in tensor memory (the softmax threads put it there once the MMAs of the segment
                // before it had all completed)
                if (!tc_wait(bar_q_full, nseg & 1u, sh, status)) return false;
                tc_fence_after();
                nseg++;
                const uint32_t n = sg.b - sg.a;
                if (!qk(g)) return false;
                for (uint32_t j = 0; j < n; j++, g++) {
                    if (j + 1u < n && !qk(g + 1u)) return false; // the next tile's scores while this one is in softmax
                    if (!tc_wait(bar_p_full, g & 1u, sh, status)) return false;
                    tc_fence_after();
                    const uint32_t vb = smem_base + (g % TC_NST) * TC_KV_STAGE + 4 * TC_SUB, pb = smem_base + TC_OFF_P;
#pragma unroll
                    for (uint32_t ks = 0; ks < 4u; ks++) { // 16 keys per MMA
                        const uint64_t a = tc_desc_sw128(pb + ks * 32u, 16, 1024);
                        // V tile [64 keys][64 dims] x 4 sub-boxes, N-major: next 64 dims 8192 bytes on, next 8 keys 1024
                        const uint64_t b = tc_desc_sw128(vb + ks * 2048u, TC_SUB, 1024);
                        if (phase != 1u) tc_mma_f16(tmem + TC_COL_O, a, b, IDESC_PV, (j > 0 || ks > 0) ? 1u : 0u);
                    }
                    tc_commit(bar_kv_empty + 8u * (g % TC_NST)); // K and V of the stage are free
                    tc_commit(bar_pv_done);                      // O holds the segment's tiles so far; P may be overwritten
                }
                return true;
            });
        }
    } else {
        // ---------------- softmax: one thread per row (TMEM lane) ----------------
        const uint32_t row = 32u * (warp & 3u) + lane; // the TMEM lanes this warp may access
        const uint32_t lane_addr = (32u * (warp & 3u)) << 16;
        uint32_t g = 0;
        pf_segments(work, [&](const PfSegment &sg) {
            const uint32_t grp = work.ngroups - 1u - (sg.item >> 1), kvh = sg.item & 1u;
            const uint32_t tok0 = grp * 16u;
            const uint32_t tok = tok0 + (row & 15u), head = 8u * kvh + (row >> 4);
            const uint32_t vis = pos0 + 1u + tok;              // the row's token sees keys < vis
            const uint32_t full_below = pos0 + 1u + tok0;      // keys below this are visible to every row
            bool ok = true;
            // Q of the item goes to tensor memory as the A operand of S = Q K^T (q_f16 of the reference,
            // W/fa_mx.wgsl:313-319): the thread that owns a row converts it to f16 and stores it in its lane, two
            // values per 32-bit column. Q in TMEM instead of shared memory leaves room for a third K/V stage. The MMAs
            // of the segment before this one have completed: its epilogue waited for them.
            {
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
                tc_fence_before();
                mbar_arrive(bar_q_full);
            }
            float m_ref = NEG_BIG, l_run = 0.0f;
            const uint32_t n = sg.b - sg.a;
            for (uint32_t j = 0; j < n; j++, g++) {
                // the warp takes every wait's outcome together: the TMEM loads below are warp-collective
                if (!(ok = __all_sync(0xffffffffu, tc_wait(bar_s_full + 8u * (g & 1u), (g >> 1) & 1u, sh, status)))) break;
                tc_fence_after();
                if (phase != 0u) { // measurement: no softmax math, P left as it is
                    if (j > 0 && !(ok = __all_sync(0xffffffffu, tc_wait(bar_pv_done, (g - 1u) & 1u, sh, status)))) break;
                    tc_fence_before();
                    mbar_arrive(bar_p_full);
                    continue;
                }
                uint32_t sr[2][32];
                tmem_ld32(tmem + lane_addr + TC_COL_S + 64u * (g & 1u), sr[0]);
                tmem_ld32(tmem + lane_addr + TC_COL_S + 64u * (g & 1u) + 32u, sr[1]);
                tmem_wait_ld();
                const uint32_t key_base = (work.t0 + sg.a + j) * TC_TILE;
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
                // P and O belong to the MMAs of the tile before until those have completed
                if (j > 0 && !(ok = __all_sync(0xffffffffu, tc_wait(bar_pv_done, (g - 1u) & 1u, sh, status)))) break;
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
            // ---------------- end of the segment: all its MMAs have completed ----------------
            if (ok && n > 0) ok = __all_sync(0xffffffffu, tc_wait(bar_pv_done, (g - 1u) & 1u, sh, status));
            tc_fence_after();
            if (!ok) return false;
            if (sg.npieces == 1u) {
                // the whole item: out[tok][head][:] = O / l
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
            } else {
                // a part of an item: its partial goes to scratch memory; the part that arrives last merges all of them
                float *ps = scratch + pf_slot(sg.cta0, sg.piece) * TC_PART + (size_t)row * REC;
                *reinterpret_cast<float2 *>(ps) = make_float2(m_ref, l_run);
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < 256u; c0 += 32u) {
                    uint32_t orow[32];
                    tmem_ld32(tmem + lane_addr + TC_COL_O + c0, orow);
                    tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 32; c += 2)
                        *reinterpret_cast<float2 *>(ps + 2u + c0 + c) = make_float2(__uint_as_float(orow[c]), __uint_as_float(orow[c + 1]));
                }
                tc_bar_sync(); // every row of the partial is written
                if (row == 0u) {
                    fence_acq_rel_gpu(); // release: the partial before the ticket; acquire: the other parts after it
                    sh->ticket = atomicAdd(counters + sg.item, 1u);
                    fence_acq_rel_gpu();
                }
                tc_bar_sync();
                if (sh->ticket == sg.npieces - 1u) {
                    if (row == 0u) counters[sg.item] = 0u; // every part has arrived: ready for the next launch
                    // merge in index order, this part's own partial included (read back like the others), so that the
                    // result does not depend on which part came last
                    float M = NEG_BIG, l = 0.0f;
                    for (uint32_t pc = 0; pc < sg.npieces; pc++)
                        M = fmaxf(M, __ldcg(scratch + pf_slot(sg.cta0, pc) * TC_PART + (size_t)row * REC));
                    float dst_acc[32];
                    float *dst = out + (size_t)tok * 4096u + (size_t)head * 256u;
                    for (uint32_t pc = 0; pc < sg.npieces; pc++) {
                        const float2 ml = __ldcg(reinterpret_cast<const float2 *>(scratch + pf_slot(sg.cta0, pc) * TC_PART + (size_t)row * REC));
                        l += ml.y * (ml.x > NEG_TEST ? exp2f(ml.x - M) : 0.0f);
                    }
                    const float inv = 1.0f / l;
#pragma unroll 1
                    for (uint32_t c0 = 0; c0 < 256u; c0 += 32u) {
#pragma unroll
                        for (int c = 0; c < 32; c++) dst_acc[c] = 0.0f;
                        for (uint32_t pc = 0; pc < sg.npieces; pc++) {
                            const float *pp = scratch + pf_slot(sg.cta0, pc) * TC_PART + (size_t)row * REC;
                            const float mq = __ldcg(pp);
                            const float e = mq > NEG_TEST ? exp2f(mq - M) : 0.0f;
#pragma unroll
                            for (int c = 0; c < 32; c += 2) {
                                const float2 v = __ldcg(reinterpret_cast<const float2 *>(pp + 2u + c0 + c));
                                dst_acc[c] = fmaf(e, v.x, dst_acc[c]);
                                dst_acc[c + 1] = fmaf(e, v.y, dst_acc[c + 1]);
                            }
                        }
                        if (tok < ntok) {
#pragma unroll
                            for (int c = 0; c < 32; c += 4)
                                *reinterpret_cast<float4 *>(dst + c0 + c) =
                                    make_float4(dst_acc[c] * inv, dst_acc[c + 1] * inv, dst_acc[c + 2] * inv, dst_acc[c + 3] * inv);
                        }
                    }
                }
                tc_bar_sync(); // sh->ticket is free for the next segment
            }
            return true;
        });
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

// Scratch of the split items: two partials per CTA and one arrival counter per item, allocated with the context's
// first prefill launch that needs them and kept until the context goes.
static mkv_status prefill_scratch(Ctx *ctx) {
    if (ctx->pf_scratch) return MKV_OK;
    const size_t bytes = 2u * (size_t)ctx->sm_count * TC_PART * sizeof(float);
    if (cudaMalloc(&ctx->pf_scratch, bytes) != cudaSuccess || cudaMalloc(&ctx->pf_counters, TC_MAX_ITEMS * sizeof(uint32_t)) != cudaSuccess) {
        cudaGetLastError();
        set_error("out of device memory for the prefill partials (%zu bytes)", bytes);
        return MKV_ERR_NOMEM;
    }
    MKV_CUDA(cudaMemsetAsync(ctx->pf_counters, 0, TC_MAX_ITEMS * sizeof(uint32_t), ctx->stream));
    return MKV_OK;
}

mkv_status launch_prefill_f16_tc(Ctx *ctx, Cache *c, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                                 const void *q, bool q_is_f16, float *out) {
#ifdef MKV_MEASURE
    static const uint32_t phase = [] { const char *e = getenv("MKV_PHASE"); return e ? (uint32_t)atoi(e) : 0u; }();
#else
    const uint32_t phase = 0u;
#endif
    const uint32_t nitems = 2u * ((ntok + 15u) / 16u);
    if (nitems > TC_MAX_ITEMS) {
        set_error("a prefill block of %u tokens is %u work items, at most %u are built", ntok, nitems, TC_MAX_ITEMS);
        return MKV_ERR_INVALID;
    }
    // tiles of all items (the host's copy of PfWork::tiles_of)
    uint64_t tiles = 0;
    for (uint32_t grp = 0; grp < nitems / 2u; grp++)
        tiles += 2ull * ((pos0 + 1u + std::min(grp * 16u + 15u, ntok - 1u) + TC_TILE - 1u) / TC_TILE - first_pos / TC_TILE);
    // MKV_PREFILL_SPLIT=0 keeps one CTA per item (the schedule the persistent grid is measured against)
    static const bool allow_split = [] { const char *e = getenv("MKV_PREFILL_SPLIT"); return !(e && e[0] == '0'); }();
    const bool split = allow_split && 4u * nitems <= 3u * (uint32_t)ctx->sm_count && tiles >= 4ull * (uint64_t)ctx->sm_count;
    const uint32_t grid = split ? (uint32_t)ctx->sm_count : nitems;
    if (split) {
        mkv_status st = prefill_scratch(ctx);
        if (st != MKV_OK) return st;
    }
    const CUtensorMap &km = c->maps_host[2 * (c->n_layers + layer)], &vm = c->maps_host[2 * (c->n_layers + layer) + 1];
    if (q_is_f16)
        prefill_f16_tc_kernel<true><<<grid, 192, TC_SMEM, ctx->stream>>>(km, vm, q, out, first_pos, pos0, ntok, c->shard_first,
                                                                         ctx->pf_scratch, ctx->pf_counters, split ? 1u : 0u, ctx->dev_status, phase);
    else
        prefill_f16_tc_kernel<false><<<grid, 192, TC_SMEM, ctx->stream>>>(km, vm, q, out, first_pos, pos0, ntok, c->shard_first,
                                                                          ctx->pf_scratch, ctx->pf_counters, split ? 1u : 0u, ctx->dev_status, phase);
    ctx->launches++;
    MKV_CUDA(cudaGetLastError());
    return MKV_OK;
}

} // namespace mkv
