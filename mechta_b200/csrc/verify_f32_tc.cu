// Decode / verify attention over the f32 cache on the 5th-generation tensor cores, with f32-grade arithmetic.
//
// Same contract as verify_f32_kernel (stands in for attn_fd / attn_fd2h + attn_fd_combine, W/ops.wgsl:325-538) and the
// same split of every f32 operand into two f16 values, hi = f16(x), lo = f16(x - hi); a product is
// a_hi.b_hi + a_hi.b_lo + a_lo.b_hi with exact f16 x f16 products in f32 accumulators. Same transposed formulation as
// verify_tc.cu: the keys, then the head dims, fill the 128 TMEM lanes, tiles of 128 keys.
//
// The cache tile is converted IN PLACE. TMA brings a sub-tile [128 keys][64 dims] of f32 (32 KB, two blocks of
// [128 keys][32 dims] whose rows are 128 bytes, 128-byte swizzle) into a ring slot; a converter warp rewrites every
// 64-byte half row (16 floats) as 16 hi halves followed by 16 lo halves, so the same 32 KB become an f16 operand tile
// with rows [hi d0-15 | lo d0-15 | hi d16-31 | lo d16-31], and no second buffer is needed: the whole of shared memory
// beside Q and P is ring (five slots, 160 KB in flight).
//   S^T[128 keys][64] = K'_tile . Q'^T     K-major A = the converted K sub-tile, one MMA per 16 halves: an MMA over hi
//                                          halves takes B = [Q hi; Q lo] (N = 64: columns 0-31 get Q_hi.K_hi, columns
//                                          32-63 Q_lo.K_hi), one over lo halves B = Q hi (N = 32: Q_hi.K_lo into 0-31);
//                                          a score is column r + column 32 + r
//   O_t^T[512][64]    = V'_tile^T . P'^T   M-major A = the converted V sub-tile: the 128 TMEM lanes of a block are 64
//                                          dims as [hi 16 | lo 16 | hi 16 | lo 16 | ...]; B = [P hi; P lo] (N = 64);
//                                          an output is the sum of lanes d_hi, d_lo (16 apart: one shuffle) and of
//                                          columns r, 32 + r
// The tensor core's f32 accumulation truncates, so a long chain of accumulations drifts (measured 1.5e-5 over 100+
// tiles in the warp-MMA kernel); every tile's O_t^T therefore starts from zero and the softmax threads fold it into O
// kept in registers with a rounded FMA, O = O * cf + O_t (64 values per thread), which also makes the rescale after
// a move of the reference maxima a register operation.
// Roles (512 threads, four warpgroups whose register budgets are set with setmaxnreg): warp 0 = TMA producer, warp 1 = MMA
// issuer and TMEM owner (warps 2-3 idle), warps 4-11 = converters (four warps per sub-tile, 64 keys of one block each; a ring
// slot always goes to the same four, so each slot's barrier phases are consumed in order), warps 12-15 = softmax (one thread
// per key of the tile) and owners of O. Stream order K0 K1 V0 K2 V1 ... in sub-tiles of four per K or V tile.
// Same pieces, in-kernel merge and programmatic dependent launch as the f16 kernel; every wait is bounded.
#include <stdlib.h>

#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int FT_NSLOT = 5;
#ifndef FT_CONV_UNROLL
#define FT_CONV_UNROLL 2
#endif
#if defined(FT_X_NOMMA) || defined(FT_X_NOQK)
#define FT_X_QK(x) do { (void)a; } while (0)
#else
#define FT_X_QK(x) x
#endif
#if defined(FT_X_NOMMA) || defined(FT_X_NOPV)
#define FT_X_PV(x) do { (void)a; } while (0)
#else
#define FT_X_PV(x) x
#endif
constexpr uint32_t FT_CONV_ITERS = 4, FT_CONV_WARPS = 4; // a sub-tile is converted by four warps: 64 keys of one block each
constexpr int FT_CONV_UNROLL_N = FT_CONV_UNROLL; // half rows a converter lane has in flight
constexpr int FT_THREADS = 512;
constexpr uint32_t FT_SOFTMAX_TID0 = 384;
constexpr uint32_t FT_TILE = 128;                     // keys per tile
constexpr uint32_t FT_SLOT = 32768;                   // sub-tile [128 keys][64 dims] f32 = two blocks of [128 keys][128 bytes]
constexpr uint32_t FT_BLK = 16384;
constexpr uint32_t FT_BOX = 4096;                     // one TMA box [32 keys][32 floats]
constexpr uint32_t FT_OFF_Q = FT_NSLOT * FT_SLOT;     // [4 blocks of 64 dims][64 rows: Q hi 0-31, Q lo 32-63][128 bytes]
constexpr uint32_t FT_QB = 8192;
constexpr uint32_t FT_OFF_P = FT_OFF_Q + 4 * FT_QB;   // 2 buffers of [2 blocks of 64 keys][64 rows: P hi, P lo][128 bytes]
constexpr uint32_t FT_PB = 8192;
constexpr uint32_t FT_PBUF = 2 * FT_PB;
constexpr uint32_t FT_OFF_RED = FT_OFF_P + 2 * FT_PBUF;   // two buffers of [32 rows][4 warps] floats
constexpr uint32_t FT_OFF_REF = FT_OFF_RED + 1024;        // -(reference maximum) of the 32 rows, then the rescale factors
constexpr uint32_t FT_OFF_BAR = FT_OFF_REF + 256;
// barriers: full[NSLOT], conv[NSLOT], empty[NSLOT], s_full[2], p_full[2], o_full, o_free, q_full
constexpr uint32_t FT_NBAR = 3 * FT_NSLOT + 7;
constexpr uint32_t FT_OFF_MISC = FT_OFF_BAR + FT_NBAR * 8;
constexpr uint32_t FT_SMEM = FT_OFF_MISC + 64 + 1024;
constexpr uint32_t FT_COL_S = 0, FT_COL_O = 128, FT_COLS = 512; // S^T: 2 x 64 columns; O_t^T: 4 blocks x 64 columns
constexpr int FT_ROW_OUTSIDE = 1 << 30; // a row coordinate beyond any cache (at most 2^18 + 2^10 rows)
constexpr long long FT_WAIT_LIMIT = 2000000000ll;
constexpr float FT_LOG2E = 1.4426950408889634f;
constexpr float FT_C2 = SCALE * FT_LOG2E;
constexpr float FT_LAZY2 = 8.0f * FT_LOG2E;
constexpr float FT_UNSET = 1.0e30f;
static_assert(FT_SMEM <= 232448, "shared memory of verify_f32_tc_kernel");

struct FtShared {
    uint32_t tmem_base;
    volatile uint32_t abort;
    uint32_t ticket;
};

// Measurement build only: cycles each role spent waiting, summed over the CTAs of all launches since the last read.
#ifdef MKV_MEASURE
enum { FP_CTAS, FP_TOTAL, FP_PDL, FP_PROD_EMPTY, FP_MMA_IDLE, FP_MMA_Q, FP_CONV_FULL, FP_SM_S, FP_SM_O, FP_SM_PDL, FP_FIRST_S,
       FP_MERGE, FP_T_PDL, FP_T_QDONE, FP_T_LASTS, FP_T_FOLDED, FP_T_PUBLISH, FP_T_ROLES, FP_N };
__device__ unsigned long long g_ft_probe[24];
#define FT_PROBE_BEGIN(cond) long long fp_t0 = 0; if (cond) fp_t0 = clock64()
#define FT_PROBE_END(cond, which) do { if (cond) atomicAdd(&g_ft_probe[which], (unsigned long long)(clock64() - fp_t0)); } while (0)
#define FT_STAMP(cond, which) do { if (cond) atomicAdd(&g_ft_probe[which], (unsigned long long)(clock64() - fp_start)); } while (0)
#else
#define FT_STAMP(cond, which) do { } while (0)
#define FT_PROBE_BEGIN(cond) do { } while (0)
#define FT_PROBE_END(cond, which) do { } while (0)
#endif

__device__ __forceinline__ bool ft_wait(uint32_t bar, uint32_t parity, FtShared *sh, uint32_t *status) {
    if (sh->abort) return false;
    if (mbar_wait_bounded(bar, parity, FT_WAIT_LIMIT)) return true;
    sh->abort = 1;
    atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
    return false;
}
// named barrier 1: the 128 softmax threads
__device__ __forceinline__ void ft_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool ft_bar_or(bool x) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "bar.red.or.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"((uint32_t)x)
        : "memory");
    return r != 0;
}
// named barrier 2: all warps, at the end of their roles
__device__ __forceinline__ void ft_bar_roles() { asm volatile("bar.sync 2, 512;" ::: "memory"); }
// as vt_transpose_reduce of verify_tc.cu: v[i] of lane L -> reduction over the lanes of v[L], in lane L
template <bool MAX>
__device__ __forceinline__ float ft_transpose_reduce(float (&v)[32], uint32_t lane) {
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
        const bool up = (lane & (uint32_t)s) != 0;
#pragma unroll
        for (int i = 0; i < s; i++) {
            const float keep = up ? v[i + s] : v[i];
            const float send = up ? v[i] : v[i + s];
            const float got = __shfl_xor_sync(0xffffffffu, send, s);
            v[i] = MAX ? fmaxf(keep, got) : keep + got;
        }
    }
    return v[0];
}
// hi and lo halves of 8 floats as two 16-byte vectors of f16
__device__ __forceinline__ void ft_split8(const float4 &a, const float4 &b, uint4 &hi, uint4 &lo) {
    const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 hh = __floats2half2_rn(x[2 * i], x[2 * i + 1]);
        const float2 hf = __half22float2(hh);
        const __half2 ll = __floats2half2_rn(x[2 * i] - hf.x, x[2 * i + 1] - hf.y);
        h[i] = *reinterpret_cast<const uint32_t *>(&hh);
        l[i] = *reinterpret_cast<const uint32_t *>(&ll);
    }
    hi = make_uint4(h[0], h[1], h[2], h[3]);
    lo = make_uint4(l[0], l[1], l[2], l[3]);
}

template <bool EXT, typename Launch>
__global__ void __launch_bounds__(FT_THREADS, 1)
verify_f32_tc_kernel(const VerifyItem *__restrict__ items, int n_items, const __grid_constant__ Launch single,
                     uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const VerifyItem &it = pick_item(items, n_items, single, blockIdx.x);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t local = blockIdx.x - it.cta_begin;
    if (local >= 2u * it.nsplit) return;
    pdl_launch_dependents();
#ifdef MKV_MEASURE
    const long long fp_start = clock64();
#endif
    const uint32_t kvh = local & 1u, split = local >> 1;
    const uint32_t t0 = it.tile_begin + split * it.tiles_per_split; // in 32-key units
    const uint32_t t1 = min(t0 + it.tiles_per_split, it.tile_end);
    const uint32_t k_begin = t0 * TILE32, k_end = t1 * TILE32;
    const uint32_t nt = (k_end - k_begin + FT_TILE - 1u) / FT_TILE;
    const uint32_t nsub = 8u * nt; // four sub-tiles per K tile and per V tile
    const CUtensorMap *kmap = launch_map(items, it, single, false), *vmap = launch_map(items, it, single, true);
    const uint32_t bar0 = smem_base + FT_OFF_BAR;
    const uint32_t bar_full = bar0, bar_conv = bar_full + 8u * FT_NSLOT, bar_empty = bar_conv + 8u * FT_NSLOT;
    const uint32_t bar_s_full = bar_empty + 8u * FT_NSLOT, bar_p_full = bar_s_full + 16u, bar_o_full = bar_p_full + 16u;
    const uint32_t bar_o_free = bar_o_full + 8u, bar_q_full = bar_o_free + 8u;
    FtShared *sh = reinterpret_cast<FtShared *>(smem + FT_OFF_MISC);

    // The stream: units K0 K1 V0 K2 V1 K3 V2 ... (K one tile ahead of V, so that the softmax of a tile is over by the
    // time its V has been converted), each unit four sub-tiles (dims 0-63, 64-127, 128-191, 192-255); sub-tile n goes
    // to ring slot n % NSLOT.
    auto unit = [&](uint32_t u, bool &is_v) -> uint32_t { // the tile of unit u
        if (u == 0u) { is_v = false; return 0u; }
        if ((u & 1u) == 0u) { is_v = true; return (u - 2u) >> 1; }
        const uint32_t j = (u + 1u) >> 1;
        is_v = j >= nt;
        return is_v ? nt - 1u : j;
    };
    auto unit_k = [&](uint32_t j) { return j < 2u ? j : 2u * j - 1u; };                       // where K of tile j sits in the stream
    auto unit_v = [&](uint32_t j) { return j + 1u == nt ? 2u * nt - 1u : 2u * j + 2u; };      // and V of tile j

    if (tid == 0) {
        for (int i = 0; i < FT_NSLOT; i++) {
            mbar_init(bar_full + 8u * i, 1);
            mbar_init(bar_conv + 8u * i, FT_CONV_WARPS);
            mbar_init(bar_empty + 8u * i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_s_full + 8u * i, 1);
            mbar_init(bar_p_full + 8u * i, 128);
        }
        mbar_init(bar_o_full, 1);
        mbar_init(bar_o_free, 128);
        mbar_init(bar_q_full, 128);
        sh->abort = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    if (warp == 1) tmem_alloc(smem_base + FT_OFF_MISC, FT_COLS); // writes sh->tmem_base
    tc_fence_before();
    __syncthreads(); // the barriers and the TMEM address are there for every role; nothing global has been touched yet
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    if (warp < 4) {
      asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
      if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool waited = false; // griddepcontrol.wait passed: rows the kernels in front may have written can be loaded
            for (uint32_t n = 0; n < nsub; n++) {
                const uint32_t slot = n % FT_NSLOT;
                bool is_v;
                const uint32_t tile = unit(n >> 2, is_v), sub = n & 3u;
                const uint32_t key0 = k_begin + tile * FT_TILE;
                // tiles wholly below safe_below hold rows no kernel still in flight writes: their loads start at once
                if (!waited && key0 + FT_TILE > it.safe_below) {
                    FT_PROBE_BEGIN(true);
                    pdl_wait();
                    FT_PROBE_END(true, FP_PDL);
                    waited = true;
                }
                // a slot comes back through the MMAs, which need the queries: the same rule for the first bounded wait here
                if (n >= (uint32_t)FT_NSLOT && !waited) {
                    pdl_wait();
                    waited = true;
                }
                FT_PROBE_BEGIN(true);
                if (n >= (uint32_t)FT_NSLOT && !ft_wait(bar_empty + 8u * slot, ((n / FT_NSLOT) - 1u) & 1u, sh, status)) break;
                FT_PROBE_END(true, FP_PROD_EMPTY);
                const uint32_t bar = bar_full + 8u * slot, dst = smem_base + slot * FT_SLOT;
                const CUtensorMap *map = is_v ? vmap : kmap;
                const int x = (int)(kvh * 256u + sub * 64u);
                mbar_expect_tx(bar, FT_SLOT);
#pragma unroll
                for (int kb = 0; kb < 4; kb++) { // four boxes of 32 keys; in a ring cache each may wrap on its own
                    // boxes wholly past this CTA's keys (a piece need not be a whole number of tiles) are not fetched: a row
                    // far outside the tensor makes TMA fill them with zeros without touching memory; the keys are masked
                    const uint32_t kk = key0 + 32u * kb;
                    const int y = kk >= k_end ? FT_ROW_OUTSIDE : (int)(EXT ? cache_row(it, kk) : kk - it.row0);
                    tma_load_2d(dst + kb * FT_BOX, map, x, y, bar);
                    tma_load_2d(dst + FT_BLK + kb * FT_BOX, map, x + 32, y, bar);
                }
            }
        }
      } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t IDESC_QK64 = tc_idesc_f16(128, 64, false, false);
            constexpr uint32_t IDESC_QK32 = tc_idesc_f16(128, 32, false, false);
            constexpr uint32_t IDESC_PV = tc_idesc_f16(128, 64, false, true);
            const uint32_t qb = smem_base + FT_OFF_Q, pb = smem_base + FT_OFF_P;
            // No bounded wait may start before the launch in front has finished, however long that takes: the queries come
            // after it, and everything below waits for them in the end.
            pdl_wait();
            FT_PROBE_BEGIN(true);
            bool ok = ft_wait(bar_q_full, 0, sh, status);
            FT_PROBE_END(true, FP_MMA_Q);
            tc_fence_after();
            // Event loop over sub-tiles: whichever of "the next K sub-tile is converted (and its S^T buffer is free)"
            // and "the next V sub-tile is converted, its P^T written and O_t^T free" holds first is issued first.
            uint32_t kq = 0, vq = 0; // next K sub-tile (tile kq / 4, part kq % 4), next V sub-tile
            // A slot's barrier may only be tested for the use after the last one consumed here (a parity test two uses
            // ahead is satisfied by the use before last): sub-tile n is the next use of its slot once n - NSLOT is consumed.
            auto consumed = [&](uint32_t n) {
                if (n < (uint32_t)FT_NSLOT) return true;
                bool is_v;
                const uint32_t m = n - FT_NSLOT, t = unit(m >> 2, is_v), q = 4u * t + (m & 3u);
                return is_v ? vq > q : kq > q;
            };
            long long tlast = clock64();
            while (ok && vq < 4u * nt) {
                bool did = false;
                if (kq < 4u * nt) {
                    const uint32_t j = kq >> 2, p = kq & 3u, n = 4u * unit_k(j) + p, slot = n % FT_NSLOT;
                    // S^T buffer j & 1 is free once the softmax of tile j - 2 has published its P^T
                    const bool s_free = j < 2u || p != 0u || mbar_test(bar_p_full + 8u * (j & 1u), ((j >> 1) - 1u) & 1u);
                    if (s_free && consumed(n) && mbar_test(bar_conv + 8u * slot, (n / FT_NSLOT) & 1u)) {
                        tc_fence_after();
                        const uint32_t kb = smem_base + slot * FT_SLOT, d = tmem + FT_COL_S + 64u * (j & 1u);
#pragma unroll
                        for (uint32_t b = 0; b < 2u; b++)     // block of 32 dims
#pragma unroll
                            for (uint32_t s = 0; s < 4u; s++) { // hi d0-15, lo d0-15, hi d16-31, lo d16-31
                                const uint32_t dim = 64u * p + 32u * b + 16u * (s >> 1); // first of the 16 dims
                                const uint64_t a = tc_desc_sw128(kb + b * FT_BLK + s * 32u, 16, 1024);
                                const uint64_t q = tc_desc_sw128(qb + (dim >> 6) * FT_QB + (dim & 63u) * 2u, 16, 1024);
                                FT_X_QK(tc_mma_f16(d, a, q, (s & 1u) ? IDESC_QK32 : IDESC_QK64, (p | b | s) ? 1u : 0u));
                            }
                        tc_commit(bar_empty + 8u * slot); // the sub-tile's slot is free
                        if (p == 3u) tc_commit(bar_s_full + 8u * (j & 1u));
                        kq++;
                        did = true;
                    }
                }
                {
                    const uint32_t j = vq >> 2, p = vq & 3u, n = 4u * unit_v(j) + p, slot = n % FT_NSLOT;
                    // tile j's scores must be complete (its K sub-tiles all issued), its P^T written, and O_t^T folded
                    // away by the softmax threads (tile j - 1) before the first sub-tile of the tile overwrites it
                    bool go = (kq >> 2) > j && consumed(n) && mbar_test(bar_conv + 8u * slot, (n / FT_NSLOT) & 1u) &&
                              mbar_test(bar_p_full + 8u * (j & 1u), (j >> 1) & 1u);
                    if (go && p == 0u && j > 0u) go = mbar_test(bar_o_free, (j - 1u) & 1u);
                    if (go) {
                        tc_fence_after();
                        const uint32_t vb = smem_base + slot * FT_SLOT, pbj = pb + (j & 1u) * FT_PBUF;
#pragma unroll
                        for (uint32_t ks = 0; ks < 8u; ks++) { // 16 keys per MMA
                            // V'^T, M-major: the second block of 32 dims one block on, the next 8 keys 1024 bytes on
                            const uint64_t a = tc_desc_sw128(vb + ks * 2048u, FT_BLK, 1024);
                            const uint64_t b = tc_desc_sw128(pbj + (ks >> 2) * FT_PB + (ks & 3u) * 32u, 16, 1024);
                            FT_X_PV(tc_mma_f16(tmem + FT_COL_O + 64u * p, a, b, IDESC_PV, ks ? 1u : 0u));
                        }
                        tc_commit(bar_empty + 8u * slot);
                        if (p == 3u) tc_commit(bar_o_full); // O_t^T of tile j is complete; P^T buffer j & 1 may be overwritten
                        vq++;
                        did = true;
                    }
                }
                if (did) {
#ifdef MKV_MEASURE
                    atomicAdd(&g_ft_probe[FP_MMA_IDLE], (unsigned long long)(clock64() - tlast));
#endif
                    tlast = clock64();
                } else if (sh->abort || clock64() - tlast > FT_WAIT_LIMIT) {
                    if (!sh->abort) {
                        sh->abort = 1;
                        atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
                    }
                    break;
                }
            }
        }
      }
      __syncwarp(); // the lanes that had no role wait here for the one that had: the barrier below wants whole warps
      ft_bar_roles(); // registers come back only after the softmax warps have returned theirs (see there)
      asm volatile("setmaxnreg.inc.sync.aligned.u32 128;");
    } else if (warp < 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
        // ---------------- converters: f32 sub-tile -> f16 hi / lo operand tile, in place ----------------
        // Every use of a ring slot is converted by the same four warps, in order (a barrier's phases must be waited for in
        // order by whoever waits on it).
        const uint32_t c = (warp - 4u) >> 2, blk = warp & 1u, rbase = 64u * ((warp >> 1) & 1u);
        for (uint32_t n = 0; n < nsub; n++) {
            if (((n % FT_NSLOT) & 1u) != c) continue; // slots 0, 2, 4 -> the first four warps, 1, 3 -> the other four
            const uint32_t slot = n % FT_NSLOT;
            // the sub-tiles beyond the first ring-full are loaded once slots come back, i.e. after the queries: as above
            if (n >= (uint32_t)FT_NSLOT && n < 2u * FT_NSLOT) pdl_wait();
            FT_PROBE_BEGIN(tid == 128u);
            if (!__all_sync(0xffffffffu, ft_wait(bar_full + 8u * slot, (n / FT_NSLOT) & 1u, sh, status))) break;
            FT_PROBE_END(tid == 128u, FP_CONV_FULL);
            uint8_t *base = smem + slot * FT_SLOT;
            // 128 half rows of 64 bytes for this warp; a lane takes half row (row = rbase + i * 16 + lane / 2, half = lane % 2)
#ifndef FT_X_NOCONV
#pragma unroll FT_CONV_UNROLL_N
            for (uint32_t i = 0; i < FT_CONV_ITERS; i++) {
                const uint32_t row = rbase + i * 16u + (lane >> 1), half = lane & 1u;
                uint8_t *r = base + blk * FT_BLK + row * 128u;
                const uint32_t x = row & 7u, c0 = 4u * half;
                float4 f[4];
#pragma unroll
                for (int q = 0; q < 4; q++) f[q] = *reinterpret_cast<const float4 *>(r + (((c0 + q) ^ x) << 4));
                uint4 h0, l0, h1, l1;
                ft_split8(f[0], f[1], h0, l0);
                ft_split8(f[2], f[3], h1, l1);
                *reinterpret_cast<uint4 *>(r + (((c0 + 0u) ^ x) << 4)) = h0;
                *reinterpret_cast<uint4 *>(r + (((c0 + 1u) ^ x) << 4)) = h1;
                *reinterpret_cast<uint4 *>(r + (((c0 + 2u) ^ x) << 4)) = l0;
                *reinterpret_cast<uint4 *>(r + (((c0 + 3u) ^ x) << 4)) = l1;
            }
#endif
            fence_proxy_async(); // the tensor core reads the tile through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_conv + 8u * slot);
        }
        __syncwarp();
        ft_bar_roles();
        asm volatile("setmaxnreg.inc.sync.aligned.u32 128;");
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
        // ---------------- softmax: one thread per key of the tile (TMEM lane); owners of O ----------------
        const uint32_t w4 = warp & 3u; // the warp's TMEM lane group
        const uint32_t klane = 32u * w4 + lane, lane_addr = (32u * w4) << 16;
        // Q of this KV head towards L2 while the kernel waits for its predecessor: 8 KB per token, two 128-byte lines per thread
#pragma unroll
        for (uint32_t i = 0; i < 2u; i++) {
            const uint32_t line = (tid - FT_SOFTMAX_TID0) + 128u * i; // 64 lines per token
            if (line < 64u * it.ntok) prefetch_l2(it.q + (size_t)(line >> 6) * 4096u + (size_t)kvh * 2048u + (size_t)(line & 63u) * 32u);
        }
        {
            FT_PROBE_BEGIN(tid == FT_SOFTMAX_TID0);
            pdl_wait(); // Q and every global write come after this
            FT_PROBE_END(tid == FT_SOFTMAX_TID0, FP_SM_PDL);
            FT_STAMP(tid == FT_SOFTMAX_TID0, FP_T_PDL);
        }
        // Q of this KV head to shared memory as f16 hi (rows 0-31) and lo (rows 32-63), the B operands of S^T:
        // row = tok * 8 + head % 8 (the order of q_dmx, M/dmx.rs:128-138), rows of tokens >= ntok zero; per 64-dim block
        // [64 rows][128 bytes], 128-byte swizzle. All loads of a thread go out before the first conversion.
        {
            const uint32_t st = tid - FT_SOFTMAX_TID0; // 0..127: 1024 chunks of 8 dims, eight per thread
            float4 qa[8], qbv[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t idx = st + 128u * i, row = idx >> 5, chunk = idx & 31u, tok = row >> 3;
                qa[i] = qbv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (tok < it.ntok) {
                    const float4 *src = reinterpret_cast<const float4 *>(it.q + (size_t)tok * 4096u +
                                                                         (size_t)(8u * kvh + (row & 7u)) * 256u + chunk * 8u);
                    qa[i] = __ldcg(src);
                    qbv[i] = __ldcg(src + 1);
                }
            }
            uint8_t *qs = smem + FT_OFF_Q;
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t idx = st + 128u * i, row = idx >> 5, chunk = idx & 31u;
                uint4 hi, lo;
                ft_split8(qa[i], qbv[i], hi, lo);
                uint8_t *blk = qs + (chunk >> 3) * FT_QB;
                *reinterpret_cast<uint4 *>(blk + swz128(row, chunk & 7u)) = hi;
                *reinterpret_cast<uint4 *>(blk + swz128(32u + row, chunk & 7u)) = lo;
            }
            fence_proxy_async();
            mbar_arrive(bar_q_full);
            FT_STAMP(tid == FT_SOFTMAX_TID0, FP_T_QDONE);
        }
        // token t of the step sees lowest_key(t) <= key < min(pos + 1 + t, end of the shard, end of this piece)
        const uint32_t klo = max(it.first_pos, it.key_lo);
        uint32_t lim[4];
#pragma unroll
        for (uint32_t t = 0; t < 4u; t++) lim[t] = min(min(it.pos + 1u + t, it.key_hi), k_end);
        const uint32_t lo_max = EXT ? lowest_key(it, 3u) : klo;
        // -(reference maximum) of the rows (base-2 units) and the rescale factors live in shared memory (all threads
        // hold the same 32 values); this thread's share of the row sums and of O live in registers
        float *ref = reinterpret_cast<float *>(smem + FT_OFF_REF), *cfs = ref + 32;
        if (klane < 32u) ref[klane] = FT_UNSET;
        float lpart[32];
#pragma unroll
        for (int r = 0; r < 32; r++) lpart[r] = 0.0f;
        // O: this thread's lane is (block of 32 dims b = w4 / 2, hi or lo half of 16 dims h = lane / 16 of pair w4 % 2);
        // after the exchange with lane ^ 16 it owns, for each of the four 64-dim parts, its dim and 16 of the 32 rows
        float O[4][16];
#pragma unroll
        for (int p = 0; p < 4; p++)
#pragma unroll
            for (int i = 0; i < 16; i++) O[p][i] = 0.0f;
        const uint32_t my_dim = 32u * (w4 >> 1) + 16u * (w4 & 1u) + (lane & 15u); // + 64 p
        const uint32_t my_row0 = (lane & 16u);                                      // rows my_row0 .. my_row0 + 15
        float *red_base = reinterpret_cast<float *>(smem + FT_OFF_RED);
        uint32_t red_turn = 0;
        // P'^T[row][key]: this thread's column, 2 bytes in each of the 64 rows (K-major B operand, 128-byte swizzle)
        uint8_t *pcol = smem + FT_OFF_P + (klane >> 6) * FT_PB + (klane & 7u) * 2u;
        const uint32_t kchunk = (klane & 63u) >> 3;
        ft_bar_sync(); // ref[] is initialised
        bool stopped = false;
        uint32_t folded = 0; // tiles whose O_t^T has been folded into O
        auto fold = [&](uint32_t j) -> bool { // O = O + O_t^T of tile j (the rescale for a moved maximum was applied before)
            FT_PROBE_BEGIN(tid == FT_SOFTMAX_TID0);
            bool ok = __all_sync(0xffffffffu, ft_wait(bar_o_full, j & 1u, sh, status));
            FT_PROBE_END(tid == FT_SOFTMAX_TID0, FP_SM_O);
            tc_fence_after();
            if (ok) {
#pragma unroll
                for (uint32_t p = 0; p < 4u; p++) {
                    uint32_t a[32], b[32];
                    tmem_ld32(tmem + lane_addr + FT_COL_O + 64u * p, a);
                    tmem_ld32(tmem + lane_addr + FT_COL_O + 64u * p + 32u, b);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        // this lane's sums over P hi and P lo for rows i and 16 + i; the partner lane (the other half of
                        // the hi / lo pair of this dim) needs the one this lane does not keep
                        const float u0 = __uint_as_float(a[i]) + __uint_as_float(b[i]);
                        const float u1 = __uint_as_float(a[16 + i]) + __uint_as_float(b[16 + i]);
                        const float mine = my_row0 ? u1 : u0, send = my_row0 ? u0 : u1;
                        const float got = __shfl_xor_sync(0xffffffffu, send, 16);
                        O[p][i] += mine + got;
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_o_free);
            return ok;
        };
        for (uint32_t j = 0; j < nt; j++) {
            // a warp takes every wait's outcome together: the TMEM loads are warp-collective
            FT_PROBE_BEGIN(tid == FT_SOFTMAX_TID0);
            bool ok = __all_sync(0xffffffffu, ft_wait(bar_s_full + 8u * (j & 1u), (j >> 1) & 1u, sh, status));
            FT_PROBE_END(tid == FT_SOFTMAX_TID0, FP_SM_S);
#ifdef MKV_MEASURE
            if (tid == FT_SOFTMAX_TID0 && j == 0u) atomicAdd(&g_ft_probe[FP_FIRST_S], (unsigned long long)(clock64() - fp_start));
            FT_STAMP(tid == FT_SOFTMAX_TID0 && j + 1u == nt, FP_T_LASTS);
#endif
            tc_fence_after();
            float t[32];
            {
                uint32_t s0[32], s1[32];
                tmem_ld32(tmem + lane_addr + FT_COL_S + 64u * (j & 1u), s0);
                tmem_ld32(tmem + lane_addr + FT_COL_S + 64u * (j & 1u) + 32u, s1);
                tmem_wait_ld();
                const uint32_t tile_lo = k_begin + j * FT_TILE, key = tile_lo + klane;
                const bool masked = tile_lo < lo_max || tile_lo + FT_TILE > lim[0];
#pragma unroll
                for (int r = 0; r < 32; r++) {
                    const float s = (__uint_as_float(s0[r]) + __uint_as_float(s1[r])) * FT_C2; // scale, then mask (W/ops.wgsl:361)
                    bool seen = true;
                    if (masked) seen = key >= (EXT ? lowest_key(it, (uint32_t)r >> 3) : klo) && key < lim[r >> 3];
                    t[r] = seen ? s : NEG_BIG;
                }
            }
            bool over = false;
            {
                const float4 *r4 = reinterpret_cast<const float4 *>(ref);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float4 n4 = r4[q];
                    over |= t[4 * q] + n4.x > FT_LAZY2 || t[4 * q + 1] + n4.y > FT_LAZY2 || t[4 * q + 2] + n4.z > FT_LAZY2 ||
                            t[4 * q + 3] + n4.w > FT_LAZY2;
                }
            }
            if (ft_bar_or(over || !ok)) {
                if (ft_bar_or(!ok)) { // a wait ran out somewhere: all 128 threads leave together
                    stopped = true;
                    break;
                }
                // Move the reference maxima to the true maxima so far (the reference's running maximum, W/ops.wgsl:366-372,
                // taken lazily). The warp's transposing reduction leaves the maximum of row L over the warp's 32 keys in
                // lane L; after the four warps have met, the threads of lanes 0..31 of the first warp work out row L's new
                // reference and rescale factor and publish them.
                float *red = red_base + 128u * (red_turn & 1u);
                {
                    float mx[32];
#pragma unroll
                    for (int r = 0; r < 32; r++) mx[r] = t[r];
                    red[w4 * 32u + lane] = ft_transpose_reduce<true>(mx, lane);
                }
                ft_bar_sync();
                if (klane < 32u) {
                    const float mt = fmaxf(fmaxf(red[klane], red[32u + klane]), fmaxf(red[64u + klane], red[96u + klane]));
                    const float old = ref[klane];
                    float cf = 1.0f;
                    if (mt > NEG_TEST) {
                        const bool set = old < 0.5f * FT_UNSET;
                        const float m_new = set ? fmaxf(-old, mt) : mt;
                        if (set) cf = exp2f(-old - m_new);
                        ref[klane] = -m_new;
                    }
                    cfs[klane] = cf;
                }
                red_turn++;
                // O must hold every tile whose weights used the old references before it is rescaled
                if (folded < j) {
                    ok = fold(folded);
                    folded++;
                }
                ft_bar_sync(); // ref[] and cfs[] are published
                if (ft_bar_or(!ok)) {
                    stopped = true;
                    break;
                }
                {
                    const float4 *c4 = reinterpret_cast<const float4 *>(cfs);
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const float4 c = c4[q];
                        lpart[4 * q] *= c.x; lpart[4 * q + 1] *= c.y; lpart[4 * q + 2] *= c.z; lpart[4 * q + 3] *= c.w;
                    }
                    const float4 *o4 = c4 + (my_row0 >> 2);
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const float4 c = o4[q];
#pragma unroll
                        for (int p = 0; p < 4; p++) {
                            O[p][4 * q] *= c.x; O[p][4 * q + 1] *= c.y; O[p][4 * q + 2] *= c.z; O[p][4 * q + 3] *= c.w;
                        }
                    }
                }
            }
            // weights 2^(t - m) as hi + lo halves; the row sums run over the f32 weights
            {
                const float4 *r4 = reinterpret_cast<const float4 *>(ref);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float4 n4 = r4[q];
                    const float nm[4] = {n4.x, n4.y, n4.z, n4.w};
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int r = 4 * q + e;
                        float w;
                        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(t[r] + nm[e]));
                        lpart[r] += w;
                        const __half h = __float2half_rn(w);
                        const __half l = __float2half_rn(w - __half2float(h));
                        uint8_t *dst = pcol + (j & 1u) * FT_PBUF + ((kchunk ^ (uint32_t)(r & 7)) << 4);
                        *reinterpret_cast<__half *>(dst + r * 128u) = h;
                        *reinterpret_cast<__half *>(dst + (32u + r) * 128u) = l;
                    }
                }
            }
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar_p_full + 8u * (j & 1u));
            // the tile before this one is folded while this tile's V is on its way (its P^T buffer is this tile's next one)
            if (folded < j) {
                ok = fold(folded) && ok;
                folded++;
                if (!__all_sync(0xffffffffu, ok)) {
                    // the other warps find out at their next wait (the abort flag is set)
                }
            }
        }
        // ---------------- the piece's partial: [m, l] per row and O[32][256] ----------------
        if (!stopped) {
            bool ok = true;
            while (folded < nt && ok) {
                ok = fold(folded);
                folded++;
            }
            FT_STAMP(tid == FT_SOFTMAX_TID0, FP_T_FOLDED);
            const size_t piece = (size_t)kvh * it.nsplit + split;
            float *red = red_base + 128u * (red_turn & 1u);
            red[lane * 4u + w4] = ft_transpose_reduce<false>(lpart, lane);
            ft_bar_sync();
            if (w4 == 0) {
                const float4 x = *reinterpret_cast<const float4 *>(red + 4 * lane);
                const float mrow = ref[lane];
                const float m = mrow < 0.5f * FT_UNSET ? -mrow * 0.6931471805599453f : NEG_BIG; // back to natural units
                reinterpret_cast<float2 *>(it.part_ml)[piece * 32u + lane] = make_float2(m, (x.x + x.y) + (x.z + x.w));
            }
            float *po = it.part_o + piece * 32u * 256u + my_dim;
#pragma unroll
            for (int p = 0; p < 4; p++)
#pragma unroll
                for (int i = 0; i < 16; i++) po[(size_t)(my_row0 + i) * 256u + 64u * p] = ok ? O[p][i] : 0.0f;
        }
        // the piece is published by the threads that wrote it, before the CTA's teardown (see verify_tc.cu)
        ft_bar_sync();
        if (tid == FT_SOFTMAX_TID0) sh->ticket = publish_piece(it);
        FT_STAMP(tid == FT_SOFTMAX_TID0, FP_T_PUBLISH);
        // The other warpgroups take their registers back (for the code all warps share) only behind this barrier: a warp
        // that asked earlier, e.g. an idle one at once, could take what the softmax warp of its scheduler still waits for
        // at the top of this branch, and that warp would wait for ever.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 128;");
        ft_bar_roles();
    }

    // ---------------- teardown: nothing of this CTA may still be in flight, then free the tensor memory ----------------
    tc_fence_before();
    __syncthreads();
    if (sh->abort && tid == 0) {
        // a wait ran out somewhere: give copies already issued into this CTA's shared memory a bounded time to land
        for (int s = 0; s < FT_NSLOT; s++) mbar_wait_bounded(bar_full + 8u * s, 0, 200000000ll);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, FT_COLS);
    }
    // this CTA's share of the merge, if its ticket gives it one (scratch in the ring, which is drained by now)
#ifdef MKV_MEASURE
    const long long fp_merge = clock64();
    FT_STAMP(tid == 0, FP_T_ROLES);
#endif
    finish_item<FT_THREADS, EXT>(it, *reinterpret_cast<FinishSmem *>(smem), status, sh->ticket);
#ifdef MKV_MEASURE
    if (tid == 0) {
        const long long now = clock64();
        atomicAdd(&g_ft_probe[FP_CTAS], 1ull);
        atomicAdd(&g_ft_probe[FP_TOTAL], (unsigned long long)(now - fp_start));
        atomicAdd(&g_ft_probe[FP_MERGE], (unsigned long long)(now - fp_merge));
    }
#endif
}

#ifdef MKV_MEASURE
// Measurement build only: copies the 24 role counters of verify_f32_tc_kernel to `out24` and clears them.
extern "C" int mkv_measure_f32_roles(unsigned long long *out24) {
    if (cudaMemcpyFromSymbol(out24, g_ft_probe, sizeof g_ft_probe) != cudaSuccess) return 1;
    const unsigned long long zero[24] = {};
    return cudaMemcpyToSymbol(g_ft_probe, zero, sizeof zero) != cudaSuccess;
}
#endif

mkv_status verify_f32_tc_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_tc_kernel<false, VerifyLaunch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_tc_kernel<true, VerifyLaunch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_tc_kernel<false, VerifyLaunchBatch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_tc_kernel<true, VerifyLaunchBatch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM));
    return MKV_OK;
}

template <typename Launch>
static mkv_status launch_verify_f32_tc_any(Ctx *ctx, const VerifyItem *items_dev, int n, const Launch &single, uint32_t total_ctas, bool ext) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(total_ctas);
    cfg.blockDim = dim3(FT_THREADS);
    cfg.dynamicSmemBytes = FT_SMEM;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (ext) MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_tc_kernel<true, Launch>, items_dev, n, single, ctx->dev_status));
    else MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_tc_kernel<false, Launch>, items_dev, n, single, ctx->dev_status));
    ctx->launches++;
    return MKV_OK;
}

mkv_status launch_verify_f32_tc(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas, bool ext) {
    return launch_verify_f32_tc_any(ctx, items_dev, n, single, total_ctas, ext);
}

// a few items in the parameter space (see VerifyLaunchBatch)
mkv_status launch_verify_f32_tc_few(Ctx *ctx, const VerifyLaunchBatch &few, int n, uint32_t total_ctas, bool ext) {
    return launch_verify_f32_tc_any(ctx, static_cast<const VerifyItem *>(nullptr), n, few, total_ctas, ext);
}

} // namespace mkv
