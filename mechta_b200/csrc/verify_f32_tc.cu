// Decode / verify attention over the f32 cache on the 5th-generation tensor cores, with f32-grade arithmetic.
//
// Same contract and same split of every f32 operand into two f16 values as verify_f32_kernel (hi = f16(x),
// lo = f16(x - hi); a product is a_hi.b_hi + a_hi.b_lo + a_lo.b_hi, exact f16 x f16 products in f32 accumulators),
// same transposed formulation as verify_tc.cu (keys, then head dims, in the TMEM lanes), for 64-key tiles:
//   S^T[64 keys][32 rows]    = K_tile . Q^T      M = 64: row i of the accumulator lives in TMEM lane 32 (i / 16) + i % 16
//   O_t^T[256 dims][32 rows] = V_tile^T . P^T    per tile, M = 128 twice
// Roles (256 threads): warp 0 = TMA producer of raw f32 sub-tiles ([64 keys][128 dims], 32 KB), warps 2-3 = converters
// (one thread per key: 8 floats -> 8 hi + 8 lo halves at a time, written in the 128-byte-swizzled operand layout),
// warp 1 = MMA issuer and TMEM owner, warps 4-7 = softmax (the 16 low lanes of each warp hold a key's 32 scores)
// and the owners of O: the tensor core's f32 accumulation truncates, so a long chain of accumulations drifts
// (measured 1.5e-5 over 100+ tiles in the warp-MMA kernel); here every tile's O_t^T starts from zero and the
// softmax threads fold it into O kept in registers with a rounded FMA, O = O * cf + O_t (thread = head dim, 64
// values), which also makes the rescale after a move of the reference maxima a register operation. The small
// product terms get their own accumulators and are added in the same fold.
#include <stdlib.h>

#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int FT_NRAW = 3;                            // ring of raw sub-tiles
constexpr int FT_NOP = 2;                             // converted operand buffers
constexpr uint32_t FT_TILE = 64;                      // keys per tile
constexpr uint32_t FT_SUB = 32768;                    // raw sub-tile: 8 boxes [32 keys][32 floats]; converted: hi 16 KB + lo 16 KB
constexpr uint32_t FT_BOX = 4096;
constexpr uint32_t FT_HBLK = 8192;                    // converted: one block [64 keys][64 dims] f16
constexpr uint32_t FT_OFF_OP = FT_NRAW * FT_SUB;
constexpr uint32_t FT_OFF_Q = FT_OFF_OP + FT_NOP * FT_SUB;   // Q hi then Q lo: [4 dim blocks][32 rows][64 dims] f16 each
constexpr uint32_t FT_QB = 4096;
constexpr uint32_t FT_OFF_P = FT_OFF_Q + 32768;       // 2 buffers of P^T hi, lo: [32 rows][64 keys] f16 each
constexpr uint32_t FT_PBUF = 8192;
constexpr uint32_t FT_OFF_RED = FT_OFF_P + 2 * FT_PBUF;
constexpr uint32_t FT_OFF_BAR = FT_OFF_RED + 1024;
// barriers: raw_full[NRAW], raw_empty[NRAW], op_full[NOP], op_empty[NOP], s_full[2], p_full[2], o_full[3], o_free[3]
constexpr uint32_t FT_NBAR = 2 * FT_NRAW + 2 * FT_NOP + 10;
constexpr uint32_t FT_OFF_MISC = FT_OFF_BAR + FT_NBAR * 8;
constexpr uint32_t FT_SMEM = FT_OFF_MISC + 64 + 1024;
// TMEM columns: S^T main and small x 2 buffers, then three O_t buffers (so that folding a tile into the registers is
// never what the next product waits for), each: main half 0, main half 1, small half 0, small half 1
constexpr uint32_t FT_COL_S = 0, FT_COL_O = 128, FT_COLS = 512;
constexpr long long FT_WAIT_LIMIT = 2000000000ll;
constexpr float FT_LOG2E = 1.4426950408889634f;
constexpr float FT_C2 = SCALE * FT_LOG2E;
constexpr float FT_LAZY2 = 8.0f * FT_LOG2E;
constexpr float FT_UNSET = 1.0e30f;

struct FtShared {
    uint32_t tmem_base;
    volatile uint32_t abort;
};

__device__ __forceinline__ bool ft_wait(uint32_t bar, uint32_t parity, FtShared *sh, uint32_t *status) {
    if (sh->abort) return false;
    if (mbar_wait_bounded(bar, parity, FT_WAIT_LIMIT)) return true;
    sh->abort = 1;
    atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
    return false;
}
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

template <bool EXT>
__global__ void __launch_bounds__(256, 1)
verify_f32_tc_kernel(const VerifyItem *__restrict__ items, int n_items, const __grid_constant__ VerifyLaunch single,
                     uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const VerifyItem &it = pick_item(items, n_items, single.item, blockIdx.x);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t local = blockIdx.x - it.cta_begin;
    if (local >= 2u * it.nsplit) return;
    const uint32_t ph = MKV_PHASE_OF(it);
    if (ph == 2u) return;
    pdl_launch_dependents();
    const uint32_t kvh = local & 1u, split = local >> 1;
    const uint32_t t0 = it.tile_begin + split * it.tiles_per_split; // in 32-key units
    const uint32_t t1 = min(t0 + it.tiles_per_split, it.tile_end);
    const uint32_t k_begin = t0 * TILE32, k_end = t1 * TILE32;
    const uint32_t nt = ph == 3u ? 0u : (k_end - k_begin + FT_TILE - 1u) / FT_TILE;
    const uint32_t nsub = 4u * nt; // sub-tiles: K dims 0..127, K dims 128..255, V dims 0..127, V dims 128..255 per tile
    const CUtensorMap *kmap = items ? it.kmap : &single.kmap, *vmap = items ? it.vmap : &single.vmap;
    const uint32_t bar0 = smem_base + FT_OFF_BAR;
    const uint32_t bar_raw_full = bar0, bar_raw_empty = bar_raw_full + 8u * FT_NRAW, bar_op_full = bar_raw_empty + 8u * FT_NRAW;
    const uint32_t bar_op_empty = bar_op_full + 8u * FT_NOP, bar_s_full = bar_op_empty + 8u * FT_NOP;
    const uint32_t bar_p_full = bar_s_full + 16u, bar_o_full = bar_p_full + 16u, bar_o_free = bar_o_full + 24u;
    FtShared *sh = reinterpret_cast<FtShared *>(smem + FT_OFF_MISC);

    // The stream of raw sub-tiles: items K0 K1 V0 K2 V1 K3 V2 ... (K one tile ahead of V, so that the softmax of a tile
    // is over by the time its V has been converted), each item two sub-tiles: dims 0..127, then dims 128..255.
    auto item = [&](uint32_t n, bool &is_v) -> uint32_t { // the tile of item n
        if (n == 0u) { is_v = false; return 0u; }
        if ((n & 1u) == 0u) { is_v = true; return (n - 2u) >> 1; }
        const uint32_t j = (n + 1u) >> 1;
        is_v = j >= nt;
        return is_v ? nt - 1u : j;
    };
    // boxes of a sub-tile: [dim box d of the half][key half kb]
    auto issue = [&](uint32_t s) {
        const uint32_t slot = s % FT_NRAW, bar = bar_raw_full + 8u * slot, dst = smem_base + slot * FT_SUB;
        bool is_v;
        const uint32_t tile = item(s >> 1, is_v);
        const CUtensorMap *map = is_v ? vmap : kmap;
        const uint32_t key0 = k_begin + tile * FT_TILE;
        const int y0 = (int)(EXT ? cache_row(it, key0) : key0 - it.row0), y1 = EXT ? (int)cache_row(it, key0 + 32u) : y0 + 32;
        const int x = (int)(kvh * 256u + (s & 1u) * 128u);
        mbar_expect_tx(bar, FT_SUB);
#pragma unroll
        for (int d = 0; d < 4; d++) {
            tma_load_2d(dst + (2 * d) * FT_BOX, map, x + 32 * d, y0, bar);
            tma_load_2d(dst + (2 * d + 1) * FT_BOX, map, x + 32 * d, y1, bar);
        }
    };
    auto sub_safe = [&](uint32_t s) { // does the sub-tile's tile lie wholly below safe_below?
        bool is_v;
        return k_begin + (item(s >> 1, is_v) + 1u) * FT_TILE <= it.safe_below;
    };
    uint32_t early = 0;
    if (tid == 0) {
        for (int i = 0; i < FT_NRAW; i++) {
            mbar_init(bar_raw_full + 8u * i, 1);
            mbar_init(bar_raw_empty + 8u * i, 64);
        }
        for (int i = 0; i < FT_NOP; i++) {
            mbar_init(bar_op_full + 8u * i, 64);
            mbar_init(bar_op_empty + 8u * i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(bar_s_full + 8u * i, 1);
            mbar_init(bar_p_full + 8u * i, 128);
        }
        for (int i = 0; i < 3; i++) {
            mbar_init(bar_o_full + 8u * i, 1);
            mbar_init(bar_o_free + 8u * i, 128);
        }
        sh->abort = 0;
        fence_barrier_init();
        fence_proxy_async();
        // sub-tiles of tiles wholly below safe_below may load before the kernel in front has finished
        const uint32_t pre = min(nsub, (uint32_t)FT_NRAW);
        for (; early < pre && sub_safe(early); early++) issue(early);
    }
    if (tid < 64u * it.ntok) prefetch_l2(it.q + (size_t)(tid >> 6) * 4096u + (size_t)kvh * 2048u + (size_t)(tid & 63u) * 32u);
    if (warp == 1) tmem_alloc(smem_base + FT_OFF_MISC, FT_COLS);
    pdl_wait();

    // Q of this KV head as hi and lo f16, the B operands of S^T: per 64-dim block [32 rows][128 bytes], swizzled
    {
        uint8_t *qh = smem + FT_OFF_Q, *ql = qh + 16384;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t idx = tid + 256u * i; // 32 rows x 32 chunks of 8 dims
            const uint32_t row = idx >> 5, chunk = idx & 31u, tok = row >> 3;
            uint4 hi = make_uint4(0, 0, 0, 0), lo = hi;
            if (tok < it.ntok) {
                const float *src = it.q + (size_t)tok * 4096u + (size_t)(8u * kvh + (row & 7u)) * 256u + chunk * 8u;
                ft_split8(*reinterpret_cast<const float4 *>(src), *reinterpret_cast<const float4 *>(src + 4), hi, lo);
            }
            const uint32_t off = (chunk >> 3) * FT_QB + swz128(row, chunk & 7u);
            *reinterpret_cast<uint4 *>(qh + off) = hi;
            *reinterpret_cast<uint4 *>(ql + off) = lo;
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    // Conversion of raw sub-tile s into operand buffer s % NOP by the 64 threads of warps 2 and 3 (p = key of the tile):
    // per 8 dims two raw 16-byte chunks of dim box c / 4 -> one f16 chunk of block c / 8, hi and lo. Consecutive threads
    // take consecutive keys, which keeps both the swizzled loads and stores free of bank conflicts. (Letting the softmax
    // warps convert a share as well was measured: conversion alone got faster, the whole kernel slower.)
    auto convert = [&](uint32_t s, uint32_t p) -> bool {
        const uint32_t slot = s % FT_NRAW, ob = s % FT_NOP;
        if (!ft_wait(bar_raw_full + 8u * slot, (s / FT_NRAW) & 1u, sh, status)) return false;
        if (s >= (uint32_t)FT_NOP && !ft_wait(bar_op_empty + 8u * ob, ((s / FT_NOP) - 1u) & 1u, sh, status)) return false;
        const uint8_t *raw = smem + slot * FT_SUB;
        uint8_t *oph = smem + FT_OFF_OP + ob * FT_SUB, *opl = oph + 16384;
        if (ph != 6u) { // (measurement 6: no conversion)
#pragma unroll 8
            for (uint32_t k = 0; k < 16u; k++) {
                const uint32_t i = p + 64u * k;
                {
                    const uint32_t key = i & 63u, c = i >> 6, kb = key >> 5, kr = key & 31u;
                    const uint8_t *box = raw + (2u * (c >> 2) + kb) * FT_BOX;
                    const float4 a = *reinterpret_cast<const float4 *>(box + swz128(kr, 2u * (c & 3u)));
                    const float4 b = *reinterpret_cast<const float4 *>(box + swz128(kr, 2u * (c & 3u) + 1u));
                    uint4 hi, lo;
                    ft_split8(a, b, hi, lo);
                    const uint32_t off = (c >> 3) * FT_HBLK + swz128(key, c & 7u);
                    *reinterpret_cast<uint4 *>(oph + off) = hi;
                    *reinterpret_cast<uint4 *>(opl + off) = lo;
                }
            }
        }
        fence_proxy_async(); // the tensor core reads the operands through the async proxy
        mbar_arrive(bar_op_full + 8u * ob);
        mbar_arrive(bar_raw_empty + 8u * slot);
        return true;
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (uint32_t s = early; s < nsub; s++) {
                const uint32_t slot = s % FT_NRAW;
                if (s >= (uint32_t)FT_NRAW && !ft_wait(bar_raw_empty + 8u * slot, ((s / FT_NRAW) - 1u) & 1u, sh, status)) break;
                issue(s);
            }
        }
    } else if (warp == 2 || warp == 3) {
        // ---------------- converters ----------------
        for (uint32_t s2 = 0; s2 < nsub; s2++)
            if (!convert(s2, tid - 64u)) break;
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t IDESC_QK = tc_idesc_f16(64, 32, false, false);
            constexpr uint32_t IDESC_PV = tc_idesc_f16(128, 32, false, true);
            const uint32_t qh = smem_base + FT_OFF_Q, ql = qh + 16384u;
            bool ok = true;
            for (uint32_t s = 0; ok && s < nsub; s++) {
                bool is_v;
                const uint32_t j = item(s >> 1, is_v), ob = s % FT_NOP, half = s & 1u, part = (is_v ? 2u : 0u) + half;
                const uint32_t oph = smem_base + FT_OFF_OP + ob * FT_SUB, opl = oph + 16384u;
                if (!(ok = ft_wait(bar_op_full + 8u * ob, (s / FT_NOP) & 1u, sh, status))) break;
                if (part == 0u && j >= 2u && !(ok = ft_wait(bar_p_full + 8u * (j & 1u), ((j >> 1) - 1u) & 1u, sh, status))) break; // S^T buffer free
                if (part == 2u) {
                    if (!(ok = ft_wait(bar_p_full + 8u * (j & 1u), (j >> 1) & 1u, sh, status))) break;                         // P^T written
                    if (j >= 3u && !(ok = ft_wait(bar_o_free + 8u * (j % 3u), ((j / 3u) - 1u) & 1u, sh, status))) break;       // O_t buffer folded
                }
                tc_fence_after();
                if (part < 2u) { // S^T (+)= K_half . Q_half^T : main = hi.hi, small = hi.lo + lo.hi
                    const uint32_t d_main = tmem + FT_COL_S + 64u * (j & 1u), d_small = d_main + 32u;
#pragma unroll
                    for (uint32_t ks = 0; ks < 8u; ks++) { // 16 dims per MMA
                        const uint32_t ao = (ks >> 2) * FT_HBLK + (ks & 3u) * 32u, bo = (2u * half + (ks >> 2)) * FT_QB + (ks & 3u) * 32u;
                        const uint64_t ah = tc_desc_sw128(oph + ao, 16, 1024), al = tc_desc_sw128(opl + ao, 16, 1024);
                        const uint64_t bh = tc_desc_sw128(qh + bo, 16, 1024), bl = tc_desc_sw128(ql + bo, 16, 1024);
                        if (ph != 5u) {
                            tc_mma_f16(d_main, ah, bh, IDESC_QK, (half | ks) ? 1u : 0u);
                            tc_mma_f16(d_small, ah, bl, IDESC_QK, (half | ks) ? 1u : 0u);
                            tc_mma_f16(d_small, al, bh, IDESC_QK, 1u);
                        }
                    }
                    tc_commit(bar_op_empty + 8u * ob);
                    if (half) tc_commit(bar_s_full + 8u * (j & 1u));
                } else { // O_t^T half = V_half^T . P^T, from zero: main = hi.hi, small = hi.lo + lo.hi
                    const uint32_t pb = smem_base + FT_OFF_P + (j & 1u) * FT_PBUF, pl = pb + 4096u;
                    const uint32_t d_main = tmem + FT_COL_O + 128u * (j % 3u) + 32u * half, d_small = d_main + 64u;
#pragma unroll
                    for (uint32_t ks = 0; ks < 4u; ks++) { // 16 keys per MMA
                        // V^T, M-major: the next 64 dims one block on, the next 8 keys 1024 bytes on
                        const uint64_t ah = tc_desc_sw128(oph + ks * 2048u, FT_HBLK, 1024), al = tc_desc_sw128(opl + ks * 2048u, FT_HBLK, 1024);
                        const uint64_t bh = tc_desc_sw128(pb + ks * 32u, 16, 1024), bl = tc_desc_sw128(pl + ks * 32u, 16, 1024);
                        if (ph != 5u) {
                            tc_mma_f16(d_main, ah, bh, IDESC_PV, ks ? 1u : 0u);
                            tc_mma_f16(d_small, ah, bl, IDESC_PV, ks ? 1u : 0u);
                            tc_mma_f16(d_small, al, bh, IDESC_PV, 1u);
                        }
                    }
                    tc_commit(bar_op_empty + 8u * ob);
                    if (half) tc_commit(bar_o_full + 8u * (j % 3u));
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax (lanes 0..15 of each warp: one key each) and the owners of O (all lanes: one dim) ----------------
        const uint32_t q4 = warp & 3u, dlane = 32u * q4 + lane;     // TMEM lane; for O^T the head dim inside its half
        const uint32_t lane_addr = (32u * q4) << 16;
        const bool has_key = lane < 16u;
        const uint32_t kslot = 16u * q4 + (lane & 15u);             // key of the tile held by this lane (M = 64 layout)
        const uint32_t klo = max(it.first_pos, it.key_lo);
        uint32_t lim[4];
#pragma unroll
        for (uint32_t t = 0; t < 4u; t++) lim[t] = min(min(it.pos + 1u + t, it.key_hi), k_end);
        const uint32_t lo_max = EXT ? lowest_key(it, 3u) : klo;
        float negm[32], lpart[32], o[2][32];
#pragma unroll
        for (int r = 0; r < 32; r++) {
            negm[r] = FT_UNSET;
            lpart[r] = 0.0f;
            o[0][r] = o[1][r] = 0.0f;
        }
        float *red_base = reinterpret_cast<float *>(smem + FT_OFF_RED);
        uint32_t red_turn = 0;
        // P^T[row][key]: this key's column, 2 bytes in each of the 32 rows, hi at +0 and lo at +4096
        uint8_t *pcol = smem + FT_OFF_P + (kslot & 7u) * 2u;
        const uint32_t kchunk = kslot >> 3;
        bool stopped = false;
        uint32_t folded = 0; // tiles whose O_t has been folded into o

        // O = O * 1 + O_t of tile jj (main and small accumulators of both halves), then the buffer is free
        auto fold = [&](uint32_t jj) -> bool {
            bool ok = __all_sync(0xffffffffu, ft_wait(bar_o_full + 8u * (jj % 3u), (jj / 3u) & 1u, sh, status));
            tc_fence_after();
            const uint32_t ob = tmem + lane_addr + FT_COL_O + 128u * (jj % 3u);
#pragma unroll
            for (uint32_t mh = 0; mh < 2u; mh++) {
                uint32_t a[32], b[32];
                tmem_ld32(ob + 32u * mh, a);
                tmem_ld32(ob + 64u + 32u * mh, b);
                tmem_wait_ld();
#pragma unroll
                for (int r = 0; r < 32; r++) o[mh][r] = __fadd_rn(o[mh][r], __fadd_rn(__uint_as_float(a[r]), __uint_as_float(b[r])));
            }
            tc_fence_before();
            mbar_arrive(bar_o_free + 8u * (jj % 3u));
            return ok;
        };

        // the softmax of tile j; false = a wait ran out and all 128 threads stop
        auto softmax_tile = [&](uint32_t j) -> bool {
            bool ok = __all_sync(0xffffffffu, ft_wait(bar_s_full + 8u * (j & 1u), (j >> 1) & 1u, sh, status));
            tc_fence_after();
            float t[32];
            {
                uint32_t sa[32], sb[32];
                tmem_ld32(tmem + lane_addr + FT_COL_S + 64u * (j & 1u), sa);
                tmem_ld32(tmem + lane_addr + FT_COL_S + 64u * (j & 1u) + 32u, sb);
                tmem_wait_ld();
                const uint32_t tile_lo = k_begin + j * FT_TILE, key = tile_lo + kslot;
                const bool masked = tile_lo < lo_max || tile_lo + FT_TILE > lim[0];
#pragma unroll
                for (int r = 0; r < 32; r++) {
                    const float sc = __fadd_rn(__uint_as_float(sa[r]), __uint_as_float(sb[r])) * FT_C2;
                    bool seen = has_key;
                    if (masked) seen = seen && key >= (EXT ? lowest_key(it, (uint32_t)r >> 3) : klo) && key < lim[r >> 3];
                    t[r] = seen ? sc : NEG_BIG; // scale, then mask (W/ops.wgsl:361)
                }
            }
            bool over = false;
#pragma unroll
            for (int r = 0; r < 32; r++) over |= t[r] + negm[r] > FT_LAZY2;
            // P^T buffer j & 1 belongs to the MMAs of tile j-2 until those have completed (its O_t is then full)
            if (j >= 2u) ok = __all_sync(0xffffffffu, ft_wait(bar_o_full + 8u * ((j - 2u) % 3u), ((j - 2u) / 3u) & 1u, sh, status)) && ok;
            if (ft_bar_or(over || !ok)) {
                if (ft_bar_or(!ok)) {
                    stopped = true;
                    return false;
                }
                float *red = red_base + 128u * (red_turn & 1u);
                {
                    float mx[32];
#pragma unroll
                    for (int r = 0; r < 32; r++) mx[r] = t[r];
                    red[q4 * 32u + lane] = ft_transpose_reduce<true>(mx, lane);
                }
                ft_bar_sync();
                float my_negm = FT_UNSET, my_cf = 1.0f;
#pragma unroll
                for (int r = 0; r < 32; r++)
                    if (lane == (uint32_t)r) my_negm = negm[r];
                {
                    const float mt = fmaxf(fmaxf(red[lane], red[32u + lane]), fmaxf(red[64u + lane], red[96u + lane]));
                    if (mt > NEG_TEST) {
                        const bool set = my_negm < 0.5f * FT_UNSET;
                        const float m_new = set ? fmaxf(-my_negm, mt) : mt;
                        if (set) my_cf = exp2f(-my_negm - m_new);
                        my_negm = -m_new;
                    }
                }
                bool any = false;
                float cf[32];
#pragma unroll
                for (int r = 0; r < 32; r++) {
                    cf[r] = __shfl_sync(0xffffffffu, my_cf, r);
                    negm[r] = __shfl_sync(0xffffffffu, my_negm, r);
                    lpart[r] *= cf[r];
                    any |= cf[r] != 1.0f;
                }
                red_turn++;
                if (any) {
                    // O must hold every tile whose weights used the old references before it is rescaled
                    while (ok && folded < j) ok = fold(folded++);
                    if (ft_bar_or(!ok)) {
                        stopped = true;
                        return false;
                    }
#pragma unroll
                    for (int r = 0; r < 32; r++) {
                        o[0][r] *= cf[r];
                        o[1][r] *= cf[r];
                    }
                }
            }
            // weights 2^(t - m) in f32, split into hi and lo halves for the product with V; the sums run over the f32 values
            if (has_key) {
#pragma unroll
                for (int r = 0; r < 32; r++) {
                    float w;
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(t[r] + negm[r]));
                    lpart[r] += w;
                    const __half h = __float2half_rn(w);
                    const __half l = __float2half_rn(w - __half2float(h));
                    uint8_t *pp = pcol + (j & 1u) * FT_PBUF + r * 128u + ((kchunk ^ (uint32_t)(r & 7)) << 4);
                    *reinterpret_cast<__half *>(pp) = h;
                    *reinterpret_cast<__half *>(pp + 4096u) = l;
                }
            }
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar_p_full + 8u * (j & 1u));
            // off the critical path: fold the tiles whose products are done (the third O_t buffer gives the slack)
            bool okf = true;
            while (okf && j >= 2u && folded + 2u <= j) okf = fold(folded++);
            return true;
        };

        for (uint32_t j = 0; j < nt; j++)
            if (!softmax_tile(j)) break;

        // ---------------- the piece's partial: [m, l] per row and O[32][256] ----------------
        if (!stopped) {
            bool ok = true;
            while (ok && folded < nt) ok = fold(folded++);
            const size_t piece = (size_t)kvh * it.nsplit + split;
            float mrow = FT_UNSET;
#pragma unroll
            for (int r = 0; r < 32; r++)
                if (lane == (uint32_t)r) mrow = negm[r];
            float *red = red_base + 128u * (red_turn & 1u);
            red[lane * 4u + q4] = ft_transpose_reduce<false>(lpart, lane);
            ft_bar_sync();
            if (q4 == 0) {
                const float4 x = *reinterpret_cast<const float4 *>(red + 4 * lane);
                const float m = mrow < 0.5f * FT_UNSET ? -mrow * 0.6931471805599453f : NEG_BIG;
                reinterpret_cast<float2 *>(it.part_ml)[piece * 32u + lane] = make_float2(m, (x.x + x.y) + (x.z + x.w));
            }
            float *po = it.part_o + piece * 32u * 256u;
#pragma unroll
            for (uint32_t mh = 0; mh < 2u; mh++)
#pragma unroll
                for (int r = 0; r < 32; r++) po[(size_t)r * 256u + 128u * mh + dlane] = ok ? o[mh][r] : 0.0f;
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (sh->abort && tid == 0) {
        for (int i = 0; i < FT_NRAW; i++) mbar_wait_bounded(bar_raw_full + 8u * i, 0, 200000000ll);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, FT_COLS);
    }
    finish_item<256, EXT>(it, *reinterpret_cast<FinishSmem *>(smem), status);
}

mkv_status verify_f32_tc_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FT_SMEM));
    return MKV_OK;
}

mkv_status launch_verify_f32_tc(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas,
                                bool ext) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(total_ctas);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = FT_SMEM;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (ext) MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_tc_kernel<true>, items_dev, n, single, ctx->dev_status));
    else MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_tc_kernel<false>, items_dev, n, single, ctx->dev_status));
    ctx->launches++;
    return MKV_OK;
}

} // namespace mkv
