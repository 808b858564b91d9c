// Decode / verify attention over the f16 cache on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), K/V tiles staged by TMA. Same contract as verify_f16_kernel: split-K flash-decode for up to
// 4 tokens x 8 query heads (32 rows) per KV head, pieces merged by the CTAs that finish last (combine.cuh).
//
// Stands in for q_dmx + attn_dmx2 + attn_fd_combine of the reference (M/dmx.rs:19-141, W/ops.wgsl:523-538).
//
// A tcgen05 MMA needs M >= 64 rows in its accumulator and a step has only 32, so both products are taken
// transposed and the KEYS (or the head dims) fill the 128 TMEM lanes:
//   S^T[128 keys][32 rows]  = K_tile[128 keys][256 dims] . Q^T        A = K tile as TMA left it (K-major),
//                                                                      B = Q as f16 in shared memory (K-major)
//   O^T[256 dims][32 rows] += V_tile^T[256 dims][128 keys] . P^T      A = V tile as TMA left it (M-major),
//                                                                      B = P^T as f16 in shared memory (K-major)
// Roles (256 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 4..7 = softmax, one
// thread per key of the tile holding that key's 32 scores. Because a row's keys are spread over 128 threads,
// the running maximum is the reference's lazy maximum (M/dmx.rs:80, threshold 8): one vote per tile tells
// whether any score exceeds its row's reference by more than 8; only then (the first tile, and rarely after)
// the threads reduce the tile maxima, move the references and rescale O^T. Row sums are kept per thread and
// reduced once at the end. The tensor pipe and the softmax warps both need a fraction of a tile's load time,
// so the kernel runs at the speed of its TMA stream. Every wait is bounded; TMEM is freed on every path.
#include <stdlib.h>

#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

// The ring holds whole K or V tiles in the order K0 K1 V0 K2 V1 K3 V2 ...: K runs one tile ahead of V, so the
// scores and the softmax of tile j+1 are done while V of tile j is still on its way, and every slot goes back
// to the producer as soon as the one product that reads it has been issued. That order, two P^T buffers and
// two S^T buffers keep the softmax out of the chain "slot freed -> next load lands -> product -> slot freed",
// which is what limits a CTA when its tiles come from L2 faster than DRAM could deliver them.
constexpr int VT_NSLOT = 3;
constexpr uint32_t VT_TILE = 128;                    // keys per tile = two boxes of the verify tensor maps
constexpr uint32_t VT_SLOT = 65536;                  // 4 dim blocks of [128 keys][64 dims] f16
constexpr uint32_t VT_DB = 16384;                    // one dim block
constexpr uint32_t VT_OFF_Q = VT_NSLOT * VT_SLOT;    // [4 dim blocks][32 rows][64 dims] f16
constexpr uint32_t VT_QB = 4096;
constexpr uint32_t VT_OFF_P = VT_OFF_Q + 16384;      // 2 buffers of [2 key blocks][32 rows][64 keys] f16
constexpr uint32_t VT_PBUF = 8192;
constexpr uint32_t VT_OFF_RED = VT_OFF_P + 2 * VT_PBUF;     // two buffers of [32 rows][4 warps] floats
constexpr uint32_t VT_OFF_BAR = VT_OFF_RED + 1024;
// barriers: full[NSLOT], empty[NSLOT], s_full[2], p_full[2], pv_done[2]
constexpr uint32_t VT_NBAR = 2 * VT_NSLOT + 6;
constexpr uint32_t VT_OFF_MISC = VT_OFF_BAR + VT_NBAR * 8;
constexpr uint32_t VT_MISC_BYTES = 512;               // VtShared (a few words; a timeline record in trace builds)
constexpr uint32_t VT_SMEM = VT_OFF_MISC + VT_MISC_BYTES + 1024;
constexpr uint32_t VT_COL_S = 0, VT_COL_O = 64, VT_COLS = 128; // S^T: 2 x 32 columns, O^T: 2 halves x 32
constexpr long long VT_WAIT_LIMIT = 2000000000ll;
constexpr float VT_LOG2E = 1.4426950408889634f;
constexpr float VT_C2 = SCALE * VT_LOG2E;            // scores to base-2 exponents
constexpr float VT_LAZY2 = 8.0f * VT_LOG2E;          // the reference's threshold of 8, in base-2 units
constexpr float VT_UNSET = 1.0e30f;                  // -(reference maximum) of a row that has seen no key yet

#ifdef MKV_TRACE
// Timeline of one CTA for performance work (builds with -DMKV_MEASURE only; read by mechta_b200/trace_timeline.py,
// which lists the same fields in the same order). All times are %globaltimer nanoseconds.
struct VtTrace {
    unsigned long long launch, cta, sm, nt, ticket;               // launch = the item's ticket base, unique per launch
    unsigned long long start, wait_done, q_ready, piece, exit_;   // CTA start, griddepcontrol.wait returned, Q converted,
                                                                  // piece written, after the merge
    unsigned long long fin_ticket, fin_seen, fin_merged;          // merge: ticket taken, all pieces seen, rows merged
    unsigned long long fin_loads, fin_max, fin_summed;            // merge of a row: loads issued, maximum known, pieces summed
    unsigned long long t0_scores, t0_scaled, t0_votes, t0_reduced, t0_moved, t0_weights; // softmax of the first tile
    unsigned long long st_issued[8], softmax_done[8], ot_issued[8]; // per tile (the first eight)
};
__device__ VtTrace g_vt_trace[65536];
__device__ unsigned int g_vt_trace_n;
__device__ __forceinline__ unsigned long long vt_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define VT_STAMP(cond, field) do { if (cond) sh->trace.field = vt_now(); } while (0)
#else
#define VT_STAMP(cond, field) do { } while (0)
#endif

struct VtShared {
    uint32_t tmem_base;
    volatile uint32_t abort;
    uint32_t ticket; // this CTA's arrival number within its item (publish_piece)
#ifdef MKV_TRACE
    VtTrace trace;
#endif
};
constexpr int VT_ROW_OUTSIDE = 1 << 30; // a row coordinate beyond any cache (at most 2^18 + 2^10 rows)
static_assert(sizeof(VtShared) <= VT_MISC_BYTES, "VtShared outgrew its place in shared memory");

__device__ __forceinline__ bool vt_wait(uint32_t bar, uint32_t parity, VtShared *sh, uint32_t *status) {
    if (sh->abort) return false;
    if (mbar_wait_bounded(bar, parity, VT_WAIT_LIMIT)) return true;
    sh->abort = 1;
    atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
    return false;
}
// named barrier 1: the 128 softmax threads
__device__ __forceinline__ void vt_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ bool vt_bar_or(bool x) {
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
// v[i] of lane L, i = 0..31 -> the reduction over the warp's lanes of v[L], left in v[0] of lane L
// (31 shuffles: every step halves the number of live values).
template <bool MAX>
__device__ __forceinline__ float vt_transpose_reduce(float (&v)[32], uint32_t lane) {
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

// EXT: ring rows, sliding window and sinks (mkv_attn_verify_window, ring caches); the plain path is instantiated
// without them, which keeps a division and some branches out of the producer's refill path.
template <bool EXT, typename Launch>
__global__ void __launch_bounds__(256, 1)
verify_f16_tc_kernel(const VerifyItem *__restrict__ items, int n_items, const __grid_constant__ Launch single,
                     uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const VerifyItem &it = pick_item(items, n_items, single, blockIdx.x);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t local = blockIdx.x - it.cta_begin;
    if (local >= 2u * it.nsplit) return;
    const uint32_t ph = MKV_PHASE_OF(it);
    if (ph == 2u) return; // measurement: launch cost alone
    pdl_launch_dependents();    // the next kernel in the stream may begin its own prologue
    const uint32_t kvh = local & 1u, split = local >> 1;
    const uint32_t t0 = it.tile_begin + split * it.tiles_per_split; // in 64-key units
    const uint32_t t1 = min(t0 + it.tiles_per_split, it.tile_end);
    const uint32_t k_begin = t0 * TILE, k_end = t1 * TILE;          // this CTA's keys
    const uint32_t nt = ph == 3u ? 0u : (k_end - k_begin + VT_TILE - 1u) / VT_TILE;
    const CUtensorMap *kmap = launch_map(items, it, single, false), *vmap = launch_map(items, it, single, true);
    const uint32_t bar0 = smem_base + VT_OFF_BAR;
    const uint32_t bar_full = bar0, bar_empty = bar0 + 8u * VT_NSLOT, bar_s_full = bar0 + 16u * VT_NSLOT;
    const uint32_t bar_p_full = bar_s_full + 16u, bar_pv_done = bar_p_full + 16u;
    VtShared *sh = reinterpret_cast<VtShared *>(smem + VT_OFF_MISC);

    // Item n of the stream K0 K1 V0 K2 V1 ... goes to ring position n % NSLOT: eight boxes of [64 keys][64 dims].
    // The last tile of a CTA may reach past k_end (rows of the next piece, or zero fill past the buffer); those
    // keys are masked.
    auto seq_k = [&](uint32_t j) { return j < 2u ? j : 2u * j - 1u; };
    auto seq_v = [&](uint32_t j) { return j + 1u == nt ? 2u * nt - 1u : 2u * j + 2u; };
    auto item = [&](uint32_t n, bool &is_v) -> uint32_t { // the tile of item n
        if (n == 0u) { is_v = false; return 0u; }
        if ((n & 1u) == 0u) { is_v = true; return (n - 2u) >> 1; }
        const uint32_t j = (n + 1u) >> 1;
        is_v = j >= nt;
        return is_v ? nt - 1u : j;
    };
    auto boxes = [&](uint32_t n, auto &&f) {
        bool is_v;
        const uint32_t tile = item(n, is_v);
        const CUtensorMap *map = is_v ? vmap : kmap;
        // the two 64-key boxes of the tile are placed on their own: in a ring cache the second may wrap to row 0
        const uint32_t key0 = k_begin + tile * VT_TILE;
        // A second half wholly past this CTA's keys (its piece is an odd number of 64-key units long) is not fetched: its box
        // starts at a row far outside the tensor, which TMA answers with the fill value, zero, without touching memory.
        // Those keys are masked, and zeros keep the masked weights' 0 x V finite.
        const int y0 = (int)(EXT ? cache_row(it, key0) : key0 - it.row0);
        const int y1 = key0 + 64u >= k_end ? VT_ROW_OUTSIDE : EXT ? (int)cache_row(it, key0 + 64u) : y0 + 64;
        const int x = (int)(kvh * 256u);
#pragma unroll
        for (int db = 0; db < 4; db++) {
            f(map, (uint32_t)db * VT_DB, x + 64 * db, y0);
            f(map, (uint32_t)db * VT_DB + 8192u, x + 64 * db, y1);
        }
    };
    auto issue = [&](uint32_t n) {
        const uint32_t s = n % VT_NSLOT, bar = bar_full + 8u * s, dst = smem_base + s * VT_SLOT;
        mbar_expect_tx(bar, VT_SLOT);
        boxes(n, [&](const CUtensorMap *map, uint32_t off, int x, int y) { tma_load_2d(dst + off, map, x, y, bar); });
    };
    auto item_safe = [&](uint32_t n) { // does item n lie wholly below safe_below?
        bool is_v;
        return k_begin + (item(n, is_v) + 1u) * VT_TILE <= it.safe_below;
    };
    // Tiles wholly below `safe_below` hold rows the kernel before this one in the stream did not write: thread 0
    // starts their loads before that kernel is known to have finished, and before the rest of this prologue.
    uint32_t early = 0;
    if (tid == 0) {
        VT_STAMP(true, start);
        for (int s = 0; s < VT_NSLOT; s++) {
            mbar_init(bar_full + 8u * s, 1);
            mbar_init(bar_empty + 8u * s, 1);
        }
        mbar_init(bar_s_full, 1);
        mbar_init(bar_s_full + 8u, 1);
        mbar_init(bar_p_full, 128);
        mbar_init(bar_p_full + 8u, 128);
        mbar_init(bar_pv_done, 1);
        mbar_init(bar_pv_done + 8u, 1);
        sh->abort = 0;
        fence_barrier_init();
        fence_proxy_async();
        const uint32_t pre = min(2u * nt, (uint32_t)VT_NSLOT);
        for (; early < pre && item_safe(early); early++) issue(early);
    }
    // Q of this KV head towards L2 while the kernel waits for its predecessor: 8 KB per token, one 128-byte line
    // per thread. (Prefetching K/V tiles beyond the ring into L2 in the same way was measured: it takes DRAM
    // bandwidth from the tail of the kernel in front, which is the critical path, and loses more than it gains.)
    if (tid < 64u * it.ntok) {
        prefetch_l2(it.q + (size_t)(tid >> 6) * 4096u + (size_t)kvh * 2048u + (size_t)(tid & 63u) * 32u);
    }
    if (warp == 1) tmem_alloc(smem_base + VT_OFF_MISC, VT_COLS); // writes sh->tmem_base
    pdl_wait(); // Q, the newest rows and every global write come after this
    VT_STAMP(tid == 0, wait_done);

    // Q of this KV head to shared memory as f16, the B operand of S^T: row = tok * 8 + head % 8 (the order of
    // q_dmx, M/dmx.rs:128-138), rows of tokens >= ntok zero; per 64-dim block [32 rows][128 bytes], 128-byte swizzle
    {
        uint8_t *qs = smem + VT_OFF_Q;
        // All eight loads of a thread go out before the first conversion: written as one loop they would alternate
        // with the shared-memory stores (the compiler cannot tell the two apart through generic pointers) and the
        // four round trips to L2 would run one after the other, on the critical path of every launch.
        float4 qa[4], qb[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t idx = tid + 256u * i; // 32 rows x 32 chunks of 8 dims
            const uint32_t row = idx >> 5, chunk = idx & 31u, tok = row >> 3;
            qa[i] = qb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tok < it.ntok) {
                const float4 *src = reinterpret_cast<const float4 *>(it.q + (size_t)tok * 4096u + (size_t)(8u * kvh + (row & 7u)) * 256u +
                                                                     chunk * 8u);
                qa[i] = __ldcg(src);
                qb[i] = __ldcg(src + 1);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t idx = tid + 256u * i;
            const uint32_t row = idx >> 5, chunk = idx & 31u;
            const __half2 h0 = __floats2half2_rn(qa[i].x, qa[i].y), h1 = __floats2half2_rn(qa[i].z, qa[i].w);
            const __half2 h2 = __floats2half2_rn(qb[i].x, qb[i].y), h3 = __floats2half2_rn(qb[i].z, qb[i].w);
            const uint4 w = make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                                       *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
            *reinterpret_cast<uint4 *>(qs + (chunk >> 3) * VT_QB + swz128(row, chunk & 7u)) = w;
        }
    }
    fence_proxy_async(); // the tensor core reads Q through the async proxy
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;
    VT_STAMP(tid == 0, q_ready);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (uint32_t i = early; i < 2u * nt; i++) {
                const uint32_t s = i % VT_NSLOT;
                if (i >= (uint32_t)VT_NSLOT && !vt_wait(bar_empty + 8u * s, ((i / VT_NSLOT) - 1u) & 1u, sh, status)) break;
                issue(i);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0 && ph == 1u) { // measurement: stream the tiles only
            for (uint32_t i = 0; i < 2u * nt; i++) {
                if (!vt_wait(bar_full + 8u * (i % VT_NSLOT), (i / VT_NSLOT) & 1u, sh, status)) break;
                mbar_arrive(bar_empty + 8u * (i % VT_NSLOT));
            }
        } else if (lane == 0) {
            constexpr uint32_t IDESC_QK = tc_idesc_f16(128, 32, false, false);
            constexpr uint32_t IDESC_PV = tc_idesc_f16(128, 32, false, true);
            const uint32_t qb = smem_base + VT_OFF_Q, pb = smem_base + VT_OFF_P;
            const bool mma_qk = ph != 5u, mma_pv = ph != 5u; // measurement: 5 = everything but the MMAs
            // Event loop: whichever of "the next K tile has landed" (and its S^T buffer is free) and "the next V
            // tile has landed and its P^T is written" is true first is issued first, so that a tile's shared
            // memory goes back to the producer as early as possible: the bytes in flight, not the tensor pipe,
            // set the speed of this kernel.
            uint32_t jq = 0, jp = 0; // next tile of S^T = K Q^T, next tile of O^T += V^T P^T
            // A barrier may only be tested for the use that follows the last one this thread consumed: a parity
            // test two uses ahead is satisfied by the use before last. Item n is the next use of its slot once item
            // n - NSLOT has been consumed here.
            auto slot_ready = [&](uint32_t n) {
                if (n < (uint32_t)VT_NSLOT) return true;
                bool is_v;
                const uint32_t t = item(n - VT_NSLOT, is_v);
                return is_v ? jp > t : jq > t;
            };
            long long tlast = clock64();
            while (jp < nt) {
                bool did = false;
                if (jq < nt) {
                    const uint32_t n = seq_k(jq), s = n % VT_NSLOT;
                    // S^T buffer jq & 1 is free once the softmax of tile jq - 2 has published its P^T
                    const bool s_free = jq < 2u || mbar_test(bar_p_full + 8u * (jq & 1u), ((jq >> 1) - 1u) & 1u);
                    if (s_free && slot_ready(n) && mbar_test(bar_full + 8u * s, (n / VT_NSLOT) & 1u)) {
                        tc_fence_after();
                        const uint32_t kb = smem_base + s * VT_SLOT, d = tmem + VT_COL_S + 32u * (jq & 1u);
#pragma unroll
                        for (uint32_t ks = 0; ks < 16u; ks++) { // 16 dims per MMA; 4 per 64-dim block
                            const uint64_t a = tc_desc_sw128(kb + (ks >> 2) * VT_DB + (ks & 3u) * 32u, 16, 1024);
                            const uint64_t b = tc_desc_sw128(qb + (ks >> 2) * VT_QB + (ks & 3u) * 32u, 16, 1024);
                            if (mma_qk) tc_mma_f16(d, a, b, IDESC_QK, ks > 0 ? 1u : 0u);
                        }
                        tc_commit(bar_empty + 8u * s); // the K tile is free
                        tc_commit(bar_s_full + 8u * (jq & 1u));
                        VT_STAMP(jq < 8u, st_issued[jq]);
                        jq++;
                        did = true;
                    }
                }
                if (jp < jq) {
                    const uint32_t n = seq_v(jp), s = n % VT_NSLOT;
                    if (slot_ready(n) && mbar_test(bar_full + 8u * s, (n / VT_NSLOT) & 1u) &&
                        mbar_test(bar_p_full + 8u * (jp & 1u), (jp >> 1) & 1u)) {
                        tc_fence_after();
                        const uint32_t vb = smem_base + s * VT_SLOT, pbj = pb + (jp & 1u) * VT_PBUF;
#pragma unroll
                        for (uint32_t mh = 0; mh < 2u; mh++) // dims 128 mh .. 128 mh + 127 in the TMEM lanes
#pragma unroll
                            for (uint32_t ks = 0; ks < 8u; ks++) { // 16 keys per MMA
                                // V^T, M-major: the next 64 dims one dim block on, the next 8 keys 1024 bytes on
                                const uint64_t a = tc_desc_sw128(vb + 2u * mh * VT_DB + ks * 2048u, VT_DB, 1024);
                                const uint64_t b = tc_desc_sw128(pbj + (ks >> 2) * 4096u + (ks & 3u) * 32u, 16, 1024);
                                if (mma_pv) tc_mma_f16(tmem + VT_COL_O + 32u * mh, a, b, IDESC_PV, (jp | ks) ? 1u : 0u);
                            }
                        tc_commit(bar_empty + 8u * s);                 // the V tile is free
                        tc_commit(bar_pv_done + 8u * (jp & 1u));       // O^T holds tiles 0..jp; P^T buffer jp & 1 may be overwritten
                        VT_STAMP(jp < 8u, ot_issued[jp]);
                        jp++;
                        did = true;
                    }
                }
                if (did) {
                    tlast = clock64();
                } else if (sh->abort || clock64() - tlast > VT_WAIT_LIMIT) {
                    if (!sh->abort) {
                        sh->abort = 1;
                        atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
                    }
                    break;
                }
            }
        }
    } else if (warp >= 4) {
        // ---------------- softmax: one thread per key of the tile (TMEM lane), 32 rows each ----------------
        const uint32_t q4 = warp & 3u, klane = 32u * q4 + lane; // the TMEM lanes this warp may access
        const uint32_t lane_addr = (32u * q4) << 16;
        // token t of the step sees lowest_key(t) <= key < min(pos + 1 + t, end of the shard, end of this piece)
        // (M/dmx.rs:71); tiles between the highest lower bound and the lowest upper bound need no mask
        const uint32_t klo = max(it.first_pos, it.key_lo);
        uint32_t lim[4]; // upper bounds per token, cut to the shard and to this piece
#pragma unroll
        for (uint32_t t = 0; t < 4u; t++) lim[t] = min(min(it.pos + 1u + t, it.key_hi), k_end);
        const uint32_t lo_max = EXT ? lowest_key(it, 3u) : klo;
        float negm[32], lpart[32]; // minus the row's reference maximum (base-2 units); this key slot's share of the row sums
#pragma unroll
        for (int r = 0; r < 32; r++) {
            negm[r] = VT_UNSET;
            lpart[r] = 0.0f;
        }
        // two scratch buffers used in turn, so that a reduction's readers never race the next reduction's writers
        // (between two uses of one buffer lies the barrier of the use of the other)
        float *red_base = reinterpret_cast<float *>(smem + VT_OFF_RED);
        uint32_t red_turn = 0;
        // P^T[row][key]: this thread's column, 2 bytes in each of the 32 rows (K-major B operand, 128-byte swizzle)
        uint8_t *pcol = smem + VT_OFF_P + (klane >> 6) * 4096u + (klane & 7u) * 2u;
        const uint32_t kchunk = (klane & 63u) >> 3;
        const uint32_t nts = ph == 1u ? 0u : nt;
        bool stopped = false;
        for (uint32_t j = 0; j < nts; j++) {
            // a warp takes every wait's outcome together: the TMEM loads are warp-collective
            bool ok = __all_sync(0xffffffffu, vt_wait(bar_s_full + 8u * (j & 1u), (j >> 1) & 1u, sh, status));
            tc_fence_after();
            VT_STAMP(tid == 128 && j == 0, t0_scores);
            if (ph == 4u) { // measurement: the MMAs without the softmax math, P^T left as it is
                if (j > 1) __all_sync(0xffffffffu, vt_wait(bar_pv_done + 8u * (j & 1u), ((j >> 1) - 1u) & 1u, sh, status));
                tc_fence_before();
                mbar_arrive(bar_p_full + 8u * (j & 1u));
                continue;
            }
            float t[32];
            {
                uint32_t sr[32];
                tmem_ld32(tmem + lane_addr + VT_COL_S + 32u * (j & 1u), sr);
                tmem_wait_ld();
                const uint32_t tile_lo = k_begin + j * VT_TILE, key = tile_lo + klane;
                if (tile_lo < lo_max || tile_lo + VT_TILE > lim[0]) { // scale, then mask (M/dmx.rs:71)
                    if constexpr (EXT) { // the lower bound depends on the token: the window moves with it
#pragma unroll
                        for (uint32_t tk = 0; tk < 4u; tk++) {
                            const bool seen = key >= lowest_key(it, tk) && key < lim[tk];
#pragma unroll
                            for (int r = 8 * (int)tk; r < 8 * (int)tk + 8; r++)
                                t[r] = seen ? __uint_as_float(sr[r]) * VT_C2 : NEG_BIG;
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < 32; r++)
                            t[r] = (key >= klo && key < lim[r >> 3]) ? __uint_as_float(sr[r]) * VT_C2 : NEG_BIG;
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < 32; r++) t[r] = __uint_as_float(sr[r]) * VT_C2;
                }
            }
            bool over = false;
#pragma unroll
            for (int r = 0; r < 32; r++) over |= t[r] + negm[r] > VT_LAZY2;
            VT_STAMP(tid == 128 && j == 0, t0_scaled);
            // P^T buffer j & 1 belongs to the MMAs of tile j-2 until those have completed
            if (j > 1) ok = __all_sync(0xffffffffu, vt_wait(bar_pv_done + 8u * (j & 1u), ((j >> 1) - 1u) & 1u, sh, status)) && ok;
            tc_fence_after();
            if (vt_bar_or(over || !ok)) {
                if (vt_bar_or(!ok)) { // a wait ran out somewhere: all 128 threads leave together
                    stopped = true;
                    break;
                }
                VT_STAMP(tid == 128 && j == 0, t0_votes);
                // move the reference maxima to the true maxima so far. The warp's transposing reduction leaves the
                // maximum of row L over the warp's 32 keys in lane L; after the four warps have met, lane L works
                // out row L's new reference and rescale factor once and the warp passes them round by shuffles
                // (every thread keeps all 32: its scores span all rows).
                float *red = red_base + 128u * (red_turn & 1u);
                {
                    float mx[32];
#pragma unroll
                    for (int r = 0; r < 32; r++) mx[r] = t[r];
                    red[q4 * 32u + lane] = vt_transpose_reduce<true>(mx, lane);
                }
                vt_bar_sync();
                VT_STAMP(tid == 128 && j == 0, t0_reduced);
                float my_negm = VT_UNSET, my_cf = 1.0f;
#pragma unroll
                for (int r = 0; r < 32; r++)
                    if (lane == (uint32_t)r) my_negm = negm[r];
                {
                    const float mt = fmaxf(fmaxf(red[lane], red[32u + lane]), fmaxf(red[64u + lane], red[96u + lane]));
                    if (mt > NEG_TEST) {
                        const bool set = my_negm < 0.5f * VT_UNSET;
                        const float m_new = set ? fmaxf(-my_negm, mt) : mt;
                        if (set) my_cf = exp2f(-my_negm - m_new);
                        my_negm = -m_new;
                    }
                }
                float cf[32];
                bool any = false;
#pragma unroll
                for (int r = 0; r < 32; r++) {
                    cf[r] = __shfl_sync(0xffffffffu, my_cf, r);
                    negm[r] = __shfl_sync(0xffffffffu, my_negm, r);
                    lpart[r] *= cf[r];
                    any |= cf[r] != 1.0f;
                }
                red_turn++;
                VT_STAMP(tid == 128 && j == 0, t0_moved);
                if (j > 0 && any) {
                    // O^T must hold every tile whose weights used the old references before it is rescaled: the
                    // product of tile j-1 may still be waiting for its V tile
                    ok = __all_sync(0xffffffffu, vt_wait(bar_pv_done + 8u * ((j - 1u) & 1u), ((j - 1u) >> 1) & 1u, sh, status));
                    tc_fence_after();
                    if (vt_bar_or(!ok)) {
                        stopped = true;
                        break;
                    }
                }
                if (j > 0 && any) { // rescale this lane's two halves of O^T (a column per row)
#pragma unroll
                    for (uint32_t mh = 0; mh < 2u; mh++) {
                        uint32_t oc[32];
                        tmem_ld32(tmem + lane_addr + VT_COL_O + 32u * mh, oc);
                        tmem_wait_ld();
#pragma unroll
                        for (int r = 0; r < 32; r++) oc[r] = __float_as_uint(__uint_as_float(oc[r]) * cf[r]);
                        tmem_st32(tmem + lane_addr + VT_COL_O + 32u * mh, oc);
                    }
                    tmem_wait_st();
                }
            }
            VT_STAMP(tid == 128 && j == 0, t0_weights);
            // weights: 2^(t - m), rounded to f16 as the reference does (M/dmx.rs:99); the sums run over the rounded values
#pragma unroll
            for (int r = 0; r < 32; r++) {
                float w;
                asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(w) : "f"(t[r] + negm[r]));
                const __half h = __float2half_rn(w);
                lpart[r] += __half2float(h);
                *reinterpret_cast<__half *>(pcol + (j & 1u) * VT_PBUF + r * 128u + ((kchunk ^ (uint32_t)(r & 7)) << 4)) = h;
            }
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(bar_p_full + 8u * (j & 1u));
            VT_STAMP(tid == 128 && j < 8u, softmax_done[j]);
        }

        // ---------------- the piece's partial: [m, l] per row and O[32][256] ----------------
        if (!stopped) {
            bool ok = true;
            if (nts > 0) ok = __all_sync(0xffffffffu, vt_wait(bar_pv_done + 8u * ((nts - 1u) & 1u), ((nts - 1u) >> 1) & 1u, sh, status));
            tc_fence_after();
            const size_t piece = (size_t)kvh * it.nsplit + split;
            float mrow = VT_UNSET; // -(reference maximum) of row `lane`
#pragma unroll
            for (int r = 0; r < 32; r++)
                if (lane == (uint32_t)r) mrow = negm[r];
            float *red = red_base + 128u * (red_turn & 1u);
            red[lane * 4u + q4] = vt_transpose_reduce<false>(lpart, lane);
            vt_bar_sync();
            if (q4 == 0) {
                const float4 x = *reinterpret_cast<const float4 *>(red + 4 * lane);
                const float m = mrow < 0.5f * VT_UNSET ? -mrow * 0.6931471805599453f : NEG_BIG; // back to natural units
                reinterpret_cast<float2 *>(it.part_ml)[piece * 32u + lane] = make_float2(m, (x.x + x.y) + (x.z + x.w));
            }
            float *po = it.part_o + piece * 32u * 256u;
#pragma unroll
            for (uint32_t mh = 0; mh < 2u; mh++) {
                uint32_t oc[32];
                if (nts > 0 && ok) {
                    tmem_ld32(tmem + lane_addr + VT_COL_O + 32u * mh, oc);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int r = 0; r < 32; r++) oc[r] = 0u;
                }
#pragma unroll
#ifndef VT_X_NOSTORE
                for (int r = 0; r < 32; r++) po[(size_t)r * 256u + 128u * mh + klane] = __uint_as_float(oc[r]);
#else
                if (oc[0] == 0x12345678u && oc[31] == 0x9abcdef0u) po[klane] = 1.0f; // timing only: keeps the loads alive
#endif
            }
        }
        // The piece is published by the threads that wrote it, before the CTA's teardown: what follows the last piece
        // of a launch is the critical path of the next one. (After a wait that ran out the piece is not valid; it is
        // published all the same so that nobody waits for it, and the status word says what happened.)
        vt_bar_sync();
        if (tid == 128u) sh->ticket = publish_piece(it);
    }

    // ---------------- teardown: nothing of this CTA may still be in flight, then free the tensor memory ----------------
    tc_fence_before();
    __syncthreads();
    if (sh->abort && tid == 0) {
        // a wait ran out somewhere: give copies already issued into this CTA's shared memory a bounded time to land
        for (int s = 0; s < VT_NSLOT; s++) mbar_wait_bounded(bar_full + 8u * s, 0, 200000000ll);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, VT_COLS);
    }
#ifdef MKV_TRACE
    // the record leaves shared memory before the merge reuses it
    VtTrace rec;
    if (tid == 0) {
        rec = sh->trace;
        rec.piece = vt_now();
    }
    __syncthreads();
#endif
    // this CTA's share of the merge, if its ticket gives it one (scratch in the ring, which is drained by now)
#ifndef VT_X_NOMERGE
    finish_item<256, EXT>(it, *reinterpret_cast<FinishSmem *>(smem), status, sh->ticket);
#endif
#ifdef MKV_TRACE
    if (tid == 0) {
        const unsigned int n = atomicAdd(&g_vt_trace_n, 1u);
        if (n < 65536u) {
            const FinishSmem &fs = *reinterpret_cast<const FinishSmem *>(smem);
            unsigned int smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            rec.launch = it.ticket_base; rec.cta = blockIdx.x; rec.sm = smid; rec.nt = nt; rec.ticket = sh->ticket;
            rec.fin_ticket = fs.tr[0]; rec.fin_seen = fs.tr[1]; rec.fin_merged = fs.tr[2];
            rec.fin_loads = fs.tm[0]; rec.fin_max = fs.tm[1]; rec.fin_summed = fs.tm[2];
            rec.exit_ = vt_now();
            g_vt_trace[n] = rec;
        }
    }
#endif
}

#ifdef MKV_TRACE
// Copies the records written so far to `dst` (room for max_records) and starts over. Measurement builds only.
extern "C" int mkv_trace_read(void *dst, int max_records) {
    unsigned int n = 0;
    cudaMemcpyFromSymbol(&n, g_vt_trace_n, sizeof n);
    if ((int)n > max_records) n = (unsigned int)max_records;
    if (n > 65536u) n = 65536u;
    cudaMemcpyFromSymbol(dst, g_vt_trace, (size_t)n * sizeof(VtTrace));
    const unsigned int zero = 0;
    cudaMemcpyToSymbol(g_vt_trace_n, &zero, sizeof zero);
    return (int)n;
}
#endif

mkv_status verify_tc_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_tc_kernel<false, VerifyLaunch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)VT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_tc_kernel<true, VerifyLaunch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)VT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_tc_kernel<false, VerifyLaunchBatch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)VT_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_tc_kernel<true, VerifyLaunchBatch>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)VT_SMEM));
    return MKV_OK;
}

template <typename Launch>
static mkv_status launch_verify_f16_tc_any(Ctx *ctx, const VerifyItem *items_dev, int n, const Launch &single, uint32_t total_ctas, bool ext) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(total_ctas);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = VT_SMEM;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (ext) MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f16_tc_kernel<true, Launch>, items_dev, n, single, ctx->dev_status));
    else MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f16_tc_kernel<false, Launch>, items_dev, n, single, ctx->dev_status));
    ctx->launches++;
    return MKV_OK;
}

mkv_status launch_verify_f16_tc(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas, bool ext) {
    return launch_verify_f16_tc_any(ctx, items_dev, n, single, total_ctas, ext);
}

// a few items in the parameter space (see VerifyLaunchBatch)
mkv_status launch_verify_f16_tc_few(Ctx *ctx, const VerifyLaunchBatch &few, int n, uint32_t total_ctas, bool ext) {
    return launch_verify_f16_tc_any(ctx, static_cast<const VerifyItem *>(nullptr), n, few, total_ctas, ext);
}

} // namespace mkv
