// Decode / verify attention over the f16 cache: split-K flash-decode for up to 4 tokens x 8 query heads
// (32 rows) per KV head, then a log-sum-exp combine of the pieces.
//
// Stands in for q_dmx + attn_dmx2 + attn_fd_combine of the reference (M/dmx.rs:19-141, W/ops.wgsl:523-538):
// same visibility rule (token t at pos + t sees first_pos <= key < pos + 1 + t), same mask value, same
// un-normalised partial [m, l, O] per piece, one divide at the end. What differs is the machine mapping:
//  - a CTA owns one KV head and a contiguous run of 64-key tiles; K and V tiles arrive by TMA
//    (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a 3-deep ring of 64 KB stages, each filled
//    tile signalled on an mbarrier;
//  - S = Q K^T: warp w takes keys 8w..8w+7 of the tile for all 32 rows (mma.m16n8k16, Q fragments live in
//    registers as f16), so every K byte is read from shared memory once;
//  - softmax: 8 threads per row, max and sum by warp shuffles, P rounded to f16 (as the reference does) and
//    the row sum taken over the rounded values;
//  - O += P V: warp w owns dims 32w..32w+31 for all rows, so every V byte is read from shared memory once;
//  - the CTAs that finish last merge the pieces (combine.cuh), so one launch gives the final output.
// A variant with two groups of 8 warps taking alternate 32-key tiles was measured slower (76 K against 57 K SM
// cycles at 65,536 tokens): more barriers per byte and no gain in overlap, since the loop is not compute-bound.
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int V16_NST = 3;                       // ring depth
constexpr uint32_t V16_STAGE = 65536;            // K 32 KB + V 32 KB
constexpr uint32_t V16_SUB = 8192;               // one [64 keys][64 dims] f16 sub-box
constexpr uint32_t V16_OFF_Q = V16_NST * V16_STAGE;
constexpr uint32_t V16_OFF_S = V16_OFF_Q + 32 * 512;
constexpr uint32_t V16_S_STRIDE = 68;            // floats per S row (64 + 4 of padding)
constexpr uint32_t V16_OFF_P = V16_OFF_S + 32 * V16_S_STRIDE * 4;
constexpr uint32_t V16_OFF_CF = V16_OFF_P + 32 * 128;
constexpr uint32_t V16_OFF_BAR = V16_OFF_CF + 32 * 4;
constexpr uint32_t V16_SMEM = V16_OFF_BAR + V16_NST * 8 + 1024; // + alignment slack
constexpr long long WAIT_LIMIT = 4000000000ll;   // about two seconds of SM clocks

__global__ void __launch_bounds__(256, 1)
verify_f16_kernel(const VerifyItem *__restrict__ items, int n_items, const __grid_constant__ VerifyLaunch single,
                  uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const VerifyItem &it = pick_item(items, n_items, single.item, blockIdx.x);
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t local = blockIdx.x - it.cta_begin;
    if (local >= 2u * it.nsplit) return;
    if (MKV_PHASE_OF(it) == 2u) return; // measurement: launch cost alone
    pdl_launch_dependents();    // the next kernel in the stream may begin its own prologue
    const uint32_t kvh = local & 1u, split = local >> 1;
    const uint32_t t0 = it.tile_begin + split * it.tiles_per_split;
    const uint32_t t1 = min(t0 + it.tiles_per_split, it.tile_end);
    const uint32_t nt = MKV_PHASE_OF(it) == 3u ? 0u : t1 - t0; // measurement: prologue and epilogue without tiles
    // a single launch carries its tensor maps in the parameter space
    const CUtensorMap *kmap = items ? it.kmap : &single.kmap, *vmap = items ? it.vmap : &single.vmap;
    const uint32_t bar0 = smem_base + V16_OFF_BAR;

    if (tid == 0) {
        for (int s = 0; s < V16_NST; s++) mbar_init(bar0 + 8u * s, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    auto issue = [&](uint32_t j) { // thread 0 only: tile j of this CTA into stage j % NST
        const uint32_t s = j % V16_NST, bar = bar0 + 8u * s;
        const uint32_t dst = smem_base + s * V16_STAGE;
        const int y = (int)cache_row(it, (t0 + j) * TILE);
        const int x = (int)(kvh * 256u);
        mbar_expect_tx(bar, V16_STAGE);
#pragma unroll
        for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + sb * V16_SUB, kmap, x + 64 * sb, y, bar);
#pragma unroll
        for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + 4 * V16_SUB + sb * V16_SUB, vmap, x + 64 * sb, y, bar);
    };
    // Tiles that lie wholly below `safe_below` hold rows the kernel before this one did not write: their loads
    // start before that kernel is known to have finished. Everything else (Q, the newest rows, all global
    // writes) comes after pdl_wait().
    const uint32_t pre = nt < (uint32_t)V16_NST ? nt : (uint32_t)V16_NST;
    uint32_t early = 0;
    if (tid == 0)
        for (; early < pre && (t0 + early + 1u) * TILE <= it.safe_below; early++) issue(early);
    pdl_wait();
    if (tid == 0)
        for (uint32_t j = early; j < pre; j++) issue(j);

    // Q of this KV head to shared memory as f16: row = tok * 8 + head % 8 (the order of q_dmx, M/dmx.rs:128-138),
    // rows of tokens >= ntok zero; 16-byte chunks swizzled inside each 128-byte group
    {
        uint8_t *qs = smem + V16_OFF_Q;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t idx = tid + 256u * i; // 32 rows x 32 chunks of 8 dims
            const uint32_t row = idx >> 5, chunk = idx & 31u;
            uint4 w = make_uint4(0, 0, 0, 0);
            const uint32_t tok = row >> 3;
            if (tok < it.ntok) {
                const float *src = it.q + (size_t)tok * 4096u + (size_t)(8u * kvh + (row & 7u)) * 256u + chunk * 8u;
                const float4 a = *reinterpret_cast<const float4 *>(src);
                const float4 b = *reinterpret_cast<const float4 *>(src + 4);
                __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
                __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
                w.x = *reinterpret_cast<uint32_t *>(&h0);
                w.y = *reinterpret_cast<uint32_t *>(&h1);
                w.z = *reinterpret_cast<uint32_t *>(&h2);
                w.w = *reinterpret_cast<uint32_t *>(&h3);
            }
            const uint32_t pc = (chunk & ~7u) | ((chunk ^ row) & 7u);
            *reinterpret_cast<uint4 *>(qs + row * 512u + pc * 16u) = w;
        }
    }
    __syncthreads();

    // A fragments of Q for both 16-row tiles and all 16 k-steps
    uint32_t qf[2][16][4];
    {
        const uint32_t qs = smem_base + V16_OFF_Q;
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int ks = 0; ks < 16; ks++) {
                const uint32_t row = mt * 16u + (lane & 7u) + 8u * ((lane >> 3) & 1u);
                const uint32_t chunk = 2u * ks + (lane >> 4);
                const uint32_t pc = (chunk & ~7u) | ((chunk ^ row) & 7u);
                ldmatrix_x4(qf[mt][ks], qs + row * 512u + pc * 16u);
            }
    }

    float o[2][4][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) o[a][b][c] = 0.0f;

    // softmax ownership: 8 threads per row
    const uint32_t srow = tid >> 3, seg = tid & 7u;
    const uint32_t stok = srow >> 3;
    const uint32_t vis = min(it.pos + 1u + stok, it.key_hi);
    const uint32_t klo = lowest_key(it, stok);
    float m_run = NEG_BIG, l_run = 0.0f;
    float *S = reinterpret_cast<float *>(smem + V16_OFF_S);
    float *cfs = reinterpret_cast<float *>(smem + V16_OFF_CF);
    const uint32_t Pbase = smem_base + V16_OFF_P;
    bool aborted = false;
    const uint32_t g = lane >> 2, qd = lane & 3u;

    for (uint32_t j = 0; j < nt; j++) {
        const uint32_t s = j % V16_NST;
        if (!aborted && !mbar_wait_bounded(bar0 + 8u * s, (j / V16_NST) & 1u, WAIT_LIMIT)) {
            aborted = true;
            atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        }
        const uint32_t Kb = smem_base + s * V16_STAGE, Vb = Kb + 4 * V16_SUB;
        {
            // The tile that holds the last visible key also brings rows past it. Their weights are zero, but zero
            // times whatever a caller-owned buffer holds there (NaN, infinity) is not: zero those V rows in shared
            // memory. (K needs nothing: a masked score is replaced, not multiplied.) The stores are ordered before
            // the P V reads by the two barriers in between.
            const uint32_t vend = min(it.pos + it.ntok, it.key_hi), tile0 = (t0 + j) * TILE;
            if (tile0 + TILE > vend) {
                const uint32_t r0 = vend > tile0 ? vend - tile0 : 0u;
                uint8_t *vt = smem + (Vb - smem_base);
                for (uint32_t idx = tid; idx < (TILE - r0) * 32u; idx += 256u) {
                    const uint32_t row = r0 + (idx >> 5), c = idx & 31u; // 4 dim blocks x 8 chunks of 16 bytes
                    *reinterpret_cast<uint4 *>(vt + (c >> 3) * V16_SUB + row * 128u + (c & 7u) * 16u) = make_uint4(0, 0, 0, 0);
                }
            }
        }
        if (MKV_PHASE_OF(it) == 1u) { // measurement: stream the tiles only
            __syncthreads();
            if (tid == 0 && j >= 1 && j - 1 + V16_NST < nt) issue(j - 1 + V16_NST);
            continue;
        }

        // ---- S = Q K^T for keys 8 warp .. 8 warp + 7 ----
        float sc[2][4];
#pragma unroll
        for (int a = 0; a < 2; a++)
#pragma unroll
            for (int c = 0; c < 4; c++) sc[a][c] = 0.0f;
        {
            const uint32_t krow = warp * 8u + (lane & 7u);
            const uint32_t jm = lane >> 3; // which 8x8 matrix this lane addresses
#pragma unroll
            for (int kp = 0; kp < 8; kp++) { // 32 dims per step
                uint32_t kb[4];
                ldmatrix_x4(kb, Kb + (kp >> 1) * V16_SUB + swz128(krow, (kp & 1) * 4u + jm));
                mma_f16(sc[0], qf[0][2 * kp], kb[0], kb[1]);
                mma_f16(sc[1], qf[1][2 * kp], kb[0], kb[1]);
                mma_f16(sc[0], qf[0][2 * kp + 1], kb[2], kb[3]);
                mma_f16(sc[1], qf[1][2 * kp + 1], kb[2], kb[3]);
            }
        }
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            float *r0 = S + (mt * 16u + g) * V16_S_STRIDE + warp * 8u + 2u * qd;
            *reinterpret_cast<float2 *>(r0) = make_float2(sc[mt][0], sc[mt][1]);
            *reinterpret_cast<float2 *>(r0 + 8 * V16_S_STRIDE) = make_float2(sc[mt][2], sc[mt][3]);
        }
        __syncthreads(); // S complete; every warp is past the P V of the previous tile

        if (tid == 0 && j >= 1 && j - 1 + V16_NST < nt) issue(j - 1 + V16_NST); // refill the stage just released

        // ---- softmax of row srow over this tile's 64 keys ----
        {
            const float4 a = *reinterpret_cast<const float4 *>(S + srow * V16_S_STRIDE + seg * 8u);
            const float4 b = *reinterpret_cast<const float4 *>(S + srow * V16_S_STRIDE + seg * 8u + 4u);
            float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
            const uint32_t key0 = (t0 + j) * TILE + seg * 8u;
            float mt_ = NEG_BIG;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                const uint32_t key = key0 + c;
                v[c] = (key >= klo && key < vis) ? v[c] * SCALE : NEG_BIG; // scale, then mask (M/dmx.rs:71)
                mt_ = fmaxf(mt_, v[c]);
            }
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 1));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 2));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 4));
            const float m_new = fmaxf(m_run, mt_);
            float sum = 0.0f;
            uint32_t pk[4];
#pragma unroll
            for (int c = 0; c < 8; c += 2) {
                const float w0 = v[c] > NEG_TEST ? __expf(v[c] - m_new) : 0.0f;
                const float w1 = v[c + 1] > NEG_TEST ? __expf(v[c + 1] - m_new) : 0.0f;
                const __half2 h = __floats2half2_rn(w0, w1);
                const float2 f = __half22float2(h);
                sum += f.x + f.y;
                pk[c >> 1] = *reinterpret_cast<const uint32_t *>(&h);
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            const float cf = m_run > NEG_TEST ? __expf(m_run - m_new) : 0.0f;
            l_run = l_run * cf + sum;
            m_run = m_new;
            *reinterpret_cast<uint4 *>(smem + V16_OFF_P + swz128(srow, seg)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (seg == 0) cfs[srow] = cf;
        }
        __syncthreads(); // P and the rescale factors are visible

        // ---- O = O * cf + P V for dims 32 warp .. 32 warp + 31 ----
        {
            const float c0 = cfs[g], c1 = cfs[g + 8], c2 = cfs[16 + g], c3 = cfs[24 + g];
#pragma unroll
            for (int n = 0; n < 4; n++) {
                o[0][n][0] *= c0; o[0][n][1] *= c0; o[0][n][2] *= c1; o[0][n][3] *= c1;
                o[1][n][0] *= c2; o[1][n][1] *= c2; o[1][n][2] *= c3; o[1][n][3] *= c3;
            }
            const uint32_t Vsub = Vb + (warp >> 1) * V16_SUB;
            const uint32_t cb = (warp & 1u) * 4u;
            const uint32_t jm = lane >> 3;
#pragma unroll
            for (int ks = 0; ks < 4; ks++) { // 16 keys per step
                uint32_t pa[2][4];
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    const uint32_t row = mt * 16u + (lane & 7u) + 8u * ((lane >> 3) & 1u);
                    ldmatrix_x4(pa[mt], Pbase + swz128(row, 2u * ks + (lane >> 4)));
                }
#pragma unroll
                for (int np = 0; np < 2; np++) { // two 8-dim tiles per load
                    uint32_t vb[4];
                    const uint32_t key = 16u * ks + (lane & 7u) + 8u * (jm & 1u);
                    ldmatrix_x4_trans(vb, Vsub + swz128(key, cb + 2u * np + (jm >> 1)));
                    mma_f16(o[0][2 * np], pa[0], vb[0], vb[1]);
                    mma_f16(o[1][2 * np], pa[1], vb[0], vb[1]);
                    mma_f16(o[0][2 * np + 1], pa[0], vb[2], vb[3]);
                    mma_f16(o[1][2 * np + 1], pa[1], vb[2], vb[3]);
                }
            }
        }
    }

    // ---- the piece's partial: [m, l] per row and O[32][256] ----
    const size_t piece = (size_t)kvh * it.nsplit + split;
    if (seg == 0) {
        float2 *ml = reinterpret_cast<float2 *>(it.part_ml) + piece * 32u + srow;
        *ml = make_float2(m_run, l_run);
    }
    {
        float *po = it.part_o + piece * 32u * 256u;
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const uint32_t row = mt * 16u + g, col = warp * 32u + n * 8u + 2u * qd;
                *reinterpret_cast<float2 *>(po + (size_t)row * 256u + col) = make_float2(o[mt][n][0], o[mt][n][1]);
                *reinterpret_cast<float2 *>(po + (size_t)(row + 8u) * 256u + col) = make_float2(o[mt][n][2], o[mt][n][3]);
            }
    }
    // the CTAs that finish last merge the pieces (scratch in the ring, which is drained by now)
    finish_item<256>(it, *reinterpret_cast<FinishSmem *>(smem), status);
}

// Log-sum-exp merge of the pieces of one row: attn_fd_combine's arithmetic (W/ops.wgsl:529-537) over this
// library's pieces. grid = (64 rows, items), 1024 threads = 16 groups of pieces x 64 lanes of 4 dims, so that
// every load of a row's pieces is in flight at once (the pieces sit in L2; the merge is latency-bound).
// In partial mode the merged, un-normalised record [M, tot, acc[256]] is written instead (row = tok * 16 + head),
// for the merge across sequence shards.
constexpr int CMB_THREADS = 1024;
constexpr int CMB_GROUPS = 16;

__global__ void __launch_bounds__(CMB_THREADS)
combine_kernel(const VerifyItem *__restrict__ items, const __grid_constant__ VerifyItem single, int only_empty) {
    const VerifyItem &it = items ? items[blockIdx.y] : single;
    if (only_empty && it.nsplit != 0) return; // items with tiles were merged by the core kernel's last CTAs
    const uint32_t r = blockIdx.x; // kvh * 32 + row
    const uint32_t kvh = r >> 5, row = r & 31u, tok = row >> 3, head = 8u * kvh + (row & 7u);
    const uint32_t tid = threadIdx.x;
    if (tok >= it.ntok) {
        if (it.partial && tid < 258u) // rows of tokens beyond the step: the empty record
            it.out[(size_t)(tok * 16u + head) * REC + tid] = tid == 0 ? NEG_BIG : 0.0f;
        return;
    }
    __shared__ float e_s[MAX_SPLITS];
    __shared__ float red[32];
    __shared__ float tot_s, M_s;
    __shared__ float4 part[CMB_GROUPS][64];
    const uint32_t ns = it.nsplit;
    const float2 *ml = reinterpret_cast<const float2 *>(it.part_ml) + (size_t)kvh * ns * 32u + row;
    float m = NEG_BIG, l = 0.0f;
    if (tid < ns) {
        const float2 x = ml[(size_t)tid * 32u];
        m = x.x;
        l = x.y;
    }
    float M = m;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
    if ((tid & 31u) == 0) red[tid >> 5] = M;
    __syncthreads();
    if (tid < 32) {
        float x = red[tid];
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, sh));
        if (tid == 0) M_s = x;
    }
    __syncthreads();
    M = M_s;
    const float e = tid < ns ? expf(m - M) : 0.0f;
    if (tid < ns) e_s[tid] = e;
    float t = e * l;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) t += __shfl_xor_sync(0xffffffffu, t, sh);
    if ((tid & 31u) == 0) red[tid >> 5] = t; // the maxima in red were all read before the barrier above
    __syncthreads();
    if (tid < 32) {
        float x = red[tid];
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) x += __shfl_xor_sync(0xffffffffu, x, sh);
        if (tid == 0) tot_s = x;
    }
    const uint32_t grp = tid >> 6, d4 = tid & 63u;
    const float4 *po = reinterpret_cast<const float4 *>(it.part_o + ((size_t)kvh * ns * 32u + row) * 256u) + d4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // two rounds of five pieces per group: the five loads of a round are issued before any is used
#pragma unroll
    for (int round = 0; round < 2; round++) {
        float4 x[5];
        const uint32_t s0 = grp + CMB_GROUPS * 5u * round;
        if (s0 >= ns) break;
#pragma unroll
        for (int i = 0; i < 5; i++) {
            const uint32_t s = s0 + CMB_GROUPS * i;
            x[i] = s < ns ? __ldcg(po + (size_t)s * 2048u) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 5; i++) {
            const uint32_t s = s0 + CMB_GROUPS * i;
            const float w = s < ns ? e_s[s] : 0.0f;
            acc.x += w * x[i].x;
            acc.y += w * x[i].y;
            acc.z += w * x[i].z;
            acc.w += w * x[i].w;
        }
    }
    part[grp][d4] = acc;
    __syncthreads();
    if (tid < 64) {
        float4 a = part[0][tid];
#pragma unroll
        for (int g = 1; g < CMB_GROUPS; g++) {
            const float4 b = part[g][tid];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        const float tot = tot_s;
        if (it.partial) {
            float *rec = it.out + (size_t)(tok * 16u + head) * REC; // records are 8-byte aligned only
            *reinterpret_cast<float2 *>(rec + 2 + 4 * tid) = make_float2(a.x, a.y);
            *reinterpret_cast<float2 *>(rec + 4 + 4 * tid) = make_float2(a.z, a.w);
            if (tid == 0) *reinterpret_cast<float2 *>(rec) = make_float2(M, tot);
        } else {
            const float inv = 1.0f / tot;
            *reinterpret_cast<float4 *>(it.out + (size_t)tok * 4096u + (size_t)head * 256u + 4 * tid) =
                make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
        }
    }
}

// Merge of the records of n sequence shards (W/ops.wgsl:529-537 with shards in place of blocks):
// recs = [n_shards][64][258]; grid = 16 * ntok rows; thread = dim.
__global__ void __launch_bounds__(256)
combine_shards_kernel(const float *__restrict__ recs, int n_shards, float *__restrict__ out) {
    const uint32_t r = blockIdx.x, d = threadIdx.x;
    float M = NEG_BIG;
    for (int g = 0; g < n_shards; g++) M = fmaxf(M, recs[((size_t)g * 64u + r) * REC]);
    float tot = 0.0f, acc = 0.0f;
    for (int g = 0; g < n_shards; g++) {
        const float *x = recs + ((size_t)g * 64u + r) * REC;
        const float e = expf(x[0] - M);
        tot += e * x[1];
        acc += e * x[2 + d];
    }
    out[(size_t)r * 256u + d] = acc / tot;
}

// A shard that holds no visible key launches no attention kernel, but it still owes every rank its (empty) record
// rows, and its own output is the merge of the other ranks' rows: one CTA per row does both (exchange_row).
__global__ void __launch_bounds__(256)
exchange_empty_kernel(const PushInfo *__restrict__ push, uint32_t epoch, float *__restrict__ out, uint32_t *__restrict__ status) {
    const uint32_t rr = blockIdx.x, tid = threadIdx.x; // rr = tok * 16 + head
    pdl_launch_dependents();
    pdl_wait(); // the mailbox parity is free only once the launch before last has finished
    const PushInfo &P = *push;
    __shared__ float ml[2 * MAX_PEERS];
    for (uint32_t dd = 0; dd < P.world; dd++) {
        unsigned long long *rec = P.slot[epoch & 1u][dd];
        if (!rec) continue; // a rank that never joined the exchange
        rec += (size_t)rr * REC;
        for (uint32_t i = tid; i < (uint32_t)REC; i += 256u) st_relaxed_sys_u64(rec + i, exch_word(i == 0 ? NEG_BIG : 0.0f, epoch));
    }
    exchange_row<256>(P, epoch, rr, out, status, ml);
}

mkv_status launch_exchange_empty(Ctx *ctx, const PushInfo *push, uint32_t epoch, uint32_t ntok, float *out) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(16u * ntok); // one CTA per row of the record
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    MKV_CUDA(cudaLaunchKernelEx(&cfg, exchange_empty_kernel, push, epoch, out, ctx->dev_status));
    ctx->launches++;
    return MKV_OK;
}

mkv_status launch_combine_shards(Ctx *ctx, const float *recs, int n_shards, uint32_t ntok, float *out) {
    combine_shards_kernel<<<16u * ntok, 256, 0, ctx->stream>>>(recs, n_shards, out);
    ctx->launches++;
    MKV_CUDA(cudaGetLastError());
    return MKV_OK;
}

mkv_status launch_verify_f32(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas,
                             bool ext);
mkv_status verify_f32_setup_device();
mkv_status launch_verify_f16_tc(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas,
                                bool ext);
mkv_status verify_tc_setup_device();
mkv_status launch_verify_f32_tc(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas,
                                bool ext);
mkv_status verify_f32_tc_setup_device();
mkv_status launch_verify_f16_tc_few(Ctx *ctx, const VerifyLaunchBatch &few, int n, uint32_t total_ctas, bool ext);
mkv_status launch_verify_f32_tc_few(Ctx *ctx, const VerifyLaunchBatch &few, int n, uint32_t total_ctas, bool ext);

// MKV_VERIFY=mma selects the warp-MMA kernel of this file for the f16 cache; the default is the tcgen05 kernel.
static bool verify_use_tc() {
    static const bool tc = [] {
        const char *e = getenv("MKV_VERIFY");
        return !(e && strcmp(e, "mma") == 0);
    }();
    return tc;
}
// The f32 cache runs on the tcgen05 kernel of verify_f32_tc.cu; MKV_VERIFY32=mma selects the warp-MMA kernel of
// verify_f32.cu (kept for comparison).
static bool verify32_use_tc() {
    static const bool tc = [] {
        const char *e = getenv("MKV_VERIFY32");
        return !(e && strcmp(e, "mma") == 0);
    }();
    return tc;
}

// dynamic shared memory opt-in for the current device (once per context creation)
mkv_status verify_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)V16_SMEM));
    mkv_status st = verify_tc_setup_device();
    if (st != MKV_OK) return st;
    if ((st = verify_f32_tc_setup_device()) != MKV_OK) return st;
    return verify_f32_setup_device();
}

// items_host[0..n) are planned and have their scratch. Fills in the arrival counters, stages the items
// (batch) or puts the item and its tensor maps in the parameter space (single), launches the core kernel,
// whose last CTAs also merge the pieces. Items without any tile get their (empty) result from the small
// merge kernel.
mkv_status launch_verify(Ctx *ctx, mkv_fmt fmt, VerifyItem *items_host, int n, bool batch, const CUtensorMap *kmap_host,
                         const CUtensorMap *vmap_host) {
    if (n > Ctx::SLOT_ITEMS) {
        set_error("verify batch of %d items exceeds %d", n, Ctx::SLOT_ITEMS);
        return MKV_ERR_INVALID;
    }
    uint32_t total = 0;
    bool any_empty = false, ext = false; // ext: some item uses ring rows, a window or sinks
    for (int i = 0; i < n; i++) {
        ext |= items_host[i].ring != 0 || items_host[i].win != 0 || items_host[i].sinks != nullptr;
        total += 2u * items_host[i].nsplit;
        any_empty |= items_host[i].nsplit == 0;
        items_host[i].counter = ctx->counters_dev + i;
        items_host[i].ticket_base = ctx->counter_base[i];
    }
    // A batch of a few items travels in the kernel's parameter space: no staging copy between two launches (a copy in
    // the stream ends the programmatic overlap of the launches either side of it). Larger batches, and the rare batch with
    // an item that sees no key (its empty result comes from the small merge kernel, which reads the staged items), are staged.
    const bool tc = fmt == MKV_F16 ? verify_use_tc() : verify32_use_tc();
    const bool few = batch && tc && n <= PARAM_ITEMS && !any_empty && total > 0;
    const VerifyItem *items_dev = nullptr;
    if (batch && !few) {
        // next staging slot; wait for the copy that last used it
        const int slot = ctx->slot_next;
        ctx->slot_next = (slot + 1) % Ctx::SLOTS;
        if (ctx->slot_used[slot]) MKV_CUDA(cudaEventSynchronize(ctx->slot_done[slot]));
        VerifyItem *h = ctx->items_host + (size_t)slot * Ctx::SLOT_ITEMS;
        VerifyItem *d = ctx->items_dev + (size_t)slot * Ctx::SLOT_ITEMS;
        memcpy(h, items_host, sizeof(VerifyItem) * (size_t)n);
        MKV_CUDA(cudaMemcpyAsync(d, h, sizeof(VerifyItem) * (size_t)n, cudaMemcpyHostToDevice, ctx->stream));
        MKV_CUDA(cudaEventRecord(ctx->slot_done[slot], ctx->stream));
        ctx->slot_used[slot] = true;
        items_dev = d;
    }
    VerifyLaunch single;
    single.item = items_host[0];
    if (!batch) {
        single.kmap = *kmap_host;
        single.vmap = *vmap_host;
    } else {
        memset(&single.kmap, 0, sizeof single.kmap);
        memset(&single.vmap, 0, sizeof single.vmap);
    }
    cudaEvent_t e1 = nullptr;
    if (ctx->prof) {
        if (ctx->prof_used == ctx->prof_events.size()) {
            cudaEvent_t a, b;
            MKV_CUDA(cudaEventCreate(&a));
            MKV_CUDA(cudaEventCreate(&b));
            ctx->prof_events.push_back({a, b});
        }
        const cudaEvent_t e0 = ctx->prof_events[ctx->prof_used].first;
        e1 = ctx->prof_events[ctx->prof_used].second;
        ctx->prof_used++;
        MKV_CUDA(cudaEventRecord(e0, ctx->stream));
    }
    if (few) {
        VerifyLaunchBatch pb;
        memset(&pb, 0, sizeof pb);
        memcpy(pb.items, items_host, sizeof(VerifyItem) * (size_t)n);
        mkv_status st = fmt == MKV_F16 ? launch_verify_f16_tc_few(ctx, pb, n, total, ext) : launch_verify_f32_tc_few(ctx, pb, n, total, ext);
        if (st != MKV_OK) return st;
        for (int i = 0; i < n; i++) ctx->counter_base[i] += 2u * items_host[i].nsplit;
    } else if (total > 0) {
        if (fmt == MKV_F16 && verify_use_tc()) {
            mkv_status st = launch_verify_f16_tc(ctx, items_dev, n, single, total, ext);
            if (st != MKV_OK) return st;
        } else if (fmt == MKV_F16) {
            // programmatic dependent launch: this kernel's prologue and first tile loads may overlap the tail
            // of the kernel before it in the stream (see pdl_wait in the kernel)
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(total);
            cfg.blockDim = dim3(256);
            cfg.dynamicSmemBytes = V16_SMEM;
            cfg.stream = ctx->stream;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f16_kernel, items_dev, n, single, ctx->dev_status));
            ctx->launches++;
        } else {
            mkv_status st = verify32_use_tc() ? launch_verify_f32_tc(ctx, items_dev, n, single, total, ext)
                                              : launch_verify_f32(ctx, items_dev, n, single, total, ext);
            if (st != MKV_OK) return st;
        }
        for (int i = 0; i < n; i++) ctx->counter_base[i] += 2u * items_host[i].nsplit;
    }
    if (ctx->prof) MKV_CUDA(cudaEventRecord(e1, ctx->stream));
    if (any_empty && !batch && items_host[0].push != nullptr) {
        mkv_status st = launch_exchange_empty(ctx, items_host[0].push, items_host[0].push_epoch, items_host[0].ntok, items_host[0].out);
        if (st != MKV_OK) return st;
    } else if (any_empty) {
        combine_kernel<<<dim3(64, (unsigned)n), CMB_THREADS, 0, ctx->stream>>>(items_dev, single.item, 1);
        ctx->launches++;
        MKV_CUDA(cudaGetLastError());
    }
    return MKV_OK;
}

// ---- verify attention for callers that must not allocate ------------------------------------------------------
//
// Some hosts hand all device memory to their own planner at start-up, or call from a region where allocation
// is forbidden (a latency-critical serving loop, a callback, a driver-level hook), and so cannot let this
// library call cudaMalloc for its split-K pieces. For them the pieces, the arrival counter and the status word
// of one verify launch live in the array below, which is part of the library image: every GPU that loads the
// library holds these 5,284,096 bytes until the process exits, whether or not the entry point is used.
// It holds at most MKV_STATIC_MAX_PIECES pieces (two per CTA pair of KV heads), which covers one CTA per SM on
// a B200 (148). All calls share it and it keeps the last call's contents: calls whose kernels overlap on the
// GPU (different streams) race on it.
constexpr uint32_t STATIC_MAX_PIECES = 160;
constexpr size_t STATIC_HDR = 256; // counter at byte 0, status word at byte 64
constexpr size_t STATIC_ML = (size_t)STATIC_MAX_PIECES * 32 * 2 * sizeof(float);
constexpr size_t STATIC_O = (size_t)STATIC_MAX_PIECES * 32 * 256 * sizeof(float);
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_HDR + STATIC_ML + STATIC_O];

namespace {
constexpr int STATIC_MAX_DEVICES = 64;
struct StaticDevice {
    bool ready = false;
    unsigned char *scratch = nullptr; // device address of g_static_scratch on this device
    int sm_count = 0;
};
StaticDevice g_static_dev[STATIC_MAX_DEVICES];
std::mutex g_static_mutex; // guards g_static_dev and the driver entry point below: the entry point has no context object

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Once per device, with that device current: the device address of the array (in host code its name is only a
// stand-in, not an address a kernel can use), the shared-memory opt-in of the kernel, the SM count.
mkv_status static_setup(int device) {
    std::lock_guard<std::mutex> lock(g_static_mutex);
    StaticDevice &d = g_static_dev[device];
    if (d.ready) return MKV_OK;
    void *p = nullptr;
    MKV_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)V16_SMEM));
    MKV_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    MKV_CUDA(cudaMemset(p, 0, STATIC_HDR)); // counter and status start at zero
    d.scratch = static_cast<unsigned char *>(p);
    d.ready = true;
    return MKV_OK;
}
} // namespace

} // namespace mkv

extern "C" mkv_status mkv_attn_verify_static(int device, void *stream, const void *k_dev, const void *v_dev,
                                             uint32_t capacity_tokens, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                                             const float *q_dev, float *out_dev) {
    using namespace mkv;
    if (device < 0 || device >= STATIC_MAX_DEVICES || !k_dev || !v_dev || !q_dev || !out_dev) {
        set_error("mkv_attn_verify_static: null pointer or device outside [0, %d)", STATIC_MAX_DEVICES);
        return MKV_ERR_INVALID;
    }
    if (ntok < 1 || ntok > MKV_MAX_VERIFY || first_pos > pos) {
        set_error("mkv_attn_verify_static: ntok %u outside [1, %d] or first_pos %u > pos %u", ntok, MKV_MAX_VERIFY, first_pos, pos);
        return MKV_ERR_INVALID;
    }
    if (((uintptr_t)k_dev & 15u) || ((uintptr_t)v_dev & 15u) || ((uintptr_t)q_dev & 15u) || ((uintptr_t)out_dev & 15u)) {
        set_error("mkv_attn_verify_static: k, v, q and out must be 16-byte aligned");
        return MKV_ERR_INVALID;
    }
    if (capacity_tokens == 0 || capacity_tokens > (uint32_t)MKV_CTX_MAX || (uint64_t)pos + ntok > capacity_tokens) {
        set_error("mkv_attn_verify_static: rows [%u, %u) outside a cache of %u rows (at most %d)", first_pos, pos + ntok,
                  capacity_tokens, MKV_CTX_MAX);
        return MKV_ERR_CAPACITY;
    }
    // the caller's current device is put back on every path out of this function
    struct DeviceGuard {
        int before = -1;
        ~DeviceGuard() { if (before >= 0) cudaSetDevice(before); }
    } guard;
    MKV_CUDA(cudaGetDevice(&guard.before));
    if (guard.before == device) guard.before = -1;
    else MKV_CUDA(cudaSetDevice(device));
    mkv_status st = static_setup(device);
    if (st != MKV_OK) return st;
    const StaticDevice &d = g_static_dev[device];

    // the same plan as mkv_attn_verify: contiguous runs of 64-key tiles, one CTA per SM at most
    VerifyLaunch L;
    memset(&L, 0, sizeof L);
    VerifyItem &it = L.item;
    it.q = q_dev;
    it.out = out_dev;
    it.first_pos = first_pos;
    it.pos = pos;
    it.ntok = ntok;
    it.key_hi = capacity_tokens;
    it.tile_begin = first_pos / TILE;
    it.tile_end = (pos + ntok + TILE - 1) / TILE;
    const uint32_t tiles = it.tile_end - it.tile_begin;
    const uint32_t budget = (uint32_t)d.sm_count;
    uint32_t tps = (2u * tiles + budget - 1) / budget;
    if (tps == 0) tps = 1;
    while (2u * ((tiles + tps - 1) / tps) > budget && 2u * ((tiles + tps - 1) / tps) > 2u) tps++;
    it.tiles_per_split = tps;
    it.nsplit = (tiles + tps - 1) / tps;
    if (2u * it.nsplit > STATIC_MAX_PIECES) {
        set_error("mkv_attn_verify_static: this launch needs %u split-K pieces, the static scratch holds %u", 2u * it.nsplit,
                  STATIC_MAX_PIECES);
        return MKV_ERR_CAPACITY;
    }
    it.counter = reinterpret_cast<uint32_t *>(d.scratch);
    it.ticket_base = 0;
    it.part_ml = reinterpret_cast<float *>(d.scratch + STATIC_HDR);
    it.part_o = reinterpret_cast<float *>(d.scratch + STATIC_HDR + STATIC_ML);

    static EncodeTiledFn enc_fn = nullptr;
    EncodeTiledFn enc;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!enc_fn) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
                q != cudaDriverEntryPointSuccess) {
                set_error("cuTensorMapEncodeTiled is not available from the driver");
                return MKV_ERR_CUDA;
            }
            enc_fn = reinterpret_cast<EncodeTiledFn>(fn);
        }
        enc = enc_fn;
    }
    const cuuint64_t dims[2] = {512, capacity_tokens};
    const cuuint64_t strides[1] = {1024};
    const cuuint32_t box[2] = {64, (cuuint32_t)TILE};
    const cuuint32_t estr[2] = {1, 1};
    for (int i = 0; i < 2; i++) {
        const CUresult r = enc(i ? &L.vmap : &L.kmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(i ? v_dev : k_dev),
                               dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            set_error("cuTensorMapEncodeTiled failed with %d", (int)r);
            return MKV_ERR_CUDA;
        }
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the arrival counter must start at zero: the array still holds the last call's count
    MKV_CUDA(cudaMemsetAsync(d.scratch, 0, sizeof(uint32_t), s));
    verify_f16_kernel<<<2u * it.nsplit, 256, V16_SMEM, s>>>(nullptr, 1, L, reinterpret_cast<uint32_t *>(d.scratch + 64));
    MKV_CUDA(cudaGetLastError());
    return MKV_OK;
}

extern "C" mkv_status mkv_static_status(int device, void *stream, uint32_t *status_out) {
    using namespace mkv;
    if (device < 0 || device >= STATIC_MAX_DEVICES || !status_out) {
        set_error("mkv_static_status: null pointer or device outside [0, %d)", STATIC_MAX_DEVICES);
        return MKV_ERR_INVALID;
    }
    *status_out = 0;
    {
        std::lock_guard<std::mutex> lock(g_static_mutex);
        if (!g_static_dev[device].ready) return MKV_OK; // nothing ever ran on this device
    }
    struct DeviceGuard {
        int before = -1;
        ~DeviceGuard() { if (before >= 0) cudaSetDevice(before); }
    } guard;
    MKV_CUDA(cudaGetDevice(&guard.before));
    if (guard.before == device) guard.before = -1;
    else MKV_CUDA(cudaSetDevice(device));
    uint32_t *word = reinterpret_cast<uint32_t *>(g_static_dev[device].scratch + 64);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MKV_CUDA(cudaStreamSynchronize(s));
    MKV_CUDA(cudaMemcpy(status_out, word, sizeof(uint32_t), cudaMemcpyDeviceToHost));
    if (*status_out != 0) {
        MKV_CUDA(cudaMemset(word, 0, sizeof(uint32_t)));
        set_error("a kernel of mkv_attn_verify_static reported status 0x%x (1 = a bounded wait ran out): its output is not valid",
                  *status_out);
        return MKV_ERR_CUDA;
    }
    return MKV_OK;
}

namespace mkv {

// Chooses tiles_per_split so that all items together fill the SMs in one wave (one CTA per SM), and lays
// the items out in the flattened grid. Items must have tile_begin / tile_end set. (A piece need not be a whole number
// of the kernels' tiles: they do not fetch the part of a last tile that lies past the piece.)
void plan_items(Ctx *ctx, VerifyItem *items, int n) {
    uint64_t tiles = 0;
    uint32_t min_tps = 1;
    for (int i = 0; i < n; i++) {
        const uint32_t t = items[i].tile_end - items[i].tile_begin;
        tiles += 2ull * t;
        const uint32_t need = (t + MAX_SPLITS - 1) / MAX_SPLITS;
        if (need > min_tps) min_tps = need;
    }
    const uint32_t budget = (uint32_t)ctx->sm_count;
    uint32_t tps = (uint32_t)((tiles + budget - 1) / budget);
    if (tps < min_tps) tps = min_tps;
    for (;; tps++) {
        uint64_t ctas = 0;
        for (int i = 0; i < n; i++) ctas += 2ull * ((items[i].tile_end - items[i].tile_begin + tps - 1) / tps);
        if (ctas <= budget || ctas <= 2ull * (uint64_t)n) break; // one wave, or nothing left to merge
    }
    uint32_t cta = 0;
    for (int i = 0; i < n; i++) {
        const uint32_t t = items[i].tile_end - items[i].tile_begin;
        items[i].tiles_per_split = tps;
        items[i].nsplit = (t + tps - 1) / tps;
        items[i].cta_begin = cta;
        cta += 2u * items[i].nsplit;
    }
}

} // namespace mkv
