// Decode / verify attention over the f16 cache: split-K flash-decode for up to 4 tokens x 8 query heads
// (32 rows) per KV head, then a log-sum-exp combine of the pieces.
//
// Stands in for q_dmx + attn_dmx2 + attn_fd_combine of the reference (M/dmx.rs:19-141, W/ops.wgsl:523-538):
// same visibility rule (token t at pos + t sees first_pos <= key < pos + 1 + t), same mask value, same
// un-normalised partial [m, l, O] per piece, one divide at the end. What differs is the machine mapping:
//  - a CTA owns one KV head and a contiguous run of 32-key tiles; K and V tiles arrive by TMA
//    (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a 6-deep ring of 32 KB slots, each filled
//    tile signalled on an mbarrier;
//  - two groups of 8 warps take alternate tiles, so one group's softmax overlaps the other's tensor work;
//  - S = Q K^T by mma.m16n8k16 with the Q fragments in registers (f16); softmax with 8 threads per row, max
//    and sum by warp shuffles, P rounded to f16 (as the reference does) and the row sum taken over the
//    rounded values; O += P V with warp w of a group owning dims 32w..32w+31, so every V byte is read from
//    shared memory once per group.
#include <string.h>

#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int V16_NST = 6;                       // ring depth (three slots per warp group)
constexpr uint32_t V16_STAGE = 32768;            // K 16 KB + V 16 KB: one tile of 32 keys
constexpr uint32_t V16_SUB = 4096;               // one [32 keys][64 dims] f16 sub-box
constexpr uint32_t V16_OFF_Q = V16_NST * V16_STAGE;
constexpr uint32_t V16_S_STRIDE = 36;            // floats per S row (32 + 4 of padding)
constexpr uint32_t V16_GRP_BYTES = 32 * V16_S_STRIDE * 4 + 32 * 64 + 32 * 4; // S, P, rescale factors of one group
constexpr uint32_t V16_OFF_GRP = V16_OFF_Q + 32 * 512;
constexpr uint32_t V16_OFF_ML = V16_OFF_GRP + 2 * V16_GRP_BYTES; // [2 groups][32 rows] (m, l) for the final merge
constexpr uint32_t V16_OFF_BAR = V16_OFF_ML + 2 * 32 * 8;
constexpr uint32_t V16_OFF_PRM = V16_OFF_BAR + V16_NST * 8;      // what the TMA issuers need, kept out of registers
constexpr uint32_t V16_SMEM = V16_OFF_PRM + 32 + 1024;           // + alignment slack

struct IssueParams {
    const CUtensorMap *kmap, *vmap;
    int x, y0; // box coordinates of the CTA's first tile
    volatile uint32_t abort; // set once a bounded wait ran out: later waits are skipped
};
constexpr long long WAIT_LIMIT = 4000000000ll;   // about two seconds of SM clocks

__device__ __forceinline__ const VerifyItem &pick_item(const VerifyItem *items, int n_items, const VerifyItem &single,
                                                       uint32_t cta) {
    if (items == nullptr) return single;
    int lo = 0;
    for (int i = 1; i < n_items; i++)
        if (cta >= items[i].cta_begin) lo = i;
    return items[lo];
}

// named barriers of a warp group: 0 = S complete, 1 = P complete, 2 = the tile's slot is released
__device__ __forceinline__ void group_sync(uint32_t group, uint32_t which) {
    asm volatile("bar.sync %0, 256;" ::"r"(1u + 3u * group + which) : "memory");
}
__device__ __forceinline__ void group_arrive(uint32_t group, uint32_t which) {
    asm volatile("bar.arrive %0, 256;" ::"r"(1u + 3u * group + which) : "memory");
}
// P rows are 64 bytes (32 keys of f16): 16-byte chunk XOR (row / 2) mod 4 keeps ldmatrix conflict-free
__device__ __forceinline__ uint32_t p_off(uint32_t row, uint32_t chunk) { return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4); }

// A CTA = one KV head x a contiguous run of 32-key tiles, worked by two groups of 8 warps that take alternate
// tiles, each with its own running (m, l, O); while one group is in its softmax the other feeds the tensor
// pipe. The two states are merged through shared memory at the end, so a CTA still writes one piece.
__global__ void __launch_bounds__(512, 1)
verify_f16_kernel(const VerifyItem *__restrict__ items, int n_items, const __grid_constant__ VerifyLaunch single,
                  uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const VerifyItem &it = pick_item(items, n_items, single.item, blockIdx.x);
    const uint32_t tid = threadIdx.x, lane = tid & 31u;
    const uint32_t group = tid >> 8, gtid = tid & 255u, gw = gtid >> 5; // warp group, thread and warp inside it
    const uint32_t local = blockIdx.x - it.cta_begin;
    if (local >= 2u * it.nsplit) return;
    if (it.phase == 2u) return; // measurement: launch cost alone
    const uint32_t kvh = local & 1u, split = local >> 1;
    const uint32_t t0 = it.tile_begin + split * it.tiles_per_split;
    const uint32_t t1 = min(t0 + it.tiles_per_split, it.tile_end);
    const uint32_t nt = it.phase == 3u ? 0u : t1 - t0; // measurement: prologue and epilogue without tiles
    const uint32_t bar0 = smem_base + V16_OFF_BAR;
    IssueParams *prm = reinterpret_cast<IssueParams *>(smem + V16_OFF_PRM);

    if (tid == 0) {
        for (int s = 0; s < V16_NST; s++) mbar_init(bar0 + 8u * s, 1);
        prm->kmap = items ? it.kmap : &single.kmap; // a single launch carries its maps in the parameter space
        prm->vmap = items ? it.vmap : &single.vmap;
        prm->x = (int)(kvh * 256u);
        prm->y0 = (int)(t0 * TILE - it.row0);
        prm->abort = 0;
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    auto issue = [&](uint32_t j) { // one thread of the group that owns tile j: into slot j % NST
        const uint32_t s = j % V16_NST, bar = bar0 + 8u * s;
        const uint32_t dst = smem_base + s * V16_STAGE;
        const CUtensorMap *kmap = prm->kmap, *vmap = prm->vmap;
        const int x = prm->x, y = prm->y0 + (int)(j * TILE);
        mbar_expect_tx(bar, V16_STAGE);
#pragma unroll
        for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + sb * V16_SUB, kmap, x + 64 * sb, y, bar);
#pragma unroll
        for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + 4 * V16_SUB + sb * V16_SUB, vmap, x + 64 * sb, y, bar);
    };
    if (gtid == 0) {
        for (uint32_t j = group; j < nt && j < (uint32_t)V16_NST; j += 2) issue(j);
    }

    // Q of this KV head to shared memory as f16: row = tok * 8 + head % 8 (the order of q_dmx, M/dmx.rs:128-138),
    // rows of tokens >= ntok zero; 16-byte chunks swizzled inside each 128-byte group
    {
        uint8_t *qs = smem + V16_OFF_Q;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t idx = tid + 512u * i; // 32 rows x 32 chunks of 8 dims
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

    // S = Q K^T: warp gw of a group takes the 16-row tile mt = gw & 1 and keys 8 kq .. 8 kq + 7, kq = gw >> 1.
    // Its A fragments of Q (16 rows x 256 dims) live in registers for the whole kernel.
    const uint32_t mt = gw & 1u, kq = gw >> 1;
    uint32_t qf[16][4];
    {
        const uint32_t qs = smem_base + V16_OFF_Q;
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            const uint32_t row = mt * 16u + (lane & 7u) + 8u * ((lane >> 3) & 1u);
            const uint32_t chunk = 2u * ks + (lane >> 4);
            const uint32_t pc = (chunk & ~7u) | ((chunk ^ row) & 7u);
            ldmatrix_x4(qf[ks], qs + row * 512u + pc * 16u);
        }
    }

    float o[2][4][4]; // O += P V: warp gw owns dims 32 gw .. 32 gw + 31 of all 32 rows
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) o[a][b][c] = 0.0f;

    // softmax ownership inside the group: 8 threads per row, 4 keys each
    const uint32_t srow = gtid >> 3, seg = gtid & 7u;
    const uint32_t vis = min(it.pos + 1u + (srow >> 3), it.key_hi);
    const uint32_t klo = max(it.first_pos, it.key_lo);
    float m_run = NEG_BIG, l_run = 0.0f;
    uint8_t *gmem = smem + V16_OFF_GRP + group * V16_GRP_BYTES;
    float *S = reinterpret_cast<float *>(gmem);
    uint8_t *P = gmem + 32 * V16_S_STRIDE * 4;
    float *cfs = reinterpret_cast<float *>(P + 32 * 64);
    const uint32_t Pbase = smem_base + V16_OFF_GRP + group * V16_GRP_BYTES + 32 * V16_S_STRIDE * 4;
    const uint32_t g = lane >> 2, qd = lane & 3u;

    for (uint32_t j = group; j < nt; j += 2) {
        const uint32_t s = j % V16_NST;
        if (lane == 0 && !prm->abort && !mbar_wait_bounded(bar0 + 8u * s, (j / V16_NST) & 1u, WAIT_LIMIT)) {
            prm->abort = 1; // one lane per warp polls, so that waiting warps leave the shared-memory pipe alone
            atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        }
        __syncwarp();
        const uint32_t Kb = smem_base + s * V16_STAGE, Vb = Kb + 4 * V16_SUB;
        if (it.phase == 1u) { // measurement: stream the tiles only
            group_sync(group, 0);
            if (gtid == 0 && j + V16_NST < nt) issue(j + V16_NST);
            continue;
        }

        // ---- S(16 x 8) = Q K^T ----
        {
            float sa[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t krow = kq * 8u + (lane & 7u);
            const uint32_t jm = lane >> 3; // which 8x8 matrix this lane addresses
#pragma unroll
            for (int kp = 0; kp < 8; kp++) { // 32 dims per step
                uint32_t kb[4];
                ldmatrix_x4(kb, Kb + (kp >> 1) * V16_SUB + swz128(krow, (kp & 1) * 4u + jm));
                mma_f16(sa, qf[2 * kp], kb[0], kb[1]);
                mma_f16(sa, qf[2 * kp + 1], kb[2], kb[3]);
            }
            float *r0 = S + (mt * 16u + g) * V16_S_STRIDE + kq * 8u + 2u * qd;
            *reinterpret_cast<float2 *>(r0) = make_float2(sa[0], sa[1]);
            *reinterpret_cast<float2 *>(r0 + 8 * V16_S_STRIDE) = make_float2(sa[2], sa[3]);
        }
        group_sync(group, 0); // S complete; every warp of the group is past the P V of its previous tile

        // ---- softmax of row srow over this tile's 32 keys ----
        {
            const float4 a = *reinterpret_cast<const float4 *>(S + srow * V16_S_STRIDE + seg * 4u);
            float v[4] = {a.x, a.y, a.z, a.w};
            const uint32_t key0 = (t0 + j) * TILE + seg * 4u;
            float mt_ = NEG_BIG;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t key = key0 + c;
                v[c] = (key >= klo && key < vis) ? v[c] * SCALE : NEG_BIG; // scale, then mask (M/dmx.rs:71)
                mt_ = fmaxf(mt_, v[c]);
            }
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 1));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 2));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 4));
            const float m_new = fmaxf(m_run, mt_);
            const float w0 = v[0] > NEG_TEST ? __expf(v[0] - m_new) : 0.0f;
            const float w1 = v[1] > NEG_TEST ? __expf(v[1] - m_new) : 0.0f;
            const float w2 = v[2] > NEG_TEST ? __expf(v[2] - m_new) : 0.0f;
            const float w3 = v[3] > NEG_TEST ? __expf(v[3] - m_new) : 0.0f;
            const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            float sum = (f01.x + f01.y) + (f23.x + f23.y); // the sum of the rounded weights, as M/dmx.rs:84
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            const float cf = m_run > NEG_TEST ? __expf(m_run - m_new) : 0.0f;
            l_run = l_run * cf + sum;
            m_run = m_new;
            *reinterpret_cast<uint2 *>(P + p_off(srow, seg >> 1) + (seg & 1u) * 8u) =
                make_uint2(*reinterpret_cast<const uint32_t *>(&h01), *reinterpret_cast<const uint32_t *>(&h23));
            if (seg == 0) cfs[srow] = cf;
        }
        group_sync(group, 1); // P and the rescale factors are visible

        // ---- O = O * cf + P V for dims 32 gw .. 32 gw + 31 ----
        {
            const float c0 = cfs[g], c1 = cfs[g + 8], c2 = cfs[16 + g], c3 = cfs[24 + g];
#pragma unroll
            for (int n = 0; n < 4; n++) {
                o[0][n][0] *= c0; o[0][n][1] *= c0; o[0][n][2] *= c1; o[0][n][3] *= c1;
                o[1][n][0] *= c2; o[1][n][1] *= c2; o[1][n][2] *= c3; o[1][n][3] *= c3;
            }
            const uint32_t Vsub = Vb + (gw >> 1) * V16_SUB;
            const uint32_t cb = (gw & 1u) * 4u;
            const uint32_t jm = lane >> 3;
#pragma unroll
            for (int ks = 0; ks < 2; ks++) { // 16 keys per step
                uint32_t pa[2][4];
#pragma unroll
                for (int m2 = 0; m2 < 2; m2++) {
                    const uint32_t row = m2 * 16u + (lane & 7u) + 8u * ((lane >> 3) & 1u);
                    ldmatrix_x4(pa[m2], Pbase + p_off(row, 2u * ks + (lane >> 4)));
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
        // the slot is free once all 8 warps are done with it: warp 0 waits for the others' arrival and
        // refills it at once with the tile three of the group's turns ahead
        if (gw != 0) group_arrive(group, 2);
        else {
            group_sync(group, 2);
            if (lane == 0 && j + V16_NST < nt) issue(j + V16_NST);
        }
    }

    // ---- merge the two groups' states through shared memory, then write the CTA's piece ----
    float2 *mls = reinterpret_cast<float2 *>(smem + V16_OFF_ML); // [group][row]
    if (seg == 0) mls[group * 32u + srow] = make_float2(m_run, l_run);
    __syncthreads(); // every tile is consumed: the ring is free to hold group 1's O
    float *xo = reinterpret_cast<float *>(smem); // [32 rows][256 + 8]: padded against bank conflicts
    constexpr uint32_t XS = 264;
    if (group == 1) {
#pragma unroll
        for (int m2 = 0; m2 < 2; m2++)
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const uint32_t row = m2 * 16u + g, col = gw * 32u + n * 8u + 2u * qd;
                *reinterpret_cast<float2 *>(xo + row * XS + col) = make_float2(o[m2][n][0], o[m2][n][1]);
                *reinterpret_cast<float2 *>(xo + (row + 8u) * XS + col) = make_float2(o[m2][n][2], o[m2][n][3]);
            }
    }
    __syncthreads();
    if (group == 0) {
        const size_t piece = (size_t)kvh * it.nsplit + split;
        float *po = it.part_o + piece * 32u * 256u;
#pragma unroll
        for (int m2 = 0; m2 < 2; m2++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint32_t row = m2 * 16u + g + 8u * h;
                const float2 a = mls[row], b = mls[32u + row];
                const float M = fmaxf(a.x, b.x);
                const float ea = __expf(a.x - M), eb = __expf(b.x - M); // both -3e38: 1 and 1, with l = 0 and O = 0
#pragma unroll
                for (int n = 0; n < 4; n++) {
                    const uint32_t col = gw * 32u + n * 8u + 2u * qd;
                    const float2 x = *reinterpret_cast<const float2 *>(xo + row * XS + col);
                    *reinterpret_cast<float2 *>(po + (size_t)row * 256u + col) =
                        make_float2(o[m2][n][2 * h] * ea + x.x * eb, o[m2][n][2 * h + 1] * ea + x.y * eb);
                }
                if (gw == 0 && qd == 0)
                    reinterpret_cast<float2 *>(it.part_ml)[piece * 32u + row] = make_float2(M, a.y * ea + b.y * eb);
            }
    }
    // the CTAs that finish last merge the pieces (scratch in the ring, beyond group 1's O)
    finish_item<512>(it, *reinterpret_cast<FinishSmem *>(smem + 65536), status);
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

mkv_status launch_combine_shards(Ctx *ctx, const float *recs, int n_shards, uint32_t ntok, float *out) {
    combine_shards_kernel<<<16u * ntok, 256, 0, ctx->stream>>>(recs, n_shards, out);
    ctx->launches++;
    MKV_CUDA(cudaGetLastError());
    return MKV_OK;
}

mkv_status launch_verify_f32(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas);
mkv_status verify_f32_setup_device();

// dynamic shared memory opt-in for the current device (once per context creation)
mkv_status verify_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)V16_SMEM));
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
    bool any_empty = false;
    for (int i = 0; i < n; i++) {
        total += 2u * items_host[i].nsplit;
        any_empty |= items_host[i].nsplit == 0;
        items_host[i].counter = ctx->counters_dev + i;
        items_host[i].ticket_base = ctx->counter_base[i];
    }
    const VerifyItem *items_dev = nullptr;
    if (batch) {
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
    if (total > 0) {
        if (fmt == MKV_F16) {
            verify_f16_kernel<<<total, 512, V16_SMEM, ctx->stream>>>(items_dev, n, single, ctx->dev_status);
            ctx->launches++;
            MKV_CUDA(cudaGetLastError());
        } else {
            mkv_status st = launch_verify_f32(ctx, items_dev, n, single, total);
            if (st != MKV_OK) return st;
        }
        for (int i = 0; i < n; i++) ctx->counter_base[i] += 2u * items_host[i].nsplit;
    }
    if (ctx->prof) MKV_CUDA(cudaEventRecord(e1, ctx->stream));
    if (any_empty) {
        combine_kernel<<<dim3(64, (unsigned)n), CMB_THREADS, 0, ctx->stream>>>(items_dev, single.item, 1);
        ctx->launches++;
        MKV_CUDA(cudaGetLastError());
    }
    return MKV_OK;
}

// Chooses tiles_per_split so that all items together fill the SMs in one wave (one CTA per SM), and lays
// the items out in the flattened grid. Items must have tile_begin / tile_end set.
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
