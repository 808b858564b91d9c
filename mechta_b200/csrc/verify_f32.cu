// Decode / verify attention over the f32 cache (and the MTP window, which the reference also runs through
// its f32-math kernels): split-K flash-decode with f32-grade arithmetic on the tensor cores.
//
// Stands in for attn_fd / attn_fd2h (W/ops.wgsl:325-516), which compute in f32. The tolerance here is 1e-5,
// which one f16 or tf32 product cannot give, and a scalar f32 version is bound by the FMA pipe at a quarter of
// the HBM rate (16 FMA per cache byte; measured 1.6 TB/s). So every f32 operand x is split into two f16 values,
// hi = f16(x) and lo = f16(x - hi) (together 22 bits of mantissa), and a product a.b is taken as
//   a_hi.b_hi + a_hi.b_lo + a_lo.b_hi     (the dropped a_lo.b_lo is below 2^-22 of the product)
// with f16 x f16 products exact in the f32 accumulator: three mma.m16n8k16 instead of one. The small terms get
// their own accumulators in Q K^T. Against an f64 computation this gives 8e-7 on seeded N(0,1) data, the same as
// plain f32.
//  - K and V tiles of 32 keys arrive as f32 by TMA (128-byte swizzle, no multicast) into a 2-deep ring;
//  - all threads convert the tile to four f16 tiles (K hi/lo, V hi/lo) in the layout the ldmatrix loads expect;
//  - S = Q K^T: warp w takes the 16-row tile w & 1 and keys 8 (w >> 1) .. +7; its Q fragments (hi and lo) live in
//    registers; softmax with 8 threads per row as in the f16 kernel, P written as hi and lo;
//  - O += P V: warp w owns dims 32w..32w+31 of all rows.
// Same pieces, in-kernel merge and programmatic dependent launch as the f16 kernel.
#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int V32_NST = 2;
constexpr uint32_t V32_STAGE = 65536;                     // raw f32: K 32 KB + V 32 KB (32 keys)
constexpr uint32_t V32_SUB = 4096;                        // one raw [32 keys][32 dims] f32 sub-box
constexpr uint32_t V32_HSUB = 4096;                       // one converted [32 keys][64 dims] f16 sub-box
constexpr uint32_t V32_OFF_H = V32_NST * V32_STAGE;       // K hi, K lo, V hi, V lo: 4 x 16 KB (Q hi/lo before the loop)
constexpr uint32_t V32_HTILE = 16384;
constexpr uint32_t V32_OFF_QL = V32_OFF_H + 4 * V32_HTILE;  // Q lo, [32 rows][512 B], read again for every tile
constexpr uint32_t V32_OFF_S = V32_OFF_QL + V32_HTILE;
constexpr uint32_t V32_S_STRIDE = 36;                     // floats per S row (32 keys + 4 of padding)
constexpr uint32_t V32_OFF_P = V32_OFF_S + 32 * V32_S_STRIDE * 4; // P hi then P lo: [32 rows][64 B] each
constexpr uint32_t V32_OFF_CF = V32_OFF_P + 2 * 32 * 64;
constexpr uint32_t V32_OFF_BAR = V32_OFF_CF + 32 * 4;
constexpr uint32_t V32_SMEM = V32_OFF_BAR + V32_NST * 8 + 1024;
constexpr long long WAIT_LIMIT32 = 4000000000ll;

// P rows are 64 bytes (32 keys of f16): 16-byte chunk XOR (row / 2) mod 4 keeps ldmatrix conflict-free
__device__ __forceinline__ uint32_t p32_off(uint32_t row, uint32_t chunk) { return row * 64u + ((chunk ^ ((row >> 1) & 3u)) << 4); }

// hi and lo halves of 8 floats as two 16-byte vectors of f16
__device__ __forceinline__ void split8(const float (&x)[8], uint4 &hi, uint4 &lo) {
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

template <bool EXT> // ring rows, sliding window and sinks compiled in or out, as in verify_tc.cu
__global__ void __launch_bounds__(256, 1)
verify_f32_kernel(const VerifyItem *__restrict__ items, int n_items, const __grid_constant__ VerifyLaunch single,
                  uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));

    const VerifyItem *itp = &single.item;
    if (items != nullptr) {
        int lo = 0;
        for (int i = 1; i < n_items; i++)
            if (blockIdx.x >= items[i].cta_begin) lo = i;
        itp = items + lo;
    }
    const VerifyItem &it = *itp;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t local = blockIdx.x - it.cta_begin;
    if (local >= 2u * it.nsplit) return;
    pdl_launch_dependents(); // the next kernel in the stream may begin its own prologue
    const uint32_t kvh = local & 1u, split = local >> 1;
    const uint32_t t0 = it.tile_begin + split * it.tiles_per_split;
    const uint32_t t1 = min(t0 + it.tiles_per_split, it.tile_end);
    const uint32_t nt = t1 - t0;
    const CUtensorMap *kmap = items ? it.kmap : &single.kmap, *vmap = items ? it.vmap : &single.vmap;
    const uint32_t bar0 = smem_base + V32_OFF_BAR;

    if (tid == 0) {
        for (int s = 0; s < V32_NST; s++) mbar_init(bar0 + 8u * s, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    auto issue = [&](uint32_t j) {
        const uint32_t s = j % V32_NST, bar = bar0 + 8u * s;
        const uint32_t dst = smem_base + s * V32_STAGE;
        const int y = (int)(EXT ? cache_row(it, (t0 + j) * TILE32) : (t0 + j) * TILE32 - it.row0);
        const int x = (int)(kvh * 256u);
        mbar_expect_tx(bar, V32_STAGE);
#pragma unroll
        for (int sb = 0; sb < 8; sb++) tma_load_2d(dst + sb * V32_SUB, kmap, x + 32 * sb, y, bar);
#pragma unroll
        for (int sb = 0; sb < 8; sb++) tma_load_2d(dst + 8 * V32_SUB + sb * V32_SUB, vmap, x + 32 * sb, y, bar);
    };
    // tiles wholly below `safe_below` were not written by the kernel before this one: their loads start before
    // that kernel is known to have finished; Q, the newest rows and all global writes come after pdl_wait()
    const uint32_t pre = nt < (uint32_t)V32_NST ? nt : (uint32_t)V32_NST;
    uint32_t early = 0;
    if (tid == 0)
        for (; early < pre && (t0 + early + 1u) * TILE32 <= it.safe_below; early++) issue(early);
    pdl_wait();
    if (tid == 0)
        for (uint32_t j = early; j < pre; j++) issue(j);

    // Q of this KV head as f16 hi and lo to shared memory (where the converted tiles go later): row = tok * 8 +
    // head % 8, rows of tokens >= ntok zero; 16-byte chunks swizzled inside each 128-byte group
    {
        uint8_t *qh = smem + V32_OFF_H, *ql = smem + V32_OFF_QL;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t idx = tid + 256u * i; // 32 rows x 32 chunks of 8 dims
            const uint32_t row = idx >> 5, chunk = idx & 31u;
            float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if ((row >> 3) < it.ntok) {
                const float *src = it.q + (size_t)(row >> 3) * 4096u + (size_t)(8u * kvh + (row & 7u)) * 256u + chunk * 8u;
                const float4 a = *reinterpret_cast<const float4 *>(src);
                const float4 b = *reinterpret_cast<const float4 *>(src + 4);
                x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
            }
            uint4 hi, lo;
            split8(x, hi, lo);
            const uint32_t off = row * 512u + (((chunk & ~7u) | ((chunk ^ row) & 7u)) << 4);
            *reinterpret_cast<uint4 *>(qh + off) = hi;
            *reinterpret_cast<uint4 *>(ql + off) = lo;
        }
    }
    __syncthreads();

    // this warp's A fragments of Q hi (16-row tile mt, all 16 k-steps) stay in registers; the lo fragments are
    // read from shared memory for every tile (there are not enough registers for both)
    const uint32_t mt = warp & 1u, kq = warp >> 1;
    uint32_t qfh[16][4];
    const uint32_t qrow = mt * 16u + (lane & 7u) + 8u * ((lane >> 3) & 1u);
    {
        const uint32_t qs = smem_base + V32_OFF_H;
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            const uint32_t chunk = 2u * ks + (lane >> 4);
            ldmatrix_x4(qfh[ks], qs + qrow * 512u + (((chunk & ~7u) | ((chunk ^ qrow) & 7u)) << 4));
        }
    }
    const uint32_t qlo = smem_base + V32_OFF_QL + qrow * 512u;
    __syncthreads(); // Q hi's place in shared memory is free for the converted tiles

    float o[2][4][4]; // O += P V: warp w owns dims 32w..32w+31 of all 32 rows
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) o[a][b][c] = 0.0f;

    const uint32_t srow = tid >> 3, seg = tid & 7u; // softmax: 8 threads per row, 4 keys each
    const uint32_t vis = min(it.pos + 1u + (srow >> 3), it.key_hi);
    const uint32_t klo = EXT ? lowest_key(it, srow >> 3) : max(it.first_pos, it.key_lo);
    float m_run = NEG_BIG, l_run = 0.0f;
    float *S = reinterpret_cast<float *>(smem + V32_OFF_S);
    float *cfs = reinterpret_cast<float *>(smem + V32_OFF_CF);
    uint8_t *Ph = smem + V32_OFF_P, *Pl = Ph + 32 * 64;
    const uint32_t Hb = smem_base + V32_OFF_H; // K hi, K lo, V hi, V lo
    const uint32_t g = lane >> 2, qd = lane & 3u;
    bool aborted = false;

    for (uint32_t j = 0; j < nt; j++) {
        const uint32_t s = j % V32_NST;
        if (!aborted && !mbar_wait_bounded(bar0 + 8u * s, (j / V32_NST) & 1u, WAIT_LIMIT32)) {
            aborted = true;
            atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        }
        // ---- f32 tile -> K hi, K lo, V hi, V lo as f16: lane = key, the warp walks groups of 8 dims ----
        {
            const uint8_t *raw = smem + s * V32_STAGE;
            uint8_t *H = smem + V32_OFF_H;
#pragma unroll
            for (int kv = 0; kv < 2; kv++)
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint32_t jj = warp + 8u * i; // dims 8 jj .. 8 jj + 7
                    const uint8_t *src = raw + kv * 8 * V32_SUB + (jj >> 2) * V32_SUB;
                    const float4 a = *reinterpret_cast<const float4 *>(src + swz128(lane, (jj & 3u) * 2u));
                    const float4 b = *reinterpret_cast<const float4 *>(src + swz128(lane, (jj & 3u) * 2u + 1u));
                    const float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                    uint4 hi, lo;
                    split8(x, hi, lo);
                    uint8_t *dst = H + kv * 2 * V32_HTILE + (jj >> 3) * V32_HSUB + swz128(lane, jj & 7u);
                    *reinterpret_cast<uint4 *>(dst) = hi;
                    *reinterpret_cast<uint4 *>(dst + V32_HTILE) = lo;
                }
        }
        __syncthreads(); // the converted tile is complete; the raw stage is free
        if (tid == 0 && j + V32_NST < nt) issue(j + V32_NST);

        // ---- S(16 x 8) = Q K^T in three terms ----
        {
            float shh[4] = {0.f, 0.f, 0.f, 0.f}, shl[4] = {0.f, 0.f, 0.f, 0.f}, slh[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t krow = kq * 8u + (lane & 7u), jm = lane >> 3;
#pragma unroll
            for (int kp = 0; kp < 8; kp++) { // 32 dims per step
                uint32_t kh[4], kl[4], ql0[4], ql1[4];
                const uint32_t a = Hb + (kp >> 1) * V32_HSUB + swz128(krow, (kp & 1) * 4u + jm);
                ldmatrix_x4(kh, a);
                ldmatrix_x4(kl, a + V32_HTILE);
                {
                    const uint32_t c0 = 4u * kp + (lane >> 4), c1 = c0 + 2u;
                    ldmatrix_x4(ql0, qlo + (((c0 & ~7u) | ((c0 ^ qrow) & 7u)) << 4));
                    ldmatrix_x4(ql1, qlo + (((c1 & ~7u) | ((c1 ^ qrow) & 7u)) << 4));
                }
                mma_f16(shh, qfh[2 * kp], kh[0], kh[1]);
                mma_f16(shl, qfh[2 * kp], kl[0], kl[1]);
                mma_f16(slh, ql0, kh[0], kh[1]);
                mma_f16(shh, qfh[2 * kp + 1], kh[2], kh[3]);
                mma_f16(shl, qfh[2 * kp + 1], kl[2], kl[3]);
                mma_f16(slh, ql1, kh[2], kh[3]);
            }
            float *r0 = S + (mt * 16u + g) * V32_S_STRIDE + kq * 8u + 2u * qd;
            *reinterpret_cast<float2 *>(r0) = make_float2(shh[0] + (shl[0] + slh[0]), shh[1] + (shl[1] + slh[1]));
            *reinterpret_cast<float2 *>(r0 + 8 * V32_S_STRIDE) = make_float2(shh[2] + (shl[2] + slh[2]), shh[3] + (shl[3] + slh[3]));
        }
        __syncthreads(); // S complete; every warp is past the P V of the previous tile

        // ---- softmax of row srow over this tile's 32 keys; P as hi + lo ----
        {
            const float4 a = *reinterpret_cast<const float4 *>(S + srow * V32_S_STRIDE + seg * 4u);
            float v[4] = {a.x, a.y, a.z, a.w};
            const uint32_t key0 = (t0 + j) * TILE32 + seg * 4u;
            float mt_ = NEG_BIG;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t key = key0 + c;
                v[c] = (key >= klo && key < vis) ? v[c] * SCALE : NEG_BIG; // scale, then mask (W/ops.wgsl:361)
                mt_ = fmaxf(mt_, v[c]);
            }
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 1));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 2));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 4));
            const float m_new = fmaxf(m_run, mt_);
            float w[4], sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                w[c] = v[c] > NEG_TEST ? expf(v[c] - m_new) : 0.0f;
                sum += w[c];
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            const float cf = m_run > NEG_TEST ? expf(m_run - m_new) : 0.0f;
            l_run = l_run * cf + sum;
            m_run = m_new;
            const __half2 h01 = __floats2half2_rn(w[0], w[1]), h23 = __floats2half2_rn(w[2], w[3]);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            const __half2 l01 = __floats2half2_rn(w[0] - f01.x, w[1] - f01.y), l23 = __floats2half2_rn(w[2] - f23.x, w[3] - f23.y);
            const uint32_t off = p32_off(srow, seg >> 1) + (seg & 1u) * 8u;
            *reinterpret_cast<uint2 *>(Ph + off) =
                make_uint2(*reinterpret_cast<const uint32_t *>(&h01), *reinterpret_cast<const uint32_t *>(&h23));
            *reinterpret_cast<uint2 *>(Pl + off) =
                make_uint2(*reinterpret_cast<const uint32_t *>(&l01), *reinterpret_cast<const uint32_t *>(&l23));
            if (seg == 0) cfs[srow] = cf;
        }
        __syncthreads(); // P and the rescale factors are visible

        // ---- O = O * cf + P V in three terms, dims 32 warp .. 32 warp + 31 ----
        {
            // The tensor core's f32 accumulation truncates; over hundreds of tiles that bias would reach 1e-5. So each
            // tile's P V starts from zero (6 MMAs deep) and is folded into O with a rounded FMA: O = O * cf + tile.
            float ot[2][4][4];
#pragma unroll
            for (int a = 0; a < 2; a++)
#pragma unroll
                for (int b = 0; b < 4; b++)
#pragma unroll
                    for (int c = 0; c < 4; c++) ot[a][b][c] = 0.0f;
            const uint32_t Vh = Hb + 2 * V32_HTILE + (warp >> 1) * V32_HSUB;
            const uint32_t cb = (warp & 1u) * 4u, jm = lane >> 3;
            const uint32_t Pb = smem_base + V32_OFF_P;
#pragma unroll
            for (int ks = 0; ks < 2; ks++) { // 16 keys per step
                uint32_t pah[2][4], pal[2][4];
#pragma unroll
                for (int m2 = 0; m2 < 2; m2++) {
                    const uint32_t row = m2 * 16u + (lane & 7u) + 8u * ((lane >> 3) & 1u);
                    const uint32_t off = p32_off(row, 2u * ks + (lane >> 4));
                    ldmatrix_x4(pah[m2], Pb + off);
                    ldmatrix_x4(pal[m2], Pb + 32 * 64 + off);
                }
#pragma unroll
                for (int np = 0; np < 2; np++) { // two 8-dim tiles per load
                    uint32_t vh[4], vl[4];
                    const uint32_t key = 16u * ks + (lane & 7u) + 8u * (jm & 1u);
                    const uint32_t a = Vh + swz128(key, cb + 2u * np + (jm >> 1));
                    ldmatrix_x4_trans(vh, a);
                    ldmatrix_x4_trans(vl, a + V32_HTILE);
#pragma unroll
                    for (int m2 = 0; m2 < 2; m2++) {
                        mma_f16(ot[m2][2 * np], pah[m2], vh[0], vh[1]);
                        mma_f16(ot[m2][2 * np], pah[m2], vl[0], vl[1]);
                        mma_f16(ot[m2][2 * np], pal[m2], vh[0], vh[1]);
                        mma_f16(ot[m2][2 * np + 1], pah[m2], vh[2], vh[3]);
                        mma_f16(ot[m2][2 * np + 1], pah[m2], vl[2], vl[3]);
                        mma_f16(ot[m2][2 * np + 1], pal[m2], vh[2], vh[3]);
                    }
                }
            }
            const float c0 = cfs[g], c1 = cfs[g + 8], c2 = cfs[16 + g], c3 = cfs[24 + g];
#pragma unroll
            for (int n = 0; n < 4; n++) {
                o[0][n][0] = fmaf(o[0][n][0], c0, ot[0][n][0]); o[0][n][1] = fmaf(o[0][n][1], c0, ot[0][n][1]);
                o[0][n][2] = fmaf(o[0][n][2], c1, ot[0][n][2]); o[0][n][3] = fmaf(o[0][n][3], c1, ot[0][n][3]);
                o[1][n][0] = fmaf(o[1][n][0], c2, ot[1][n][0]); o[1][n][1] = fmaf(o[1][n][1], c2, ot[1][n][1]);
                o[1][n][2] = fmaf(o[1][n][2], c3, ot[1][n][2]); o[1][n][3] = fmaf(o[1][n][3], c3, ot[1][n][3]);
            }
        }
        // the next iteration's conversion overwrites the f16 tiles: its barrier comes after this P V in every warp
        __syncthreads();
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
        for (int m2 = 0; m2 < 2; m2++)
#pragma unroll
            for (int n = 0; n < 4; n++) {
                const uint32_t row = m2 * 16u + g, col = warp * 32u + n * 8u + 2u * qd;
                *reinterpret_cast<float2 *>(po + (size_t)row * 256u + col) = make_float2(o[m2][n][0], o[m2][n][1]);
                *reinterpret_cast<float2 *>(po + (size_t)(row + 8u) * 256u + col) = make_float2(o[m2][n][2], o[m2][n][3]);
            }
    }
    // the CTAs that finish last merge the pieces (scratch in the ring, which is drained by now)
    finish_item<256, EXT>(it, *reinterpret_cast<FinishSmem *>(smem), status);
}

mkv_status verify_f32_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)V32_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)V32_SMEM));
    return MKV_OK;
}

mkv_status launch_verify_f32(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas,
                             bool ext) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(total_ctas);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = V32_SMEM;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (ext) MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_kernel<true>, items_dev, n, single, ctx->dev_status));
    else MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_kernel<false>, items_dev, n, single, ctx->dev_status));
    ctx->launches++;
    return MKV_OK;
}

} // namespace mkv
