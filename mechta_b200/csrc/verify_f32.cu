// Decode / verify attention over the f32 cache (and the MTP window, which the reference also runs through
// its f32-math kernels): split-K flash-decode in scalar f32, same pieces and combine as the f16 path.
//
// Stands in for attn_fd / attn_fd2h (W/ops.wgsl:325-516). The arithmetic is theirs (f32 products and sums,
// block max, exp(v - max), un-normalised accumulators); the tolerance of 1e-5 rules out tf32/f16 tensor
// cores without operand splitting, so this path is bound by the FP32 FMA pipe rather than by HBM:
// 32 rows x 256 dims x 2 (QK and PV) = 16 FMA per byte of f32 cache.
//  - K and V tiles of 32 keys arrive by TMA (128-byte swizzle, no multicast) into a 2-deep ring;
//  - scores: thread = (key, group of 4 rows); the K row chunk is one 16-byte shared load, Q chunks are
//    broadcast loads, 16 FMA per 5 loads;
//  - P V: thread = (4 dims, group of 8 rows); one 16-byte V load and two broadcast P loads per 32 FMA.
#include "combine.cuh"
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int V32_NST = 2;
constexpr uint32_t V32_STAGE = 65536; // K 32 KB + V 32 KB
constexpr uint32_t V32_SUB = 4096;    // one [32 keys][32 dims] f32 sub-box
constexpr uint32_t V32_OFF_Q = V32_NST * V32_STAGE;
constexpr uint32_t V32_OFF_S = V32_OFF_Q + 32 * 1024;
constexpr uint32_t V32_S_STRIDE = 36; // floats per key row of S/P ([key][row], 32 + 4 of padding)
constexpr uint32_t V32_OFF_CF = V32_OFF_S + 32 * V32_S_STRIDE * 4;
constexpr uint32_t V32_OFF_BAR = V32_OFF_CF + 32 * 4;
constexpr uint32_t V32_SMEM = V32_OFF_BAR + V32_NST * 8 + 1024;
constexpr long long WAIT_LIMIT32 = 4000000000ll;

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
    const uint32_t nrow = 8u * it.ntok;

    if (tid == 0) {
        for (int s = 0; s < V32_NST; s++) mbar_init(bar0 + 8u * s, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();

    auto issue = [&](uint32_t j) {
        const uint32_t s = j % V32_NST, bar = bar0 + 8u * s;
        const uint32_t dst = smem_base + s * V32_STAGE;
        const int y = (int)((t0 + j) * TILE32 - it.row0);
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

    // Q rows of this KV head: [row = tok * 8 + head % 8][256] f32, rows of tokens >= ntok zero
    float *Q = reinterpret_cast<float *>(smem + V32_OFF_Q);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t idx = tid + 256u * i; // 32 rows x 64 float4
        const uint32_t row = idx >> 6, c = idx & 63u;
        float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < nrow)
            w = *reinterpret_cast<const float4 *>(it.q + (size_t)(row >> 3) * 4096u + (size_t)(8u * kvh + (row & 7u)) * 256u + c * 4u);
        *reinterpret_cast<float4 *>(Q + row * 256u + c * 4u) = w;
    }
    __syncthreads();

    float acc[8][4];
#pragma unroll
    for (int r = 0; r < 8; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = 0.0f;

    float *S = reinterpret_cast<float *>(smem + V32_OFF_S);
    float *cfs = reinterpret_cast<float *>(smem + V32_OFF_CF);
    const uint32_t srow = tid >> 3, seg = tid & 7u; // softmax: 8 threads per row, 4 keys each
    const uint32_t vis = min(it.pos + 1u + (srow >> 3), it.key_hi);
    const uint32_t klo = max(it.first_pos, it.key_lo);
    float m_run = NEG_BIG, l_run = 0.0f;
    const uint32_t dg = tid & 63u, rq = tid >> 6; // P V: dims 4 dg.., rows 8 rq..
    bool aborted = false;

    for (uint32_t j = 0; j < nt; j++) {
        const uint32_t s = j % V32_NST;
        if (!aborted && !mbar_wait_bounded(bar0 + 8u * s, (j / V32_NST) & 1u, WAIT_LIMIT32)) {
            aborted = true;
            atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        }
        const uint8_t *Kt = smem + s * V32_STAGE, *Vt = Kt + 8 * V32_SUB;

        // ---- scores of key `lane` against rows 4 warp .. 4 warp + 3 ----
        if (4u * warp < nrow) {
            // 16 independent accumulators (4 rows x 4 lanes of the 16-byte chunk): no FMA waits on the one before
            float d[4][4];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) d[r][c] = 0.f;
            const float *q0 = Q + (4u * warp) * 256u;
#pragma unroll 8
            for (uint32_t c = 0; c < 64u; c++) {
                const float4 k4 = *reinterpret_cast<const float4 *>(Kt + (c >> 3) * V32_SUB + swz128(lane, c & 7u));
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const float4 a = *reinterpret_cast<const float4 *>(q0 + r * 256u + c * 4u);
                    d[r][0] = fmaf(a.x, k4.x, d[r][0]);
                    d[r][1] = fmaf(a.y, k4.y, d[r][1]);
                    d[r][2] = fmaf(a.z, k4.z, d[r][2]);
                    d[r][3] = fmaf(a.w, k4.w, d[r][3]);
                }
            }
            *reinterpret_cast<float4 *>(S + lane * V32_S_STRIDE + 4u * warp) =
                make_float4((d[0][0] + d[0][1]) + (d[0][2] + d[0][3]), (d[1][0] + d[1][1]) + (d[1][2] + d[1][3]),
                            (d[2][0] + d[2][1]) + (d[2][2] + d[2][3]), (d[3][0] + d[3][1]) + (d[3][2] + d[3][3]));
        }
        __syncthreads(); // scores complete; every warp is past the P V of the previous tile

        if (tid == 0 && j >= 1 && j - 1 + V32_NST < nt) issue(j - 1 + V32_NST);

        // ---- softmax of row srow over this tile's 32 keys ----
        if (srow < nrow) {
            float v[4];
            const uint32_t key0 = (t0 + j) * TILE32 + seg * 4u;
            float mt_ = NEG_BIG;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t key = key0 + c;
                const float x = S[(seg * 4u + c) * V32_S_STRIDE + srow];
                v[c] = (key >= klo && key < vis) ? x * SCALE : NEG_BIG;
                mt_ = fmaxf(mt_, v[c]);
            }
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 1));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 2));
            mt_ = fmaxf(mt_, __shfl_xor_sync(0xffffffffu, mt_, 4));
            const float m_new = fmaxf(m_run, mt_);
            float sum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float w = v[c] > NEG_TEST ? expf(v[c] - m_new) : 0.0f;
                S[(seg * 4u + c) * V32_S_STRIDE + srow] = w;
                sum += w;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            const float cf = m_run > NEG_TEST ? expf(m_run - m_new) : 0.0f;
            l_run = l_run * cf + sum;
            m_run = m_new;
            if (seg == 0) cfs[srow] = cf;
        }
        __syncthreads();

        // ---- O = O * cf + P V for dims 4 dg .. 4 dg + 3, rows 8 rq .. 8 rq + 7 ----
        if (8u * rq < nrow) {
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const float cf = cfs[8u * rq + r];
                acc[r][0] *= cf; acc[r][1] *= cf; acc[r][2] *= cf; acc[r][3] *= cf;
            }
            const uint8_t *vcol = Vt + (dg >> 3) * V32_SUB;
#pragma unroll 4
            for (uint32_t key = 0; key < 32u; key++) {
                const float4 v4 = *reinterpret_cast<const float4 *>(vcol + swz128(key, dg & 7u));
                const float4 pa = *reinterpret_cast<const float4 *>(S + key * V32_S_STRIDE + 8u * rq);
                const float4 pb = *reinterpret_cast<const float4 *>(S + key * V32_S_STRIDE + 8u * rq + 4u);
                const float p[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    acc[r][0] = fmaf(p[r], v4.x, acc[r][0]);
                    acc[r][1] = fmaf(p[r], v4.y, acc[r][1]);
                    acc[r][2] = fmaf(p[r], v4.z, acc[r][2]);
                    acc[r][3] = fmaf(p[r], v4.w, acc[r][3]);
                }
            }
        }
    }

    const size_t piece = (size_t)kvh * it.nsplit + split;
    if (seg == 0) {
        float2 *ml = reinterpret_cast<float2 *>(it.part_ml) + piece * 32u + srow;
        *ml = make_float2(m_run, l_run);
    }
    {
        float *po = it.part_o + piece * 32u * 256u;
#pragma unroll
        for (int r = 0; r < 8; r++)
            *reinterpret_cast<float4 *>(po + (size_t)(8u * rq + r) * 256u + 4u * dg) =
                make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
    }
    // the CTAs that finish last merge the pieces (scratch in the ring, which is drained by now)
    finish_item<256>(it, *reinterpret_cast<FinishSmem *>(smem), status);
}

mkv_status verify_f32_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)V32_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(verify_f32_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    return MKV_OK;
}

mkv_status launch_verify_f32(Ctx *ctx, const VerifyItem *items_dev, int n, const VerifyLaunch &single, uint32_t total_ctas) {
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
    MKV_CUDA(cudaLaunchKernelEx(&cfg, verify_f32_kernel, items_dev, n, single, ctx->dev_status));
    ctx->launches++;
    return MKV_OK;
}

} // namespace mkv
