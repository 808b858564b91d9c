// Prefill attention over the f16 cache, warp-MMA version: flash attention for a block of tokens that reads
// the prefix already in the cache plus the block's own rows (appended before, as the reference does,
// M/engine.rs:1213-1214).
//
// Stands in for q_f16 + attn_fa_mx + attn_fd_combine (W/fa_mx.wgsl:19-115,313-319; M/engine.rs:1215-1226):
// token T of the block (at pos0 + T) sees first_pos <= key < pos0 + 1 + T. A CTA takes 16 tokens x the 8 query
// heads of one KV head = 128 rows (the reference packs 16 tokens x 4 heads, W/fa_mx.wgsl:3-4), warp w = head w,
// so every K/V tile staged by TMA feeds all 8 heads. No split over keys: the online softmax runs over the whole
// visible range and the output is final (the reference's chunk partials + merge exist only to bound its
// dispatch time).
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {
using namespace ptx;

constexpr int PF_NST = 2;
constexpr uint32_t PF_STAGE = 65536;
constexpr uint32_t PF_SUB = 8192;
constexpr uint32_t PF_OFF_Q = PF_NST * PF_STAGE;       // 128 rows x 512 B
constexpr uint32_t PF_OFF_BAR = PF_OFF_Q + 128 * 512;
constexpr uint32_t PF_SMEM = PF_OFF_BAR + PF_NST * 8 + 1024;
constexpr long long PF_WAIT_LIMIT = 4000000000ll;

__global__ void __launch_bounds__(256, 1)
prefill_f16_mma_kernel(const CUtensorMap *__restrict__ kmap, const CUtensorMap *__restrict__ vmap,
                       const float *__restrict__ q, float *__restrict__ out, uint32_t first_pos, uint32_t pos0,
                       uint32_t ntok, uint32_t row0, uint32_t *__restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t ngrp = gridDim.x;
    const uint32_t grp = ngrp - 1u - blockIdx.x; // longest key ranges first
    const uint32_t kvh = blockIdx.y;
    const uint32_t tok0 = grp * 16u;
    const uint32_t last_tok = min(tok0 + 15u, ntok - 1u);
    const uint32_t lim = pos0 + 1u + last_tok; // keys seen by the group: [first_pos, lim)
    const uint32_t t0 = first_pos / PF_TILE, t1 = (lim + PF_TILE - 1u) / PF_TILE;
    const uint32_t nt = t1 - t0;
    const uint32_t bar0 = smem_base + PF_OFF_BAR;

    if (tid == 0) {
        for (int s = 0; s < PF_NST; s++) mbar_init(bar0 + 8u * s, 1);
        fence_barrier_init();
        fence_proxy_async();
    }
    __syncthreads();
    auto issue = [&](uint32_t j) {
        const uint32_t s = j % PF_NST, bar = bar0 + 8u * s;
        const uint32_t dst = smem_base + s * PF_STAGE;
        const int y = (int)((t0 + j) * PF_TILE - row0);
        const int x = (int)(kvh * 256u);
        mbar_expect_tx(bar, PF_STAGE);
#pragma unroll
        for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + sb * PF_SUB, kmap, x + 64 * sb, y, bar);
#pragma unroll
        for (int sb = 0; sb < 4; sb++) tma_load_2d(dst + 4 * PF_SUB + sb * PF_SUB, vmap, x + 64 * sb, y, bar);
    };
    if (tid == 0) {
        const uint32_t pre = nt < (uint32_t)PF_NST ? nt : (uint32_t)PF_NST;
        for (uint32_t j = 0; j < pre; j++) issue(j);
    }

    // Q to shared memory as f16 (q_f16 of the reference): row = head % 8 * 16 + token of the group
    {
        uint8_t *qs = smem + PF_OFF_Q;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const uint32_t idx = tid + 256u * i; // 128 rows x 32 chunks
            const uint32_t row = idx >> 5, chunk = idx & 31u;
            const uint32_t tok = tok0 + (row & 15u), head = 8u * kvh + (row >> 4);
            uint4 w = make_uint4(0, 0, 0, 0);
            if (tok < ntok) {
                const float *src = q + (size_t)tok * 4096u + (size_t)head * 256u + chunk * 8u;
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

    float o[32][4];
#pragma unroll
    for (int n = 0; n < 32; n++)
#pragma unroll
        for (int c = 0; c < 4; c++) o[n][c] = 0.0f;
    float m_run[2] = {NEG_BIG, NEG_BIG}, l_run[2] = {0.0f, 0.0f};
    const uint32_t g = lane >> 2, qd = lane & 3u;
    // this thread's two rows are tokens tok0 + g and tok0 + g + 8 of head `warp`
    const uint32_t vis0 = pos0 + 1u + tok0 + g, vis1 = vis0 + 8u;
    const uint32_t full_below = pos0 + 1u + tok0; // keys below this are visible to every row of the group
    const uint32_t qs = smem_base + PF_OFF_Q + warp * 16u * 512u;
    bool aborted = false;

    for (uint32_t j = 0; j < nt; j++) {
        const uint32_t s = j % PF_NST;
        if (!aborted && !mbar_wait_bounded(bar0 + 8u * s, (j / PF_NST) & 1u, PF_WAIT_LIMIT)) {
            aborted = true;
            atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        }
        const uint32_t Kb = smem_base + s * PF_STAGE, Vb = Kb + 4 * PF_SUB;
        const uint32_t key_base = (t0 + j) * PF_TILE;

        // ---- S (16 x 64) = Q K^T ----
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++)
#pragma unroll
            for (int c = 0; c < 4; c++) sc[n][c] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 16; ks++) {
            uint32_t a[4];
            {
                const uint32_t row = (lane & 7u) + 8u * ((lane >> 3) & 1u);
                const uint32_t chunk = 2u * ks + (lane >> 4);
                const uint32_t pc = (chunk & ~7u) | ((chunk ^ row) & 7u);
                ldmatrix_x4(a, qs + row * 512u + pc * 16u);
            }
#pragma unroll
            for (int np = 0; np < 4; np++) { // 16 keys per load
                uint32_t kb[4];
                const uint32_t key = 16u * np + (lane & 7u) + 8u * (lane >> 4);
                const uint32_t chunk = 2u * (ks & 3) + ((lane >> 3) & 1u);
                ldmatrix_x4(kb, Kb + (ks >> 2) * PF_SUB + swz128(key, chunk));
                mma_f16(sc[2 * np], a, kb[0], kb[1]);
                mma_f16(sc[2 * np + 1], a, kb[2], kb[3]);
            }
        }

        // ---- scale, mask, online softmax in registers ----
        const bool need_mask = key_base + PF_TILE > full_below || key_base < first_pos;
        float mx[2] = {NEG_BIG, NEG_BIG};
#pragma unroll
        for (int n = 0; n < 8; n++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float v = sc[n][c] * SCALE;
                if (need_mask) {
                    const uint32_t key = key_base + n * 8u + 2u * qd + (c & 1);
                    const uint32_t vis = (c >> 1) ? vis1 : vis0;
                    if (!(key >= first_pos && key < vis)) v = NEG_BIG;
                }
                sc[n][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        float cf[2];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            cf[r] = m_run[r] > NEG_TEST ? __expf(m_run[r] - m_new) : 0.0f;
            m_run[r] = m_new;
            l_run[r] *= cf[r];
        }
        uint32_t pa[4][4]; // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int n = 0; n < 8; n++) {
            const float w0 = sc[n][0] > NEG_TEST ? __expf(sc[n][0] - m_run[0]) : 0.0f;
            const float w1 = sc[n][1] > NEG_TEST ? __expf(sc[n][1] - m_run[0]) : 0.0f;
            const float w2 = sc[n][2] > NEG_TEST ? __expf(sc[n][2] - m_run[1]) : 0.0f;
            const float w3 = sc[n][3] > NEG_TEST ? __expf(sc[n][3] - m_run[1]) : 0.0f;
            const __half2 h01 = __floats2half2_rn(w0, w1), h23 = __floats2half2_rn(w2, w3);
            const float2 f01 = __half22float2(h01), f23 = __half22float2(h23);
            l_run[0] += f01.x + f01.y;
            l_run[1] += f23.x + f23.y;
            pa[n >> 1][(n & 1) * 2 + 0] = *reinterpret_cast<const uint32_t *>(&h01);
            pa[n >> 1][(n & 1) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&h23);
        }
#pragma unroll
        for (int n = 0; n < 32; n++) {
            o[n][0] *= cf[0]; o[n][1] *= cf[0]; o[n][2] *= cf[1]; o[n][3] *= cf[1];
        }

        // ---- O += P V ----
#pragma unroll
        for (int ks = 0; ks < 4; ks++) {
#pragma unroll
            for (int dn = 0; dn < 16; dn++) { // 16 dims per load
                uint32_t vb[4];
                const uint32_t jm = lane >> 3;
                const uint32_t key = 16u * ks + (lane & 7u) + 8u * (jm & 1u);
                const uint32_t chunk = 2u * (dn & 3) + (jm >> 1);
                ldmatrix_x4_trans(vb, Vb + (dn >> 2) * PF_SUB + swz128(key, chunk));
                mma_f16(o[2 * dn], pa[ks], vb[0], vb[1]);
                mma_f16(o[2 * dn + 1], pa[ks], vb[2], vb[3]);
            }
        }
        __syncthreads(); // every warp is done with stage s
        if (tid == 0 && j + PF_NST < nt) issue(j + PF_NST);
    }

    // ---- normalise and store: out[tok][head][d] ----
#pragma unroll
    for (int r = 0; r < 2; r++) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const uint32_t head = 8u * kvh + warp;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint32_t tok = tok0 + g + 8u * r;
        if (tok < ntok) {
            const float inv = 1.0f / l_run[r];
            float *dst = out + (size_t)tok * 4096u + (size_t)head * 256u + 2u * qd;
#pragma unroll
            for (int n = 0; n < 32; n++)
                *reinterpret_cast<float2 *>(dst + n * 8) = make_float2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
        }
    }
}

mkv_status prefill_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(prefill_f16_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM));
    MKV_CUDA(cudaFuncSetAttribute(prefill_f16_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    return MKV_OK;
}

mkv_status launch_prefill_f16_mma(Ctx *ctx, Cache *c, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                                  const float *q, float *out) {
    const dim3 grid((ntok + 15u) / 16u, 2);
    prefill_f16_mma_kernel<<<grid, 256, PF_SMEM, ctx->stream>>>(c->maps_dev + 2 * (c->n_layers + layer), c->maps_dev + 2 * (c->n_layers + layer) + 1, q, out,
                                                                first_pos, pos0, ntok, c->shard_first, ctx->dev_status);
    ctx->launches++;
    MKV_CUDA(cudaGetLastError());
    return MKV_OK;
}

} // namespace mkv
