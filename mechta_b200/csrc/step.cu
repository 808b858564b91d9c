// The layer's step either side of the KV path, fused into the two launches of that path.
//
// The reference runs, per attention layer and step (M/quad.rs:113-125): rmsnorm of the query heads, rmsnorm of
// the key heads, rope2 of the queries, kv_rope2 + kv_copy into the cache, q_dmx, the attention, its combine and
// the output gate — nine dispatches. Here one small kernel does everything before the attention (this file) and
// the attention kernel's merge applies the gate (combine.cuh), so the layer takes two launches.
//
// Arithmetic (restated by the oracle's mko_rmsnorm / mko_rope2 / mko_append_k):
//   rmsnorm (W/ops.wgsl:27-56, flag 1, scale 1): the sum of squares of a 256-value row is folded in the shader's
//     order (one value per thread, then halving strides), scale = 1 / sqrt(sum / 256 + eps), y = x * scale * w[d],
//     every operation rounded to f32 on its own;
//   rope2 / kv_rope2 (W/ops.wgsl:275-286, W/kv.wgsl:19-23): dims 0..63 rotated by the token's table, products and
//     the sum/difference rounded separately;
//   K and V rows are converted to the cache format on the store (W/kv.wgsl:24-33).
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {

// One warp per row of 256 values (per token: 16 query heads, 2 key heads, 2 halves of the value row); lane t holds the
// values t, t + 32, ..., t + 224. The shader folds partial[t] += partial[t + m] for m = 128, 64, ..., 1: with this
// layout the strides 128, 64 and 32 are lane-local and 16 ... 1 are shuffles, in the same association, so the rows are
// bit-identical to the reference's. No shared memory and no block barrier: this kernel sits between two attention
// launches on the critical path of every layer.
constexpr int PREP_WARPS = 4;

template <bool F16>
__global__ void __launch_bounds__(32 * PREP_WARPS)
step_prep_kernel(const float *__restrict__ qf, const float *__restrict__ kb, const float *__restrict__ vb,
                 const float *__restrict__ q_norm, const float *__restrict__ k_norm, const float *__restrict__ tab, float eps,
                 float *__restrict__ qr, void *__restrict__ kcache, void *__restrict__ vcache, uint32_t row_first,
                 uint32_t capacity, uint32_t ring, uint32_t pos, uint32_t nrows) {
    // Programmatic dependent launch on both sides: the attention kernel behind this one may set itself up and load
    // the tiles below `pos` while this one runs; this one touches nothing before the kernel in front has finished
    // (its inputs may come from it, and the attention in front may still read the query scratch).
    ptx::pdl_launch_dependents();
    const uint32_t lane = threadIdx.x & 31u, idx = blockIdx.x * PREP_WARPS + (threadIdx.x >> 5);
    const uint32_t tok = idx / 20u, r = idx % 20u;
    if (idx < nrows && lane < 8u) { // the row's 1 KB (and the weights and the table) towards L2 while waiting
        const float *row = r < 16u ? qf + ((size_t)tok * 16u + r) * 512u
                         : r < 18u ? kb + ((size_t)tok * 2u + (r - 16u)) * 256u : vb + (size_t)tok * ROW + (r - 18u) * 256u;
        ptx::prefetch_l2(row + lane * 32u);
        if (r < 18u) ptx::prefetch_l2((r < 16u ? q_norm : k_norm) + lane * 32u);
        if (lane < 2u) ptx::prefetch_l2(tab + (size_t)tok * 64u + lane * 32u);
    }
    ptx::pdl_wait();
    if (idx >= nrows) return;
    const uint32_t gpos = pos + tok;
    const bool held = ring || (gpos >= row_first && gpos - row_first < capacity); // the row belongs to this shard
    const size_t crow = held ? (size_t)(ring ? gpos % ring : gpos - row_first) * ROW : 0;
    if (r >= 18u) { // V: convert and store (W/kv.wgsl:29-33)
        if (!held) return;
        const uint32_t e = (r - 18u) * 256u + lane;
        float x[8];
#pragma unroll
        for (int k = 0; k < 8; k++) x[k] = vb[(size_t)tok * ROW + e + 32u * k];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (F16) static_cast<__half *>(vcache)[crow + e + 32u * k] = __float2half_rn(x[k]);
            else static_cast<float *>(vcache)[crow + e + 32u * k] = x[k];
        }
        return;
    }
    const bool is_q = r < 16u;
    if (!is_q && !held) return;
    const float *src = is_q ? qf + ((size_t)tok * 16u + r) * 512u : kb + ((size_t)tok * 2u + (r - 16u)) * 256u;
    const float *w = is_q ? q_norm : k_norm;
    // every load goes out before the arithmetic
    float x[8], wt[8];
#pragma unroll
    for (int k = 0; k < 8; k++) x[k] = src[lane + 32u * k];
#pragma unroll
    for (int k = 0; k < 8; k++) wt[k] = w[lane + 32u * k];
    const float c = tab[(size_t)tok * 64u + lane], sn = tab[(size_t)tok * 64u + 32u + lane];
    float sq[8];
#pragma unroll
    for (int k = 0; k < 8; k++) sq[k] = __fmul_rn(x[k], x[k]);
#pragma unroll
    for (int k = 0; k < 4; k++) sq[k] = __fadd_rn(sq[k], sq[k + 4]); // W/ops.wgsl:37-40, m = 128
    sq[0] = __fadd_rn(sq[0], sq[2]);                                  // m = 64
    sq[1] = __fadd_rn(sq[1], sq[3]);
    float sum = __fadd_rn(sq[0], sq[1]);                              // m = 32
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) sum = __fadd_rn(sum, __shfl_down_sync(0xffffffffu, sum, m));
    sum = __shfl_sync(0xffffffffu, sum, 0);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, 256.0f), eps)));
    float y[8];
#pragma unroll
    for (int k = 0; k < 8; k++) y[k] = __fmul_rn(__fmul_rn(x[k], scale), wt[k]);
    // rope2 / kv_rope2: dims t < 32 (k = 0) pair with t + 32 (k = 1), both in this lane
    const float r0 = __fsub_rn(__fmul_rn(y[0], c), __fmul_rn(y[1], sn));
    const float r1 = __fadd_rn(__fmul_rn(y[0], sn), __fmul_rn(y[1], c));
    y[0] = r0;
    y[1] = r1;
    if (is_q) {
        float *dst = qr + ((size_t)tok * 16u + r) * 256u;
#pragma unroll
        for (int k = 0; k < 8; k++) dst[lane + 32u * k] = y[k];
    } else {
        const uint32_t e = (r - 16u) * 256u + lane;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            if (F16) static_cast<__half *>(kcache)[crow + e + 32u * k] = __float2half_rn(y[k]);
            else static_cast<float *>(kcache)[crow + e + 32u * k] = y[k];
        }
    }
}

mkv_status launch_step_prep(Ctx *ctx, mkv_fmt fmt, const float *qf, const float *kb, const float *vb, const float *q_norm,
                            const float *k_norm, const float *tab, float eps, float *qr, void *kcache, void *vcache,
                            uint32_t row_first, uint32_t capacity, uint32_t ring, uint32_t pos, uint32_t ntok) {
    cudaLaunchConfig_t cfg = {};
    const uint32_t nrows = 20u * ntok;
    cfg.gridDim = dim3((nrows + PREP_WARPS - 1) / PREP_WARPS);
    cfg.blockDim = dim3(32 * PREP_WARPS);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (fmt == MKV_F16)
        MKV_CUDA(cudaLaunchKernelEx(&cfg, step_prep_kernel<true>, qf, kb, vb, q_norm, k_norm, tab, eps, qr, kcache, vcache, row_first,
                                    capacity, ring, pos, nrows));
    else
        MKV_CUDA(cudaLaunchKernelEx(&cfg, step_prep_kernel<false>, qf, kb, vb, q_norm, k_norm, tab, eps, qr, kcache, vcache, row_first,
                                    capacity, ring, pos, nrows));
    ctx->launches++;
    return MKV_OK;
}

} // namespace mkv
