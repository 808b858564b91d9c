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

// One block per row of 256 values: per token 16 query heads, 2 key heads, 2 halves of the value row.
template <bool F16>
__global__ void __launch_bounds__(256)
step_prep_kernel(const float *__restrict__ qf, const float *__restrict__ kb, const float *__restrict__ vb,
                 const float *__restrict__ q_norm, const float *__restrict__ k_norm, const float *__restrict__ tab, float eps,
                 float *__restrict__ qr, void *__restrict__ kcache, void *__restrict__ vcache, uint32_t row_first,
                 uint32_t capacity, uint32_t ring, uint32_t pos) {
    __shared__ float partial[256];
    __shared__ float row[256];
    // Programmatic dependent launch on both sides: the attention kernel behind this one may set itself up and load
    // the tiles below `pos` while this one runs; this one touches nothing before the kernel in front has finished
    // (its inputs may come from it, and the attention in front may still read the query scratch).
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const uint32_t t = threadIdx.x, tok = blockIdx.x / 20u, r = blockIdx.x % 20u;
    const uint32_t gpos = pos + tok;
    const bool held = ring || (gpos >= row_first && gpos - row_first < capacity); // the row belongs to this shard
    const size_t crow = held ? (size_t)(ring ? gpos % ring : gpos - row_first) * ROW : 0;
    if (r >= 18u) { // V: convert and store (W/kv.wgsl:29-33)
        if (!held) return;
        const uint32_t e = (r - 18u) * 256u + t;
        const float x = vb[(size_t)tok * ROW + e];
        if (F16) static_cast<__half *>(vcache)[crow + e] = __float2half_rn(x);
        else static_cast<float *>(vcache)[crow + e] = x;
        return;
    }
    const bool is_q = r < 16u;
    if (!is_q && !held) return;
    const float *src = is_q ? qf + ((size_t)tok * 16u + r) * 512u : kb + ((size_t)tok * 2u + (r - 16u)) * 256u;
    const float *w = is_q ? q_norm : k_norm;
    const float x = src[t];
    partial[t] = __fmul_rn(x, x);
    __syncthreads();
#pragma unroll
    for (uint32_t m = 128u; m > 0u; m >>= 1) { // W/ops.wgsl:37-40
        if (t < m) partial[t] = __fadd_rn(partial[t], partial[t + m]);
        __syncthreads();
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(partial[0], 256.0f), eps)));
    row[t] = __fmul_rn(__fmul_rn(x, scale), w[t]);
    __syncthreads();
    float y = row[t];
    if (t < 64u) {
        const float *tb = tab + (size_t)tok * 64u;
        if (t < 32u) y = __fsub_rn(__fmul_rn(row[t], tb[t]), __fmul_rn(row[t + 32u], tb[32u + t]));
        else y = __fadd_rn(__fmul_rn(row[t - 32u], tb[t]), __fmul_rn(row[t], tb[t - 32u]));
    }
    if (is_q) {
        qr[((size_t)tok * 16u + r) * 256u + t] = y;
    } else {
        const uint32_t e = (r - 16u) * 256u + t;
        if (F16) static_cast<__half *>(kcache)[crow + e] = __float2half_rn(y);
        else static_cast<float *>(kcache)[crow + e] = y;
    }
}

mkv_status launch_step_prep(Ctx *ctx, mkv_fmt fmt, const float *qf, const float *kb, const float *vb, const float *q_norm,
                            const float *k_norm, const float *tab, float eps, float *qr, void *kcache, void *vcache,
                            uint32_t row_first, uint32_t capacity, uint32_t ring, uint32_t pos, uint32_t ntok) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(20u * ntok);
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (fmt == MKV_F16)
        MKV_CUDA(cudaLaunchKernelEx(&cfg, step_prep_kernel<true>, qf, kb, vb, q_norm, k_norm, tab, eps, qr, kcache, vcache, row_first,
                                    capacity, ring, pos));
    else
        MKV_CUDA(cudaLaunchKernelEx(&cfg, step_prep_kernel<false>, qf, kb, vb, q_norm, k_norm, tab, eps, qr, kcache, vcache, row_first,
                                    capacity, ring, pos));
    ctx->launches++;
    return MKV_OK;
}

} // namespace mkv
