// K/V append for the verify step and for prefill blocks: RoPE on dims 0..63 of K, conversion to the cache
// format, 16-byte coalesced stores. One launch covers K and V of `n_layers` layers.
//
// Arithmetic contract (follows W/kv.wgsl:13-17 kv_src and W/ops.wgsl:278-285 rope2 of the reference):
//   d < 32:        a[d] * cos[d] - a[d+32] * sin[d]
//   32 <= d < 64:  a[d-32] * sin[d-32] + a[d] * cos[d-32]
//   d >= 64:       a[d]
// with each product and the sum/difference rounded to f32 on its own (no FMA contraction), then
// round-to-nearest-even to f16 for the f16 cache. V is converted and stored (W/kv.wgsl:29-33).
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {

template <bool F16>
__global__ void __launch_bounds__(256)
append_kernel(void *const *__restrict__ kbufs, void *const *__restrict__ vbufs, int n_layers, size_t layer_stride,
              uint32_t row_first, uint32_t capacity, uint32_t ring, uint32_t pos, uint32_t ntok,
              const float *__restrict__ k, const float *__restrict__ v, const float *__restrict__ tab, uint32_t which) {
    // Programmatic dependent launch on both sides: the attention kernel behind this one may set itself up and load
    // tiles below `pos` meanwhile; this kernel touches nothing before the kernel in front has finished (its inputs
    // may come from it, and the rows it overwrites after a rollback may still be read by the attention in front).
    ptx::pdl_launch_dependents();
    // one thread = 8 consecutive elements; per (layer, token): 64 groups of K then 64 groups of V
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n_layers * ntok * 128u;
    const bool in_range = gid < total;
    const uint32_t g = (uint32_t)(gid & 63u);
    const uint32_t is_v = (uint32_t)((gid >> 6) & 1u);
    const uint32_t tok = in_range ? (uint32_t)((gid >> 7) % ntok) : 0u;
    const uint32_t layer = in_range ? (uint32_t)((gid >> 7) / ntok) : 0u;
    const uint32_t e0 = g * 8u; // element inside the position: kvh * 256 + d
    const float *src = (is_v ? v : k) + layer * layer_stride + (size_t)tok * ROW;
    if (in_range && (g & 3u) == 0u && (which & (is_v ? 2u : 1u))) ptx::prefetch_l2(src + e0); // the new rows towards L2 while waiting (one line per four threads)
    ptx::pdl_wait();
    if (!in_range) return;
    if (!(which & (is_v ? 2u : 1u))) return; // bit 0: write K, bit 1: write V
    const uint32_t gpos = pos + tok;
    if (!ring && (gpos < row_first || gpos - row_first >= capacity)) return; // row belongs to another shard
    const size_t row = ring ? gpos % ring : gpos - row_first; // ring cache: row = position % ring (W/flint_attn.wgsl:3)
    float x[8];
    {
        const float4 a0 = *reinterpret_cast<const float4 *>(src + e0);
        const float4 a1 = *reinterpret_cast<const float4 *>(src + e0 + 4);
        x[0] = a0.x; x[1] = a0.y; x[2] = a0.z; x[3] = a0.w;
        x[4] = a1.x; x[5] = a1.y; x[6] = a1.z; x[7] = a1.w;
    }
    const uint32_t d0 = e0 & 255u;
    if (!is_v && tab != nullptr && d0 < 64u) {
        const float *tb = tab + (size_t)tok * 64u;
        const uint32_t i0 = d0 & 31u; // index of the pair (i, i + 32)
        const bool low = d0 < 32u;
        const float *other = src + (e0 & ~255u) + (low ? i0 + 32u : i0);
        float y[8], c[8], s[8];
        {
            const float4 b0 = *reinterpret_cast<const float4 *>(other);
            const float4 b1 = *reinterpret_cast<const float4 *>(other + 4);
            y[0] = b0.x; y[1] = b0.y; y[2] = b0.z; y[3] = b0.w;
            y[4] = b1.x; y[5] = b1.y; y[6] = b1.z; y[7] = b1.w;
            const float4 c0 = *reinterpret_cast<const float4 *>(tb + i0);
            const float4 c1 = *reinterpret_cast<const float4 *>(tb + i0 + 4);
            c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w;
            c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
            const float4 s0 = *reinterpret_cast<const float4 *>(tb + 32u + i0);
            const float4 s1 = *reinterpret_cast<const float4 *>(tb + 32u + i0 + 4);
            s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w;
            s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
        }
#pragma unroll
        for (int j = 0; j < 8; j++) {
            if (low) x[j] = __fsub_rn(__fmul_rn(x[j], c[j]), __fmul_rn(y[j], s[j]));
            else x[j] = __fadd_rn(__fmul_rn(y[j], s[j]), __fmul_rn(x[j], c[j]));
        }
    }
    void *dst_buf = is_v ? vbufs[layer] : kbufs[layer];
    const size_t eo = row * ROW + e0;
    if (F16) {
        uint4 w;
        __half2 h0 = __halves2half2(__float2half_rn(x[0]), __float2half_rn(x[1]));
        __half2 h1 = __halves2half2(__float2half_rn(x[2]), __float2half_rn(x[3]));
        __half2 h2 = __halves2half2(__float2half_rn(x[4]), __float2half_rn(x[5]));
        __half2 h3 = __halves2half2(__float2half_rn(x[6]), __float2half_rn(x[7]));
        w.x = *reinterpret_cast<uint32_t *>(&h0);
        w.y = *reinterpret_cast<uint32_t *>(&h1);
        w.z = *reinterpret_cast<uint32_t *>(&h2);
        w.w = *reinterpret_cast<uint32_t *>(&h3);
        *reinterpret_cast<uint4 *>(static_cast<__half *>(dst_buf) + eo) = w;
    } else {
        float4 *o = reinterpret_cast<float4 *>(static_cast<float *>(dst_buf) + eo);
        o[0] = make_float4(x[0], x[1], x[2], x[3]);
        o[1] = make_float4(x[4], x[5], x[6], x[7]);
    }
}

// q_f16 of the reference (W/fa_mx.wgsl:313-319): the block's rotated queries f32 -> f16, two values per 32-bit word,
// round to nearest even. One thread = 8 values (two 16-byte loads, one 16-byte store).
__global__ void __launch_bounds__(256) q_f16_kernel(const float *__restrict__ src, __half *__restrict__ dst, size_t n8) {
    ptx::pdl_launch_dependents();
    ptx::pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const float4 a = reinterpret_cast<const float4 *>(src)[2 * i], b = reinterpret_cast<const float4 *>(src)[2 * i + 1];
    const __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
    const __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
    reinterpret_cast<uint4 *>(dst)[i] = make_uint4(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1),
                                                   *reinterpret_cast<const uint32_t *>(&h2), *reinterpret_cast<const uint32_t *>(&h3));
}

mkv_status launch_q_f16(Ctx *ctx, const float *src, void *dst, size_t n_pairs) {
    const size_t n8 = n_pairs / 4; // 8 values = 4 packed words per thread
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((n8 + 255u) / 256u));
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    MKV_CUDA(cudaLaunchKernelEx(&cfg, q_f16_kernel, src, static_cast<__half *>(dst), n8));
    ctx->launches++;
    return MKV_OK;
}

mkv_status append_setup_device() {
    MKV_CUDA(cudaFuncSetAttribute(append_kernel<true>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    MKV_CUDA(cudaFuncSetAttribute(append_kernel<false>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
    return MKV_OK;
}

mkv_status launch_append(Ctx *ctx, mkv_fmt fmt, void *const *kbufs, void *const *vbufs, int n_layers,
                         size_t layer_stride_in, uint32_t row_first, uint32_t capacity, uint32_t ring, uint32_t pos,
                         uint32_t ntok, const float *k, const float *v, const float *tab, uint32_t which) {
    const size_t total = (size_t)n_layers * ntok * 128u;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((total + 255u) / 256u));
    cfg.blockDim = dim3(256);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (fmt == MKV_F16)
        MKV_CUDA(cudaLaunchKernelEx(&cfg, append_kernel<true>, kbufs, vbufs, n_layers, layer_stride_in, row_first, capacity, ring, pos,
                                    ntok, k, v, tab, which));
    else
        MKV_CUDA(cudaLaunchKernelEx(&cfg, append_kernel<false>, kbufs, vbufs, n_layers, layer_stride_in, row_first, capacity, ring, pos,
                                    ntok, k, v, tab, which));
    ctx->launches++;
    return MKV_OK;
}

} // namespace mkv
