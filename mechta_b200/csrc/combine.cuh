// Log-sum-exp merge of split-K pieces, done inside the attention kernels by the CTAs that finish last.
//
// Arithmetic: attn_fd_combine of the reference (W/ops.wgsl:529-537) over this library's pieces:
//   M = max_s m_s;  tot = sum_s e^(m_s - M) l_s;  acc[d] = sum_s e^(m_s - M) O_s[d];  out = acc / tot.
// Scheduling: every CTA publishes its piece, then takes a ticket from a counter in global memory. The last
// R = min(CTAs of the item, 64) arrivals wait (bounded) until the counter shows that all pieces are there and
// each merges a share of the item's 64 rows. Only CTAs that have already finished their own work ever wait,
// and fewer of them than there are SMs, so the others always make progress.
#pragma once
#include "internal.cuh"
#include "ptx.cuh"

namespace mkv {

// The item a CTA of a verify launch belongs to: the single item in the parameter space, or the staged item
// whose CTA range contains this CTA.
__device__ __forceinline__ const VerifyItem &pick_item(const VerifyItem *items, int n_items, const VerifyItem &single,
                                                       uint32_t cta) {
    if (items == nullptr) return single;
    int lo = 0;
    for (int i = 1; i < n_items; i++)
        if (cta >= items[i].cta_begin) lo = i;
    return items[lo];
}

constexpr int FIN_MAX_THREADS = 512;

struct FinishSmem {
    float e_s[MAX_SPLITS];
    float red[FIN_MAX_THREADS / 32];
    float tot, M;
    uint32_t ticket, ok;
#ifdef MKV_TRACE
    unsigned long long tr[3]; // ticket taken, all pieces seen, rows merged
    unsigned long long tm[4]; // inside the merge of a row: loads issued, maximum known, pieces summed, row written
#endif
    float4 part[FIN_MAX_THREADS / 64][64];
};

// One row (kvh * 32 + row) of one item, by all NT threads of the CTA.
// EXT = false compiles the sink handling out (the kernels of the plain path are instantiated without it).
template <int NT, bool EXT = true>
__device__ __forceinline__ void merge_row(const VerifyItem &it, uint32_t r, FinishSmem &sm) {
    constexpr int GROUPS = NT / 64;
    constexpr int NW = NT / 32;
    const uint32_t kvh = r >> 5, row = r & 31u, tok = row >> 3, head = 8u * kvh + (row & 7u);
    const uint32_t tid = threadIdx.x;
    const uint32_t ndst = it.push ? it.push->world : 1u; // records go to `out`, or to every rank's mailbox
    if (tok >= it.ntok) {
        if (it.partial && tid < 258u) // rows of tokens beyond the step: the empty record
            for (uint32_t dd = 0; dd < ndst; dd++) {
                float *base = it.push ? it.push->slot[it.push_epoch & 1u][dd] : it.out;
                if (base) base[(size_t)(tok * 16u + head) * REC + tid] = tid == 0 ? NEG_BIG : 0.0f;
            }
        return;
    }
    const uint32_t ns = it.nsplit;
    const float2 *ml = reinterpret_cast<const float2 *>(it.part_ml) + (size_t)kvh * ns * 32u + row;
    const uint32_t grp = tid >> 6, d4 = tid & 63u;
    const float4 *po = reinterpret_cast<const float4 *>(it.part_o + ((size_t)kvh * ns * 32u + row) * 256u) + d4;
    // The first round of piece loads goes out together with the (m, l) loads: neither depends on the other.
    // A round is RND loads per thread, all in flight at once: with one CTA per SM on 148 SMs an item has 74
    // pieces per KV head, which is one round; a second trip to L2 would cost as much as the whole merge.
    constexpr int RND = 20;
    float4 x[RND];
#pragma unroll
    for (int i = 0; i < RND; i++) {
        const uint32_t s = grp + GROUPS * i;
        x[i] = s < ns ? __ldcg(po + (size_t)s * 2048u) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#ifdef MKV_TRACE
    if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tm[0]));
#endif
    float m = NEG_BIG, l = 0.0f;
    if (tid < ns) {
        const float2 y = __ldcg(ml + (size_t)tid * 32u);
        m = y.x;
        l = y.y;
    }
    float M = m;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, sh));
    __syncthreads(); // the previous row's reads of the shared scratch are over
    if ((tid & 31u) == 0) sm.red[tid >> 5] = M;
    __syncthreads();
    if (tid < 32) {
        float y = tid < NW ? sm.red[tid] : NEG_BIG;
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) y = fmaxf(y, __shfl_xor_sync(0xffffffffu, y, sh));
        // a sink logit of the row's head joins the maximum and the sum, never the output (ggml's soft_max with sinks,
        // W/flint_attn.wgsl:243-255)
        if (tid == 0) sm.M = (EXT && it.sinks && !it.partial) ? fmaxf(y, it.sinks[head]) : y;
    }
    __syncthreads();
    M = sm.M;
#ifdef MKV_TRACE
    if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tm[1]));
#endif
    const float e = tid < ns ? expf(m - M) : 0.0f;
    if (tid < ns) sm.e_s[tid] = e;
    float t = e * l;
#pragma unroll
    for (int sh = 16; sh > 0; sh >>= 1) t += __shfl_xor_sync(0xffffffffu, t, sh);
    if ((tid & 31u) == 0) sm.red[tid >> 5] = t; // the maxima were all read before the barrier above
    __syncthreads();
    if (tid < 32) {
        float y = tid < NW ? sm.red[tid] : 0.0f;
#pragma unroll
        for (int sh = 16; sh > 0; sh >>= 1) y += __shfl_xor_sync(0xffffffffu, y, sh);
        if (tid == 0) sm.tot = (EXT && it.sinks && !it.partial) ? y + expf(it.sinks[head] - sm.M) : y;
    }
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t s0 = grp; s0 < ns; s0 += GROUPS * (uint32_t)RND) {
        if (s0 != grp) { // later rounds
#pragma unroll
            for (int i = 0; i < RND; i++) {
                const uint32_t s = s0 + GROUPS * i;
                x[i] = s < ns ? __ldcg(po + (size_t)s * 2048u) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int i = 0; i < RND; i++) {
            const uint32_t s = s0 + GROUPS * i;
            const float w = s < ns ? sm.e_s[s] : 0.0f;
            acc.x += w * x[i].x;
            acc.y += w * x[i].y;
            acc.z += w * x[i].z;
            acc.w += w * x[i].w;
        }
    }
    sm.part[grp][d4] = acc;
    __syncthreads();
#ifdef MKV_TRACE
    if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tm[2]));
#endif
    if (tid < 64) {
        float4 a = sm.part[0][tid];
#pragma unroll
        for (int g = 1; g < GROUPS; g++) {
            const float4 b = sm.part[g][tid];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        const float tot = sm.tot;
        if (it.partial) {
            for (uint32_t dd = 0; dd < ndst; dd++) { // plain peer stores over NVLink when pushing (no multicast)
                float *base = it.push ? it.push->slot[it.push_epoch & 1u][dd] : it.out;
                if (!base) continue; // a rank that never joined the exchange
                float *rec = base + (size_t)(tok * 16u + head) * REC; // records are 8-byte aligned only
                *reinterpret_cast<float2 *>(rec + 2 + 4 * tid) = make_float2(a.x, a.y);
                *reinterpret_cast<float2 *>(rec + 4 + 4 * tid) = make_float2(a.z, a.w);
                if (tid == 0) *reinterpret_cast<float2 *>(rec) = make_float2(M, tot);
            }
        } else {
            const float inv = 1.0f / tot;
            float4 y = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
            const size_t o = (size_t)tok * 4096u + (size_t)head * 256u + 4 * tid;
            if (it.gate) { // attn_gate of the reference (W/ops.wgsl:171-177): times the sigmoid of the head's gate values
                const float4 g = *reinterpret_cast<const float4 *>(it.gate + ((size_t)tok * 16u + head) * 512u + 256u + 4 * tid);
                y.x *= 1.0f / (1.0f + expf(-g.x));
                y.y *= 1.0f / (1.0f + expf(-g.y));
                y.z *= 1.0f / (1.0f + expf(-g.z));
                y.w *= 1.0f / (1.0f + expf(-g.w));
            }
            if (it.out) *reinterpret_cast<float4 *>(it.out + o) = y;
            if (it.out16) { // attn_gate16 (W/ops.wgsl:295-300): the same values as f16
                const __half2 h0 = __floats2half2_rn(y.x, y.y), h1 = __floats2half2_rn(y.z, y.w);
                *reinterpret_cast<uint2 *>(static_cast<__half *>(it.out16) + o) =
                    make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
            }
        }
    }
}

// Called by every thread of every CTA of an item after the CTA's piece has been written to global memory.
// `sm` must not alias anything still in use. Returns after this CTA's share of the merge (possibly none).
template <int NT, bool EXT = true>
__device__ __forceinline__ void finish_item(const VerifyItem &it, FinishSmem &sm, uint32_t *status) {
    const uint32_t total = 2u * it.nsplit;
    __syncthreads(); // every thread's part of the piece precedes thread 0's release below
    if (threadIdx.x == 0) {
        sm.ticket = ptx::atom_add_release_gpu(it.counter, 1u) - it.ticket_base;
#ifdef MKV_TRACE
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[0]));
        sm.tr[1] = sm.tr[2] = 0;
#endif
    }
    __syncthreads();
    const uint32_t ticket = sm.ticket;
    const uint32_t R = total < 64u ? total : 64u;
    if (ticket < total - R) return; // not among the last R: nothing to merge
    if (threadIdx.x == 0) {
        // wait until every CTA of the item has published; bounded, in case a CTA never arrives
        const long long t0 = clock64();
        bool ok = true;
        while (ptx::ld_acquire_gpu(it.counter) - it.ticket_base < total) {
            __nanosleep(32);
            if (clock64() - t0 > 4000000000ll) {
                ok = false;
                break;
            }
        }
        if (!ok) atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        sm.ok = ok ? 1u : 0u;
#ifdef MKV_TRACE
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[1]));
#endif
    }
    __syncthreads();
    if (!sm.ok) return;
    for (uint32_t r = ticket - (total - R); r < 64u; r += R) merge_row<NT, EXT>(it, r, sm);
#ifdef MKV_TRACE
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[2]));
#endif
    if (it.push != nullptr) {
        // this CTA's rows are on their way to every rank; the last of the R merging CTAs raises the flags
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t done = atomicAdd(it.push->rows_done, 1u) - it.push_base;
            if (done == R - 1u) {
                __threadfence_system();
                for (uint32_t dd = 0; dd < it.push->world; dd++)
                    if (it.push->flag[it.push_epoch & 1u][dd]) ptx::st_release_sys(it.push->flag[it.push_epoch & 1u][dd], it.push_epoch);
            }
        }
    }
}

} // namespace mkv
