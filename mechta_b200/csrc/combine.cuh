// Log-sum-exp merge of split-K pieces, done inside the attention kernels, and of the shard records of several
// GPUs, done by the same CTAs.
//
// Arithmetic: attn_fd_combine of the reference (W/ops.wgsl:529-537) over this library's pieces:
//   M = max_s m_s;  tot = sum_s e^(m_s - M) l_s;  acc[d] = sum_s e^(m_s - M) O_s[d];  out = acc / tot.
// The sums run over the pieces in index order whatever the order of their arrival, so a result does not depend
// on timing.
//
// Scheduling. Every CTA writes its piece, publishes it (one flag word per piece, written with release semantics
// and holding the launch's number) and takes a ticket from a counter in global memory. R = min(CTAs of the
// item, 64) of them each merge a share of the item's 64 rows: the ones that arrive just BEFORE the last few. A
// merging CTA gathers the pieces as their flags come up, so by the time the last piece is published everything
// else is already in its registers and what is left after the last piece is one flag, one load and the sums.
// (Letting the very last arrivals merge, as an arrival counter alone would suggest, puts the whole gather of
// ~74 pieces per row behind the last piece.) A waiting CTA has finished its own tiles, there are at most 64 of
// them and the grid is planned to fit the SMs in one wave, so the CTAs they wait for always run; every wait is
// bounded all the same. Items whose pieces carry no flags (flags == null: the allocation-free entry point) use
// the counter alone: the last R arrivals wait until it shows that all pieces are there.
//
// Sequence shards on several GPUs (`push` set): the merged rows are this rank's record. The merging CTA stores
// each row straight into every rank's mailbox (plain peer stores over NVLink, no multicast), raises that row's
// flag there (st.release.sys), waits (bounded) for the same row from every other rank in its own mailbox and
// merges the ranks' rows into the final output: one launch per layer, no collective call, no second kernel.
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
constexpr long long FIN_WAIT_LIMIT = 4000000000ll; // about two seconds of SM clocks
constexpr uint32_t FIN_LATE = 20;                  // the last arrivals that do not merge (when there are enough CTAs)

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

// Row rr (= tok * 16 + head) of this rank's record has just been stored into every rank's mailbox by the threads
// of this CTA. Raises the row's flag everywhere, waits for the same row of every other rank and merges the
// ranks' rows into out[rr][256]. All NT threads of the CTA call this. On a wait that runs out the status word
// is set and the output is left alone.
template <int NT>
__device__ __forceinline__ bool exchange_row(const PushInfo &P, uint32_t epoch, uint32_t rr, float *out, uint32_t *status) {
    const uint32_t tid = threadIdx.x, par = epoch & 1u, world = P.world;
    __syncthreads(); // the row's stores of all threads precede the releases below
    if (tid < world && P.rowflag[par][tid]) ptx::st_release_sys(P.rowflag[par][tid] + rr, epoch);
    bool ok = true;
    if (tid < world) {
        const uint32_t *f = P.inflag[par] + (size_t)tid * FLAG_WORDS + rr;
        const long long t0 = clock64();
        while (ptx::ld_acquire_sys(f) != epoch) {
            __nanosleep(40);
            if (clock64() - t0 > FIN_WAIT_LIMIT) {
                ok = false;
                break;
            }
        }
    }
    if (!__syncthreads_and(ok)) {
        if (tid == 0) atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        return false;
    }
    const float *in = P.inbox[par] + (size_t)rr * REC;
    float M = NEG_BIG;
    for (uint32_t g = 0; g < world; g++) M = fmaxf(M, __ldcg(in + (size_t)g * SLOT_FLOATS));
    for (uint32_t d = tid; d < 256u; d += NT) {
        float tot = 0.0f, acc = 0.0f;
        for (uint32_t g = 0; g < world; g++) {
            const float *x = in + (size_t)g * SLOT_FLOATS;
            const float e = expf(__ldcg(x) - M);
            tot += e * __ldcg(x + 1);
            acc += e * __ldcg(x + 2 + d);
        }
        out[(size_t)rr * 256u + d] = acc / tot;
    }
    return true;
}

// One row (kvh * 32 + row) of one item, by all NT threads of the CTA.
// GATHER: the pieces may still be arriving; a piece is read once its flag shows this launch's number.
// Otherwise all pieces are known to be in global memory.
// EXT = false compiles the sink handling out (the kernels of the plain path are instantiated without it).
template <int NT, bool EXT, bool GATHER>
__device__ __forceinline__ void merge_row(const VerifyItem &it, uint32_t r, FinishSmem &sm, uint32_t *status) {
    constexpr int GROUPS = NT / 64;
    constexpr int NW = NT / 32;
    const uint32_t kvh = r >> 5, row = r & 31u, tok = row >> 3, head = 8u * kvh + (row & 7u);
    const uint32_t tid = threadIdx.x;
    if (tok >= it.ntok) {
        if (it.partial && !it.push && tid < 258u) // rows of tokens beyond the step: the empty record
            it.out[(size_t)(tok * 16u + head) * REC + tid] = tid == 0 ? NEG_BIG : 0.0f;
        return;
    }
    const uint32_t ns = it.nsplit;
    const float2 *ml = reinterpret_cast<const float2 *>(it.part_ml) + (size_t)kvh * ns * 32u + row;
    const uint32_t grp = tid >> 6, d4 = tid & 63u;
    const float4 *po = reinterpret_cast<const float4 *>(it.part_o + ((size_t)kvh * ns * 32u + row) * 256u) + d4;
    // A round is RND loads per thread, all in flight at once: with one CTA per SM on 148 SMs an item has 74
    // pieces per KV head, which is one round; a second trip to L2 would cost as much as the whole merge.
    constexpr int RND = 20;
    float4 x[RND];
    float m = NEG_BIG, l = 0.0f;
    if (GATHER) {
        // thread (grp, d4) owns pieces grp, grp + GROUPS, ...; thread tid < ns also owns (m, l) of piece tid
        const uint32_t *fl = it.flags + (size_t)kvh * ns;
        const uint32_t ep = it.epoch;
        uint32_t pend = 0;
#pragma unroll
        for (int i = 0; i < RND; i++) {
            x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (grp + GROUPS * (uint32_t)i < ns) pend |= 1u << i;
        }
        bool mlpend = tid < ns;
        const long long t0 = clock64();
        for (;;) {
            uint32_t got = 0, f[RND];
#pragma unroll
            for (int i = 0; i < RND; i++) // the flag loads of a round are all in flight together
                f[i] = ((pend >> i) & 1u) ? ptx::ld_relaxed_gpu(fl + grp + GROUPS * i) : ~ep;
            const uint32_t fm = mlpend ? ptx::ld_relaxed_gpu(fl + tid) : ~ep;
#pragma unroll
            for (int i = 0; i < RND; i++)
                if (f[i] == ep) got |= 1u << i;
            const bool gm = fm == ep;
            if (got != 0u || gm) {
                __threadfence(); // with the relaxed flag loads above: acquire
#pragma unroll
                for (int i = 0; i < RND; i++)
                    if ((got >> i) & 1u) x[i] = __ldcg(po + (size_t)(grp + GROUPS * i) * 2048u);
                if (gm) {
                    const float2 y = __ldcg(ml + (size_t)tid * 32u);
                    m = y.x;
                    l = y.y;
                    mlpend = false;
                }
                pend &= ~got;
            }
            if (tid == 0 && clock64() - t0 > FIN_WAIT_LIMIT) sm.ok = 0u; // a piece never came
            if (__syncthreads_and(pend == 0u && !mlpend)) break;
            if (!sm.ok) {
                if (tid == 0) atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
                return;
            }
        }
    } else {
        if (tid < ns) { // (m, l) first: the maximum is needed before anything can be summed
            const float2 y = __ldcg(ml + (size_t)tid * 32u);
            m = y.x;
            l = y.y;
        }
#pragma unroll
        for (int i = 0; i < RND; i++) {
            const uint32_t s = grp + GROUPS * i;
            x[i] = s < ns ? __ldcg(po + (size_t)s * 2048u) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
#ifdef MKV_TRACE
    if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tm[0]));
#endif
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
        if (s0 != grp) { // later rounds (more pieces than one round holds; never with GATHER)
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
            const uint32_t ndst = it.push ? it.push->world : 1u; // the record goes to `out`, or to every rank's mailbox
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
    if (it.partial && it.push && !exchange_row<NT>(*it.push, it.push_epoch, tok * 16u + head, it.out, status)) {
        if (tid == 0) sm.ok = 0u; // a rank never delivered: the CTA's other rows would only wait as long again
        __syncthreads();
    }
}

// Called by every thread of every CTA of an item after the CTA's piece has been written to global memory.
// `sm` must not alias anything still in use. Returns after this CTA's share of the merge (possibly none).
template <int NT, bool EXT = true>
__device__ __forceinline__ void finish_item(const VerifyItem &it, FinishSmem &sm, uint32_t *status) {
    const uint32_t total = 2u * it.nsplit;
    // A round of gathered loads holds 20 pieces per group of 64 threads; items with more pieces per KV head (never
    // planned on a B200) and items without flags announce their pieces by the counter alone.
    const bool gather = it.flags != nullptr && it.nsplit <= (uint32_t)(NT / 64) * 20u;
    __syncthreads(); // every thread's part of the piece precedes thread 0's release below
    if (threadIdx.x == 0) {
        if (gather) {
            const uint32_t local = blockIdx.x - it.cta_begin; // piece (kvh, split) = (local & 1, local >> 1)
            ptx::st_release_gpu(it.flags + (size_t)(local & 1u) * it.nsplit + (local >> 1), it.epoch);
            sm.ticket = atomicAdd(it.counter, 1u) - it.ticket_base;
        } else {
            sm.ticket = ptx::atom_add_release_gpu(it.counter, 1u) - it.ticket_base;
        }
        sm.ok = 1u;
#ifdef MKV_TRACE
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[0]));
        sm.tr[1] = sm.tr[2] = 0;
#endif
    }
    __syncthreads();
    const uint32_t ticket = sm.ticket;
    const uint32_t R = total < 64u ? total : 64u;
    const uint32_t late = gather ? (total - R < FIN_LATE ? total - R : FIN_LATE) : 0u;
    const uint32_t first = total - R - late; // tickets [first, first + R) merge
    if (ticket < first || ticket >= first + R) return;
    if (!gather) {
        if (threadIdx.x == 0) {
            // wait until every CTA of the item has published; bounded, in case a CTA never arrives
            const long long t0 = clock64();
            bool ok = true;
            while (ptx::ld_acquire_gpu(it.counter) - it.ticket_base < total) {
                __nanosleep(32);
                if (clock64() - t0 > FIN_WAIT_LIMIT) {
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
        for (uint32_t r = ticket - first; r < 64u; r += R) {
            merge_row<NT, EXT, false>(it, r, sm, status);
            if (!sm.ok) return;
        }
    } else {
        for (uint32_t r = ticket - first; r < 64u; r += R) {
            merge_row<NT, EXT, true>(it, r, sm, status);
            if (!sm.ok) return;
        }
    }
#ifdef MKV_TRACE
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[2]));
#endif
}

} // namespace mkv
