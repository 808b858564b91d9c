// Log-sum-exp merge of split-K pieces, done inside the attention kernels, and of the shard records of several
// GPUs, done by the same CTAs.
//
// Arithmetic: attn_fd_combine of the reference (W/ops.wgsl:529-537) over this library's pieces:
//   M = max_s m_s;  tot = sum_s e^(m_s - M) l_s;  acc[d] = sum_s e^(m_s - M) O_s[d];  out = acc / tot.
// The sums run over the pieces in index order, so a result does not depend on timing.
//
// Scheduling. Every CTA writes its piece and publishes it: the threads that wrote it meet at a barrier, one of
// them issues a release fence and takes a ticket from a counter in global memory. The last R = min(CTAs of the
// item, 64) arrivals wait (bounded) until the counter shows that all pieces are there, and each merges a share of
// the item's 64 rows. Only CTAs that have finished their own work ever wait, and fewer of them than there are SMs,
// so the others always make progress; the earlier arrivals leave at once, which lets the CTAs of the next launch
// in the stream start on their SMs and load their first tiles.
// (Measured against this: per-piece flags with merging CTAs that gather the pieces as they land, whole rows or
// half rows per CTA. The CTAs that wait hold their SMs, the next launch's CTAs start later and find their first
// tiles not yet loaded when they may begin: 3 to 4 % slower at 65,536 tokens.)
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

// The same with the launch's parameter block: one item and its tensor maps, or a few items (maps in device memory).
__device__ __forceinline__ const VerifyItem &pick_item(const VerifyItem *items, int n_items, const VerifyLaunch &single, uint32_t cta) {
    return pick_item(items, n_items, single.item, cta);
}
__device__ __forceinline__ const VerifyItem &pick_item(const VerifyItem *, int n_items, const VerifyLaunchBatch &few, uint32_t cta) {
    int lo = 0;
    for (int i = 1; i < n_items; i++)
        if (cta >= few.items[i].cta_begin) lo = i;
    return few.items[lo];
}
__device__ __forceinline__ const CUtensorMap *launch_map(const VerifyItem *items, const VerifyItem &it, const VerifyLaunch &single, bool v) {
    return items ? (v ? it.vmap : it.kmap) : (v ? &single.vmap : &single.kmap);
}
__device__ __forceinline__ const CUtensorMap *launch_map(const VerifyItem *, const VerifyItem &it, const VerifyLaunchBatch &, bool v) {
    return v ? it.vmap : it.kmap;
}

constexpr int FIN_MAX_THREADS = 512;
constexpr long long FIN_WAIT_LIMIT = 4000000000ll; // about two seconds of SM clocks
constexpr uint32_t FIN_JOBS = 64;                  // one job per row (kvh * 32 + row) of the item
constexpr uint32_t FIN_COLS = 64;                  // float4 columns of a row

struct FinishSmem {
    float e_s[MAX_SPLITS];
    float red[FIN_MAX_THREADS / 32];
    float tot, M;
    uint32_t ticket, ok;
#ifdef MKV_TRACE
    unsigned long long tr[3]; // ticket taken, all pieces published, rows merged
    unsigned long long tm[4]; // inside the merge of a row: loads issued, maximum known, pieces summed
#endif
    float4 part[FIN_MAX_THREADS / FIN_COLS][FIN_COLS];
};

// Publishes the calling CTA's piece and returns its ticket (arrival number within the item). Called by ONE thread,
// after a barrier that every thread which wrote part of the piece has passed.
__device__ __forceinline__ uint32_t publish_piece(const VerifyItem &it) {
    ptx::fence_acq_rel_gpu(); // the piece (all threads' stores, ordered before this by the barrier) precedes the ticket
    return atomicAdd(it.counter, 1u) - it.ticket_base;
}

// One value of a record as it travels: the f32 bits below the epoch.
__device__ __forceinline__ unsigned long long exch_word(float v, uint32_t epoch) {
    return ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v);
}
// Polls one word of the own mailbox until it carries `epoch` (bounded); the value's bits come back in `bits`.
__device__ __forceinline__ bool exch_poll(const unsigned long long *p, uint32_t epoch, uint32_t &bits) {
    unsigned long long w = ptx::ld_relaxed_sys_u64(p);
    if ((uint32_t)(w >> 32) != epoch) {
        const long long t0 = clock64();
        do {
            __nanosleep(20);
            if (clock64() - t0 > FIN_WAIT_LIMIT) return false;
            w = ptx::ld_relaxed_sys_u64(p);
        } while ((uint32_t)(w >> 32) != epoch);
    }
    bits = (uint32_t)w;
    return true;
}

// Row rr (= tok * 16 + head) of this rank's record has just been stored into every rank's mailbox by threads of this
// CTA (words carrying `epoch`). Waits for the same row of every rank in the own mailbox, value by value, and merges the
// ranks' rows into out[rr][256]. All NT threads of the CTA call this; `ml` is shared scratch of 2 * MAX_PEERS floats.
// On a wait that runs out the status word is set and the output is left alone.
template <int NT>
__device__ __forceinline__ bool exchange_row(const PushInfo &P, uint32_t epoch, uint32_t rr, float *out, uint32_t *status, float *ml) {
    const uint32_t tid = threadIdx.x, par = epoch & 1u, world = P.world;
    const unsigned long long *in = P.inbox[par] + (size_t)rr * REC;
    bool ok = true;
    if (tid < 2u * world) { // (m, l) of every rank's row, for everybody
        uint32_t bits = 0;
        ok = exch_poll(in + (size_t)(tid >> 1) * SLOT_WORDS + (tid & 1u), epoch, bits);
        ml[tid] = __uint_as_float(bits);
    }
    if (!__syncthreads_and(ok)) {
        if (tid == 0) atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        return false;
    }
    float M = NEG_BIG;
    for (uint32_t g = 0; g < world; g++) M = fmaxf(M, ml[2u * g]);
    float tot = 0.0f, acc = 0.0f;
    if (tid < 256u) {
        // the words of all ranks are asked for at once (one round trip to L2, not one per rank); what has not arrived yet
        // is polled afterwards. (Letting every thread fetch the (m, l) words too, to save the barrier above, was measured
        // on 8 GPUs: 19.6 us per layer for the exchange against 10.7 - the polls of 256 threads per row get in the way.)
        unsigned long long w[MAX_PEERS];
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)MAX_PEERS; g++)
            w[g] = g < world ? ptx::ld_relaxed_sys_u64(in + (size_t)g * SLOT_WORDS + 2u + tid) : 0ull;
#pragma unroll
        for (uint32_t g = 0; g < (uint32_t)MAX_PEERS; g++) {
            if (g < world && ok) {
                uint32_t bits = (uint32_t)w[g];
                if ((uint32_t)(w[g] >> 32) != epoch) ok = exch_poll(in + (size_t)g * SLOT_WORDS + 2u + tid, epoch, bits);
                const float e = expf(ml[2u * g] - M);
                tot += e * ml[2u * g + 1u];
                acc += e * __uint_as_float(bits);
            }
        }
    }
    if (!__syncthreads_and(ok)) { // (also keeps `ml` until everybody has read it)
        if (tid == 0) atomicOr(status, DEV_ERR_WAIT_TIMEOUT);
        return false;
    }
    if (tid < 256u) out[(size_t)rr * 256u + tid] = acc / tot;
    return true;
}

// One row (kvh * 32 + row) of one item, by all NT threads of the CTA; all pieces are in global memory.
// EXT = false compiles the sink handling out (the kernels of the plain path are instantiated without it).
template <int NT, bool EXT>
__device__ __forceinline__ void merge_row(const VerifyItem &it, uint32_t r, FinishSmem &sm, uint32_t *status) {
    constexpr int GROUPS = NT / FIN_COLS;
    constexpr int NW = NT / 32;
    constexpr int RND = (MAX_SPLITS + GROUPS - 1) / GROUPS; // pieces a thread may own: all in flight at once, one trip to L2
    const uint32_t kvh = r >> 5, row = r & 31u, tok = row >> 3, head = 8u * kvh + (row & 7u);
    const uint32_t tid = threadIdx.x;
    if (tok >= it.ntok) {
        if (it.partial && !it.push && tid < 258u) // rows of tokens beyond the step: the empty record
            it.out[(size_t)(tok * 16u + head) * REC + tid] = tid == 0 ? NEG_BIG : 0.0f;
        return;
    }
    const uint32_t ns = it.nsplit;
    const float2 *ml = reinterpret_cast<const float2 *>(it.part_ml) + (size_t)kvh * ns * 32u + row;
    const uint32_t grp = tid / FIN_COLS, c4 = tid % FIN_COLS;
    const float4 *po = reinterpret_cast<const float4 *>(it.part_o + ((size_t)kvh * ns * 32u + row) * 256u) + c4;
    float4 x[RND];
    float m = NEG_BIG, l = 0.0f;
    // the head's gate values, if any, with the first loads: at the end of the row they would be one more round trip
    float4 gate = make_float4(0.f, 0.f, 0.f, 0.f);
    if (!it.partial && it.gate && tid < FIN_COLS)
        gate = __ldg(reinterpret_cast<const float4 *>(it.gate + ((size_t)tok * 16u + head) * 512u + 256u + 4 * tid));
    if (tid < ns) { // (m, l) first: the maximum is needed before anything can be summed
        const float2 y = __ldcg(ml + (size_t)tid * 32u);
        m = y.x;
        l = y.y;
    }
#pragma unroll
    for (int i = 0; i < RND; i++) { // thread (grp, c4) owns pieces grp, grp + GROUPS, ...
        const uint32_t s = grp + GROUPS * i;
        x[i] = s < ns ? __ldcg(po + (size_t)s * 2048u) : make_float4(0.f, 0.f, 0.f, 0.f);
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
#pragma unroll
    for (int i = 0; i < RND; i++) {
        const uint32_t s = grp + GROUPS * i;
        const float w = s < ns ? sm.e_s[s] : 0.0f;
        acc.x += w * x[i].x;
        acc.y += w * x[i].y;
        acc.z += w * x[i].z;
        acc.w += w * x[i].w;
    }
    sm.part[grp][c4] = acc;
    __syncthreads();
#ifdef MKV_TRACE
    if (tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tm[2]));
#endif
    if (tid < FIN_COLS) {
        float4 a = sm.part[0][tid];
#pragma unroll
        for (int g = 1; g < GROUPS; g++) { // in group order: pieces g, g + GROUPS, ... were summed in index order above
            const float4 b = sm.part[g][tid];
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        const float tot = sm.tot;
        if (it.partial) {
            if (it.push) { // the row goes to every rank's mailbox: plain peer stores over NVLink (no multicast), one word per value
                const PushInfo &P = *it.push;
                for (uint32_t dd = 0; dd < P.world; dd++) {
                    unsigned long long *rec = P.slot[it.push_epoch & 1u][dd];
                    if (!rec) continue; // a rank that never joined the exchange
                    rec += (size_t)(tok * 16u + head) * REC;
                    ptx::st_relaxed_sys_u64(rec + 2 + 4 * tid, exch_word(a.x, it.push_epoch));
                    ptx::st_relaxed_sys_u64(rec + 3 + 4 * tid, exch_word(a.y, it.push_epoch));
                    ptx::st_relaxed_sys_u64(rec + 4 + 4 * tid, exch_word(a.z, it.push_epoch));
                    ptx::st_relaxed_sys_u64(rec + 5 + 4 * tid, exch_word(a.w, it.push_epoch));
                    if (tid == 0) {
                        ptx::st_relaxed_sys_u64(rec, exch_word(M, it.push_epoch));
                        ptx::st_relaxed_sys_u64(rec + 1, exch_word(tot, it.push_epoch));
                    }
                }
            } else { // the un-normalised record itself (records are 8-byte aligned only)
                float *rec = it.out + (size_t)(tok * 16u + head) * REC;
                *reinterpret_cast<float2 *>(rec + 2 + 4 * tid) = make_float2(a.x, a.y);
                *reinterpret_cast<float2 *>(rec + 4 + 4 * tid) = make_float2(a.z, a.w);
                if (tid == 0) *reinterpret_cast<float2 *>(rec) = make_float2(M, tot);
            }
        } else {
            const float inv = 1.0f / tot;
            float4 y = make_float4(a.x * inv, a.y * inv, a.z * inv, a.w * inv);
            const size_t o = (size_t)tok * 4096u + (size_t)head * 256u + 4 * tid;
            if (it.gate) { // attn_gate of the reference (W/ops.wgsl:171-177): times the sigmoid of the head's gate values
                const float4 g = gate;
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
    if (it.partial && it.push && !exchange_row<NT>(*it.push, it.push_epoch, tok * 16u + head, it.out, status, sm.red)) {
        if (tid == 0) sm.ok = 0u; // a rank never delivered: the CTA's other rows would only wait as long again
        __syncthreads();
    }
}

// The CTA's share of the merge, given its ticket (publish_piece). Called by every thread of every CTA of an item;
// `sm` must not alias anything still in use and nobody may have touched it since a barrier. Returns after this
// CTA's rows (possibly none).
template <int NT, bool EXT = true>
__device__ __forceinline__ void finish_item(const VerifyItem &it, FinishSmem &sm, uint32_t *status, uint32_t ticket) {
    const uint32_t total = 2u * it.nsplit;
    const uint32_t R = total < FIN_JOBS ? total : FIN_JOBS;
    if (ticket < total - R) return; // not among the last R: nothing to merge
    if (threadIdx.x == 0) {
#ifdef MKV_TRACE
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[0]));
        sm.tr[1] = sm.tr[2] = 0;
#endif
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
    __syncthreads(); // thread 0's acquire, passed on by the barrier, orders the piece loads (which bypass L1) behind the publications
    if (!sm.ok) return;
    for (uint32_t r = ticket - (total - R); r < FIN_JOBS; r += R) {
        merge_row<NT, EXT>(it, r, sm, status);
        if (!sm.ok) return;
    }
#ifdef MKV_TRACE
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sm.tr[2]));
#endif
}

// The same for kernels that publish here: every thread's part of the piece is written, then thread 0 publishes.
template <int NT, bool EXT = true>
__device__ __forceinline__ void finish_item(const VerifyItem &it, FinishSmem &sm, uint32_t *status) {
    __syncthreads(); // every thread's part of the piece precedes thread 0's fence
    if (threadIdx.x == 0) sm.ticket = publish_piece(it);
    __syncthreads();
    const uint32_t ticket = sm.ticket;
    __syncthreads(); // (sm.ok is written next)
    finish_item<NT, EXT>(it, sm, status, ticket);
}

} // namespace mkv
