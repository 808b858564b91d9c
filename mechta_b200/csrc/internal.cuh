// Internal declarations shared by the kernels and the C-ABI host code of libmechta_kv.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/mechta_kv.h"

namespace mkv {

constexpr int HQ = 16, HKV = 2, D = 256, GROUP = 8, ROW = 512, REC = 258;
constexpr int TILE = 64;            // keys per verify tile, f16 cache (as the reference, M/dmx.rs:53)
constexpr int PF_TILE = 64;         // keys per prefill tile (as the reference, W/fa_mx.wgsl:27)
constexpr int TILE32 = 32;          // keys per tile, f32 cache
constexpr float NEG_BIG = -3.0e38f; // mask value of the reference (W/ops.wgsl:339)
constexpr float NEG_TEST = -1.0e38f;
constexpr float SCALE = 1.0f / 16.0f; // M/quad.rs:286 bits(1/16)
constexpr int MAX_SPLITS = 80;      // upper bound of split-K pieces per KV head of one item (what a merging CTA holds in registers)

// status word written by kernels instead of trapping (bit set = what went wrong)
enum : uint32_t { DEV_ERR_WAIT_TIMEOUT = 1u };

void set_error(const char *fmt, ...);

#define MKV_CUDA(expr)                                                                         \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess) {                                                              \
            mkv::set_error("%s: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
            return MKV_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

// Peer exchange of shard records without a collective library: where a rank's merged record goes. Every f32 value of a
// record travels as one 8-byte word, the value's bits below the number of the exchange call (the "epoch", never 0): a
// word is stored and loaded whole, so a receiver that polls it and finds the current epoch has the value, with no flag
// and no release / acquire round trip behind the data (the low-latency protocol of collective libraries).
constexpr int MAX_PEERS = 8;
constexpr size_t SLOT_WORDS = 64 * 258; // one record [64 rows][258], one 8-byte word per value
struct PushInfo {
    unsigned long long *slot[2][MAX_PEERS]; // [epoch parity][destination rank]: this rank's record in that rank's mailbox
    const unsigned long long *inbox[2];     // this rank's own mailbox: [epoch parity] -> records [world][64][258]
    uint32_t world;
};

// One split-K work item of the verify attention: everything a CTA needs, in device memory or in the
// kernel's parameter space.
struct VerifyItem {
    const CUtensorMap *kmap; // device address of the layer's K tensor map
    const CUtensorMap *vmap;
    const float *q; // [ntok][16][256]
    float *out;     // [ntok][16][256], or the [64][258] record in partial mode
    float *part_ml; // [2][nsplit][32][2]
    float *part_o;  // [2][nsplit][32][256]
    uint32_t first_pos, pos, ntok;
    uint32_t row0;     // global position of the cache's first row (shard_first)
    uint32_t key_lo;   // visible keys are key_lo <= key < min(key_hi, pos+1+tok)
    uint32_t key_hi;
    uint32_t tile_begin, tile_end; // absolute tile range [tile_begin, tile_end), tile j = keys [T*j, T*j+T)
    uint32_t nsplit;               // pieces per KV head
    uint32_t tiles_per_split;
    uint32_t cta_begin; // first CTA of this item in the flattened grid (2 * nsplit CTAs per item)
    uint32_t partial;   // 1: write the un-normalised record instead of the final output
    uint32_t *counter;  // arrival counter of this item's CTAs (global memory), never reset
    uint32_t ticket_base; // value of the counter before this launch
    const PushInfo *push; // partial mode only: the record's rows go to every rank's mailbox, the rows of all ranks are
                          // merged here and `out` gets the final output
    uint32_t push_world;  // number of ranks (host copy of push->world)
    uint32_t push_epoch;  // the exchange's call number
    uint32_t safe_below; // keys below this were not written by the kernel launched just before this one
    uint32_t ring;       // rows of a ring cache (row = position % ring), 0 = rows are positions minus row0
    uint32_t win;        // sliding window: token t sees keys > pos + t - win (0 = no window)
    const float *sinks;  // final mode only: [16] per-head sink logits that join the softmax's max and sum, or null
    const float *gate;   // final mode only: [ntok][16][512] with the output gate in the second half of each head, or null
    void *out16;         // final mode only: the output once more as f16 [ntok][16][256], or null
    uint32_t phase;     // read by builds with -DMKV_MEASURE only (the reference's p.f1 phases: 0 = everything, 1 = tile loads only)
};

// Measurement builds (make measure: -DMKV_MEASURE) can run parts of a kernel in isolation and record per-CTA
// timelines; the shipped library compiles all of that out, so its kernels carry no measurement branches.
#ifdef MKV_MEASURE
#define MKV_TRACE 1
#define MKV_PHASE_OF(it) ((it).phase)
#else
#define MKV_PHASE_OF(it) 0u
#endif

// What a single (non-batched) launch carries in the kernel's parameter space: the item and its two tensor
// maps, so that the TMA unit does not have to fetch the maps from global memory first.
// Row of the cache that holds absolute position `key`.
__host__ __device__ inline uint32_t cache_row(const VerifyItem &it, uint32_t key) { return it.ring ? key % it.ring : key - it.row0; }
// Lowest key token t of the step sees: the call's first position, the shard's first row, the window.
__host__ __device__ inline uint32_t lowest_key(const VerifyItem &it, uint32_t t) {
    uint32_t lo = it.first_pos > it.key_lo ? it.first_pos : it.key_lo;
    if (it.win && it.pos + t + 1u > it.win && it.pos + t + 1u - it.win > lo) lo = it.pos + t + 1u - it.win;
    return lo;
}

struct VerifyLaunch {
    VerifyItem item;
    alignas(64) CUtensorMap kmap;
    alignas(64) CUtensorMap vmap;
};

// A batch of a few items carried in the kernel's parameter space (their tensor maps stay in device memory): no staging
// copy stands between two launches, so the launches of a step's layers keep their programmatic overlap.
constexpr int PARAM_ITEMS = 16;
struct VerifyLaunchBatch {
    VerifyItem items[PARAM_ITEMS];
};
static_assert(sizeof(VerifyLaunchBatch) <= 4000, "the parameter block of a small batch must fit the 4 KB of kernel parameters");

struct Ctx;
struct Cache;

struct Ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev_compute = nullptr; // compute -> copy ordering
    cudaEvent_t ev_copy = nullptr;    // copy -> compute ordering
    uint32_t *dev_status = nullptr;   // device status word
    float *pf_scratch = nullptr;      // prefill: partials of items split over two CTAs (prefill_tc.cu), allocated on first use
    uint32_t *pf_counters = nullptr;  // prefill: arrival counter per work item, zero between launches
    uint64_t launches = 0;
    uint64_t syncs = 0;               // mkv_sync calls so far: what was enqueued before the last of them has finished
    bool pdl = true; // programmatic dependent launch of the attention kernels (MKV_PDL=0 switches it off)
    // profiling of the attention core kernels
    bool prof = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events;
    size_t prof_used = 0;
    // staging ring for batched items: pinned host slots, device slots, one event per slot
    static constexpr int SLOTS = 8;
    static constexpr int SLOT_ITEMS = 1024;
    VerifyItem *items_dev = nullptr;  // [SLOTS][SLOT_ITEMS]
    VerifyItem *items_host = nullptr; // pinned, same shape
    cudaEvent_t slot_done[SLOTS] = {};
    bool slot_used[SLOTS] = {};
    int slot_next = 0;
    uint32_t *counters_dev = nullptr;          // [SLOT_ITEMS] arrival counters, zeroed once
    std::vector<uint32_t> counter_base;        // host shadow: value of each counter after the launches so far
    // lifetime: caches hold a reference; a ctx destroyed while caches live is freed with the last of them
    int live_caches = 0;
    bool closing = false;
};

struct Cache {
    Ctx *ctx = nullptr;
    mkv_fmt fmt = MKV_F16;
    int n_layers = 0;
    uint32_t context = 0;  // tokens of the whole sequence's context
    uint32_t ring = 0;               // rows of a ring cache (then capacity == ring), 0 otherwise
    uint32_t capacity = 0; // rows held here
    uint32_t shard_first = 0;
    bool whole = true;     // holds the whole context (not a sequence shard)
    uint32_t len = 0; // global position after the last valid row
    // Lowest position the recent writers (append, restore, scrub, the host) touched, each with the number of launches
    // the context had made by then and the number of mkv_sync calls it had seen. An attention kernel may load tiles below all of them before the kernels
    // in front of it have finished: with programmatic dependent launch a whole chain of small launches can be
    // resident at once, so the writer just in front is not the only one that may still be running. Each
    // attention CTA fills an SM's shared memory, so at most one per SM can be resident and the chain is shorter
    // than WRITE_WINDOW launches. Writers noted before the context's last mkv_sync have finished and are dropped.
    static constexpr uint64_t WRITE_WINDOW = 160;
    struct Write {
        uint64_t launches, syncs;
        uint32_t pos;
    };
    std::vector<Write> writes;
    void note_write(uint32_t pos);
    uint32_t safe_below(uint32_t pos) const;
    size_t elem = 2;
    size_t buf_bytes = 0;
    std::vector<void *> k, v;
    void **kptrs_dev = nullptr;      // [n_layers] device copies of k / v
    void **vptrs_dev = nullptr;
    std::vector<CUtensorMap> maps_host;
    CUtensorMap *maps_dev = nullptr; // [n_layers][2] with the verify tile's box, then [n_layers][2] with the prefill tile's
    std::vector<std::pair<void *, size_t>> guarded; // the checked build: buffers bracketed by canary bytes (pointer, size)
    float *qr = nullptr;             // [4][16][256] normalised and rotated queries of mkv_attn_step (stream-ordered)
    float *part_ml = nullptr;        // split-K scratch, shared by the layers (stream-ordered), grow-only
    float *part_o = nullptr;
    size_t scratch_pieces = 0;       // pieces (KV head x split) the scratch holds
    cudaEvent_t ev_snapshot = nullptr;
    bool snapshot_pending = false;
};

struct Exchange {
    Ctx *ctx = nullptr;
    int rank = 0, world = 1;
    unsigned char *mailbox = nullptr; // records[2][world][SLOT_WORDS] of 8-byte (value, epoch) words
    size_t mailbox_bytes = 0;
    void *peer_base[MAX_PEERS] = {};
    PushInfo *push_dev = nullptr;
    uint32_t epoch = 0;
    bool connected = false;
};

// ---- launchers (defined in the .cu files) ---------------------------------------------------------------
mkv_status launch_append(Ctx *ctx, mkv_fmt fmt, void *const *kbufs, void *const *vbufs, int n_layers,
                         size_t layer_stride_in, uint32_t row_first, uint32_t capacity, uint32_t ring, uint32_t pos,
                         uint32_t ntok, const float *k, const float *v, const float *tab,
                         uint32_t which /*1 = K, 2 = V, 3 = both*/);
// items_host[0..n) are planned; batch = false: n == 1 and the item travels in the kernel's parameter space
mkv_status launch_verify(Ctx *ctx, mkv_fmt fmt, VerifyItem *items_host, int n, bool batch, const CUtensorMap *kmap_host,
                         const CUtensorMap *vmap_host);
mkv_status verify_setup_device();
mkv_status launch_combine_shards(Ctx *ctx, const float *recs, int n_shards, uint32_t ntok, float *out);
mkv_status launch_step_prep(Ctx *ctx, mkv_fmt fmt, const float *qf, const float *kb, const float *vb, const float *q_norm,
                            const float *k_norm, const float *tab, float eps, float *qr, void *kcache, void *vcache,
                            uint32_t row_first, uint32_t capacity, uint32_t ring, uint32_t pos, uint32_t ntok);
// a shard without any visible key: its (empty) record rows still go to every rank, and the ranks' rows are merged into `out`
mkv_status launch_exchange_empty(Ctx *ctx, const PushInfo *push, uint32_t epoch, uint32_t ntok, float *out);
// plans the split of the items so that the grid fills the SMs once
void plan_items(Ctx *ctx, VerifyItem *items, int n);

} // namespace mkv
