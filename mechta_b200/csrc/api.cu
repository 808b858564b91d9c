// C-ABI host side of libmechta_kv: contexts, caches, argument checks, stream ordering. The kernels are in the
// other .cu files; the declarations and their reference citations are in include/mechta_kv.h.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <new>

#include "internal.cuh"

namespace mkv {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
}

mkv_status prefill_setup_device();
mkv_status prefill_tc_setup_device();
mkv_status launch_prefill_f16_tc(Ctx *ctx, Cache *c, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                                 const void *q, bool q_is_f16, float *out);
mkv_status launch_q_f16(Ctx *ctx, const float *src, void *dst, size_t n_pairs);
mkv_status append_setup_device();
mkv_status launch_prefill_f16_mma(Ctx *ctx, Cache *c, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                                  const float *q, float *out);

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Tensor map of one K or V buffer seen as [rows][512] elements; boxes of 128 bytes x `box_rows` rows with the
// 128-byte swizzle. Rows past the end read as zero.
static mkv_status make_tensor_map(CUtensorMap *out, mkv_fmt fmt, void *base, uint32_t rows, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) {
        set_error("cuTensorMapEncodeTiled is not available from the driver");
        return MKV_ERR_CUDA;
    }
    const size_t elem = fmt == MKV_F16 ? 2 : 4;
    cuuint64_t dims[2] = {512, rows};
    cuuint64_t strides[1] = {512 * elem};
    cuuint32_t box[2] = {(cuuint32_t)(128 / elem), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(out, fmt == MKV_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims,
                     strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with %d", (int)r);
        return MKV_ERR_CUDA;
    }
    return MKV_OK;
}

// Measurement builds only (-DMKV_MEASURE): MKV_PHASE in the environment makes the kernels run a part of their work
// alone (1 = stream the tiles only, ...; results are then wrong). The shipped library ignores the variable.
static uint32_t measure_phase() {
#ifdef MKV_MEASURE
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("MKV_PHASE");
        v = e ? atoi(e) : 0;
    }
    return (uint32_t)v;
#else
    return 0u;
#endif
}

void Cache::note_write(uint32_t pos) {
    size_t keep = 0;
    for (size_t i = 0; i < writes.size(); i++)
        if (writes[i].launches + WRITE_WINDOW > ctx->launches && writes[i].syncs == ctx->syncs) writes[keep++] = writes[i];
    writes.resize(keep);
    writes.push_back({ctx->launches, ctx->syncs, pos});
}

uint32_t Cache::safe_below(uint32_t pos) const {
    uint32_t lo = pos;
    for (const auto &w : writes)
        if (w.launches + WRITE_WINDOW > ctx->launches && w.syncs == ctx->syncs) lo = std::min(lo, w.pos);
    return lo;
}

static mkv_status use_device(Ctx *ctx) {
    MKV_CUDA(cudaSetDevice(ctx->device));
    return MKV_OK;
}

// Reads and clears the device status word (blocks); nonzero means a kernel gave up on a wait.
static mkv_status check_device_status(Ctx *ctx) {
    uint32_t st = 0;
    MKV_CUDA(cudaMemcpy(&st, ctx->dev_status, 4, cudaMemcpyDeviceToHost));
    if (st != 0) {
        MKV_CUDA(cudaMemset(ctx->dev_status, 0, 4));
        set_error("a kernel reported status 0x%x (1 = a bounded wait ran out)", st);
        return MKV_ERR_CUDA;
    }
    return MKV_OK;
}

// ---- guarded allocations (the checked build, -DMKV_CHECKS) ---------------------------------------------------
// Every buffer of a cache (the K and V rows of each layer, the split-K pieces) is bracketed by GUARD bytes of a canary
// pattern that no kernel may touch; mkv_cache_check_guards counts the bytes that changed. The shipped build allocates
// the buffers as they are and its check has nothing to look at.
#ifdef MKV_CHECKS
static constexpr size_t GUARD = 65536; // a multiple of every alignment the kernels and TMA ask of a buffer
static constexpr int CANARY = 0xA5;
#else
static constexpr size_t GUARD = 0;
#endif
static cudaError_t guard_malloc(Cache *c, void **out, size_t bytes) {
    char *p = nullptr;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&p), bytes + 2 * GUARD);
    if (e != cudaSuccess) return e;
#ifdef MKV_CHECKS
    if ((e = cudaMemset(p, CANARY, GUARD)) != cudaSuccess || (e = cudaMemset(p + GUARD + bytes, CANARY, GUARD)) != cudaSuccess) {
        cudaFree(p);
        return e;
    }
    c->guarded.push_back({p + GUARD, bytes});
#else
    (void)c;
#endif
    *out = p + GUARD;
    return cudaSuccess;
}
static void guard_free(Cache *c, void *p) {
    if (!p) return;
#ifdef MKV_CHECKS
    for (size_t i = 0; i < c->guarded.size(); i++)
        if (c->guarded[i].first == p) {
            c->guarded.erase(c->guarded.begin() + (long)i);
            break;
        }
#else
    (void)c;
#endif
    cudaFree(static_cast<char *>(p) - GUARD);
}

static mkv_status ensure_scratch(Cache *c, size_t pieces) {
    if (pieces <= c->scratch_pieces) return MKV_OK;
    Ctx *ctx = c->ctx;
    // earlier launches may still read the old buffers
    MKV_CUDA(cudaStreamSynchronize(ctx->stream));
    guard_free(c, c->part_ml);
    guard_free(c, c->part_o);
    c->part_ml = c->part_o = nullptr;
    c->scratch_pieces = 0;
    if (guard_malloc(c, reinterpret_cast<void **>(&c->part_ml), pieces * 32 * 2 * sizeof(float)) != cudaSuccess ||
        guard_malloc(c, reinterpret_cast<void **>(&c->part_o), pieces * 32 * 256 * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        set_error("out of device memory for %zu split-K pieces", pieces);
        return MKV_ERR_NOMEM;
    }
    c->scratch_pieces = pieces;
    return MKV_OK;
}

// Fills the position-dependent part of an item and its tile range. Returns MKV_ERR_* on bad arguments.
static mkv_status fill_item(Cache *c, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok, const float *q, float *out,
                            bool partial, VerifyItem *it) {
    if (!c || !q || !out) {
        set_error("null argument");
        return MKV_ERR_INVALID;
    }
    if (layer < 0 || layer >= c->n_layers) {
        set_error("layer %d outside [0, %d)", layer, c->n_layers);
        return MKV_ERR_INVALID;
    }
    if (ntok < 1 || ntok > MKV_MAX_VERIFY) {
        set_error("ntok %u outside [1, %d]", ntok, MKV_MAX_VERIFY);
        return MKV_ERR_INVALID;
    }
    if (((uintptr_t)q & 15u) || ((uintptr_t)out & 7u)) {
        set_error("q must be 16-byte aligned and out 8-byte aligned");
        return MKV_ERR_INVALID;
    }
    const uint64_t end = (uint64_t)pos + ntok;
    if (end > (uint64_t)c->context) {
        set_error("pos %u + ntok %u exceeds the context %u", pos, ntok, c->context);
        return MKV_ERR_CAPACITY;
    }
    if (first_pos > pos) {
        set_error("first_pos %u > pos %u: token 0 would see no key", first_pos, pos);
        return MKV_ERR_INVALID;
    }
    const uint32_t shard_end = c->ring ? c->context : c->shard_first + c->capacity;
    if (c->ring && partial) {
        set_error("a ring cache is not sharded");
        return MKV_ERR_UNSUPPORTED;
    }
    if (!partial && !c->whole) {
        set_error("this cache is the shard [%u, %u) of a context of %u: use mkv_attn_verify_partial", c->shard_first, shard_end,
                  c->context);
        return MKV_ERR_INVALID;
    }
    // rows that must be valid: the visible ones held here
    const uint32_t need = (uint32_t)std::min<uint64_t>(end, shard_end);
    if (need > c->shard_first && c->len < need) {
        set_error("reads rows up to %u but only %u are valid (appended or restored)", need, c->len);
        return MKV_ERR_STATE;
    }
    const uint32_t T = c->fmt == MKV_F16 ? TILE : TILE32;
    const uint32_t lo = std::max(first_pos, c->shard_first);
    const uint32_t hi = (uint32_t)std::min<uint64_t>(end, shard_end);
    memset(it, 0, sizeof *it);
    it->kmap = c->maps_dev + 2 * layer;
    it->vmap = c->maps_dev + 2 * layer + 1;
    it->q = q;
    it->out = out;
    it->first_pos = first_pos;
    it->pos = pos;
    it->ntok = ntok;
    it->row0 = c->shard_first;
    it->key_lo = c->shard_first;
    it->key_hi = shard_end;
    it->ring = c->ring;
    it->partial = partial ? 1u : 0u;
    it->phase = measure_phase();
    it->safe_below = c->safe_below(pos);
    if (hi > lo) {
        it->tile_begin = lo / T;
        it->tile_end = (hi + T - 1) / T;
    } else {
        it->tile_begin = it->tile_end = 0;
    }
    return MKV_OK;
}

// Scratch regions per item, after planning.
static mkv_status place_scratch(Cache *const *caches, VerifyItem *items, int n) {
    // items of the same cache share its scratch; lay them out one after the other
    for (int i = 0; i < n; i++) {
        size_t before = 0;
        for (int j = 0; j < i; j++)
            if (caches[j] == caches[i]) before += 2u * (size_t)items[j].nsplit;
        size_t total = before;
        for (int j = i; j < n; j++)
            if (caches[j] == caches[i]) total += 2u * (size_t)items[j].nsplit;
        bool first = true;
        for (int j = 0; j < i; j++)
            if (caches[j] == caches[i]) first = false;
        if (first) {
            mkv_status st = ensure_scratch(caches[i], total);
            if (st != MKV_OK) return st;
        }
        items[i].part_ml = caches[i]->part_ml + before * 32 * 2;
        items[i].part_o = caches[i]->part_o + before * 32 * 256;
    }
    return MKV_OK;
}

// Window and sinks on a filled item: the key range shrinks to what token 0 still sees; on a ring cache every visible
// key and every row of the step must own its row.
static mkv_status apply_window(Cache *c, VerifyItem *it, uint32_t window, const float *sinks) {
    it->win = window;
    it->sinks = sinks;
    const uint32_t T = c->fmt == MKV_F16 ? TILE : TILE32;
    const uint32_t lo = lowest_key(*it, 0), hi = it->pos + it->ntok;
    if (c->ring && hi - lo > c->ring) {
        set_error("keys [%u, %u) do not fit a ring of %u rows: pass a window of at most %u", lo, hi, c->ring, c->ring - it->ntok + 1u);
        return MKV_ERR_CAPACITY;
    }
    it->tile_begin = lo / T;
    it->tile_end = (hi + T - 1) / T;
    return MKV_OK;
}

static mkv_status verify_common(Cache *c, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok, const float *q,
                                float *out, bool partial) {
    VerifyItem it;
    mkv_status st = fill_item(c, layer, first_pos, pos, ntok, q, out, partial, &it);
    if (st != MKV_OK) return st;
    if (c->ring && (st = apply_window(c, &it, 0, nullptr)) != MKV_OK) return st;
    if ((st = use_device(c->ctx)) != MKV_OK) return st;
    plan_items(c->ctx, &it, 1);
    Cache *cc[1] = {c};
    if ((st = place_scratch(cc, &it, 1)) != MKV_OK) return st;
    return launch_verify(c->ctx, c->fmt, &it, 1, false, &c->maps_host[2 * layer], &c->maps_host[2 * layer + 1]);
}

} // namespace mkv

using namespace mkv;

extern "C" {

const char *mkv_strerror(mkv_status s) {
    switch (s) {
    case MKV_OK: return "ok";
    case MKV_ERR_INVALID: return "invalid argument";
    case MKV_ERR_CAPACITY: return "position outside the cache";
    case MKV_ERR_CUDA: return "CUDA error";
    case MKV_ERR_NOMEM: return "out of memory";
    case MKV_ERR_UNSUPPORTED: return "not supported";
    case MKV_ERR_STATE: return "rows not valid";
    case MKV_ERR_FORMAT: return "format mismatch";
    case MKV_ERR_IO: return "I/O error";
    }
    return "unknown status";
}

const char *mkv_last_error(void) { return g_err; }
const char *mkv_version(void) { return "mechta-kv 0.1 sm_100a"; }

mkv_status mkv_ctx_create(int device, void *stream, mkv_ctx **out) {
    if (!out) {
        set_error("null out");
        return MKV_ERR_INVALID;
    }
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        set_error("no CUDA device: this library has no CPU path");
        return MKV_ERR_CUDA;
    }
    if (device < 0 || device >= ndev) {
        set_error("device %d outside [0, %d)", device, ndev);
        return MKV_ERR_INVALID;
    }
    MKV_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    MKV_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        set_error("device %d is sm_%d%d; this library is built for sm_100a only", device, prop.major, prop.minor);
        return MKV_ERR_UNSUPPORTED;
    }
    Ctx *ctx = new (std::nothrow) Ctx();
    if (!ctx) return MKV_ERR_NOMEM;
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    {
        const char *e = getenv("MKV_PDL");
        ctx->pdl = !(e && e[0] == '0');
    }
    ctx->stream = (cudaStream_t)stream; // NULL = the legacy default stream
    MKV_CUDA(cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    MKV_CUDA(cudaEventCreateWithFlags(&ctx->ev_compute, cudaEventDisableTiming));
    MKV_CUDA(cudaEventCreateWithFlags(&ctx->ev_copy, cudaEventDisableTiming));
    MKV_CUDA(cudaMalloc(&ctx->dev_status, 4));
    MKV_CUDA(cudaMemset(ctx->dev_status, 0, 4));
    const size_t ring = sizeof(VerifyItem) * (size_t)Ctx::SLOTS * Ctx::SLOT_ITEMS;
    MKV_CUDA(cudaMalloc(&ctx->items_dev, ring));
    MKV_CUDA(cudaHostAlloc(&ctx->items_host, ring, cudaHostAllocDefault));
    for (int i = 0; i < Ctx::SLOTS; i++) MKV_CUDA(cudaEventCreateWithFlags(&ctx->slot_done[i], cudaEventDisableTiming));
    MKV_CUDA(cudaMalloc(&ctx->counters_dev, sizeof(uint32_t) * Ctx::SLOT_ITEMS));
    MKV_CUDA(cudaMemset(ctx->counters_dev, 0, sizeof(uint32_t) * Ctx::SLOT_ITEMS));
    ctx->counter_base.assign(Ctx::SLOT_ITEMS, 0u);
    mkv_status st = verify_setup_device();
    if (st == MKV_OK) st = prefill_setup_device();
    if (st == MKV_OK) st = prefill_tc_setup_device();
    if (st == MKV_OK) st = append_setup_device();
    if (st != MKV_OK) return st;
    *out = reinterpret_cast<mkv_ctx *>(ctx);
    return MKV_OK;
}

static void ctx_free(Ctx *ctx) {
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->copy_stream);
    for (auto &p : ctx->prof_events) {
        cudaEventDestroy(p.first);
        cudaEventDestroy(p.second);
    }
    for (int i = 0; i < Ctx::SLOTS; i++)
        if (ctx->slot_done[i]) cudaEventDestroy(ctx->slot_done[i]);
    if (ctx->items_dev) cudaFree(ctx->items_dev);
    if (ctx->counters_dev) cudaFree(ctx->counters_dev);
    if (ctx->items_host) cudaFreeHost(ctx->items_host);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->pf_scratch) cudaFree(ctx->pf_scratch);
    if (ctx->pf_counters) cudaFree(ctx->pf_counters);
    if (ctx->ev_compute) cudaEventDestroy(ctx->ev_compute);
    if (ctx->ev_copy) cudaEventDestroy(ctx->ev_copy);
    if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
    delete ctx;
}

void mkv_ctx_destroy(mkv_ctx *h) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx || ctx->closing) return;
    if (ctx->live_caches > 0) { // freed when its last cache goes
        ctx->closing = true;
        return;
    }
    ctx_free(ctx);
}

mkv_status mkv_sync(mkv_ctx *h) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx) {
        set_error("null ctx");
        return MKV_ERR_INVALID;
    }
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    MKV_CUDA(cudaStreamSynchronize(ctx->stream));
    MKV_CUDA(cudaStreamSynchronize(ctx->copy_stream));
    ctx->syncs++;
    return check_device_status(ctx);
}

uint64_t mkv_launch_count(const mkv_ctx *h) { return h ? reinterpret_cast<const Ctx *>(h)->launches : 0; }

mkv_status mkv_prof_enable(mkv_ctx *h, int on) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx) return MKV_ERR_INVALID;
    ctx->prof = on != 0;
    ctx->prof_used = 0;
    if (on > 0) { // pre-create event pairs so that none is created inside a timed region
        mkv_status st = use_device(ctx);
        if (st != MKV_OK) return st;
        while (ctx->prof_events.size() < (size_t)on) {
            cudaEvent_t a, b;
            MKV_CUDA(cudaEventCreate(&a));
            MKV_CUDA(cudaEventCreate(&b));
            ctx->prof_events.push_back({a, b});
        }
    }
    return MKV_OK;
}

mkv_status mkv_prof_read(mkv_ctx *h, double *core_ms, uint64_t *core_launches) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx || !core_ms || !core_launches) return MKV_ERR_INVALID;
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    double ms = 0.0;
    if (ctx->prof_used > 0) MKV_CUDA(cudaEventSynchronize(ctx->prof_events[ctx->prof_used - 1].second));
    for (size_t i = 0; i < ctx->prof_used; i++) {
        float t = 0.f;
        MKV_CUDA(cudaEventElapsedTime(&t, ctx->prof_events[i].first, ctx->prof_events[i].second));
        ms += t;
    }
    *core_ms = ms;
    *core_launches = ctx->prof_used;
    ctx->prof_used = 0;
    return MKV_OK;
}

uint64_t mkv_need_bytes(uint32_t ctx_tokens, mkv_fmt fmt, int n_layers) {
    // M/engine.rs:63-67 buffer_bytes_for and M/memcheck.rs:15-18
    const uint64_t ctx = ctx_tokens;
    const uint64_t buf = 4ull * (fmt == MKV_F32 ? ctx * 512ull : ctx * 512ull / 2ull);
    const uint64_t kv = 2ull * (uint64_t)n_layers * buf;
    const uint64_t a = 8ull * (ctx / 64ull), b = 64ull * (ctx / 2048ull);
    const uint64_t partials = 4ull * 258ull * 16ull * (2ull * (ctx / 128ull) + std::max(a, b));
    return kv + partials;
}

static mkv_status cache_create_common(mkv_ctx *h, mkv_fmt fmt, int n_layers, uint32_t context, uint32_t shard_first,
                                      uint32_t shard_tokens, uint32_t ring, mkv_cache **out) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx || !out || ctx->closing) {
        set_error("null argument");
        return MKV_ERR_INVALID;
    }
    *out = nullptr;
    if (fmt != MKV_F16 && fmt != MKV_F32) {
        set_error("unknown format %d", (int)fmt);
        return MKV_ERR_INVALID;
    }
    if (n_layers < 1 || n_layers > 256) {
        set_error("n_layers %d outside [1, 256]", n_layers);
        return MKV_ERR_INVALID;
    }
    // M/engine.rs:28-33 check_ctx
    if (context % 1024 != 0 || context < MKV_CTX_MIN || context > MKV_CTX_MAX) {
        set_error("context %u: must be a multiple of 1024 between %d and %d", context, MKV_CTX_MIN, MKV_CTX_MAX);
        return MKV_ERR_INVALID;
    }
    if (ring && (ring % 128u != 0 || ring < 1024u || ring > context)) {
        set_error("ring of %u rows: must be a multiple of 128, at least 1024 and at most the context %u", ring, context);
        return MKV_ERR_INVALID;
    }
    const bool whole = shard_tokens == 0;
    const uint32_t capacity = ring ? ring : (whole ? context : shard_tokens);
    if (whole ? shard_first != 0
              : (capacity % 64 != 0 || shard_first % 64 != 0 || (uint64_t)shard_first + capacity > (uint64_t)context)) {
        set_error("shard [%u, +%u): first row and size must be multiples of 64 inside the context %u", shard_first,
                  shard_tokens, context);
        return MKV_ERR_INVALID;
    }
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    Cache *c = new (std::nothrow) Cache();
    if (!c) return MKV_ERR_NOMEM;
    c->ctx = ctx;
    c->fmt = fmt;
    c->n_layers = n_layers;
    c->context = context;
    c->capacity = capacity;
    c->ring = ring;
    c->shard_first = shard_first;
    c->whole = whole;
    ctx->live_caches++;
    c->elem = fmt == MKV_F16 ? 2 : 4;
    c->buf_bytes = (size_t)capacity * ROW * c->elem;
    c->k.assign(n_layers, nullptr);
    c->v.assign(n_layers, nullptr);
    auto fail = [&](mkv_status s) {
        mkv_cache_destroy(reinterpret_cast<mkv_cache *>(c));
        return s;
    };
    for (int l = 0; l < n_layers; l++) {
        if (guard_malloc(c, &c->k[l], c->buf_bytes) != cudaSuccess || guard_malloc(c, &c->v[l], c->buf_bytes) != cudaSuccess) {
            cudaGetLastError();
            set_error("out of device memory for layer %d of %d (%zu bytes per buffer)", l, n_layers, c->buf_bytes);
            return fail(MKV_ERR_NOMEM);
        }
        if (cudaMemsetAsync(c->k[l], 0, c->buf_bytes, ctx->stream) != cudaSuccess ||
            cudaMemsetAsync(c->v[l], 0, c->buf_bytes, ctx->stream) != cudaSuccess) {
            set_error("cudaMemsetAsync failed");
            return fail(MKV_ERR_CUDA);
        }
    }
    // two sets of tensor maps per layer: boxes of the verify tile, then boxes of the prefill tile
    std::vector<CUtensorMap> &maps = c->maps_host;
    maps.resize(4 * (size_t)n_layers);
    const uint32_t box_rows = fmt == MKV_F16 ? TILE : TILE32;
    const uint32_t pf_rows = fmt == MKV_F16 ? PF_TILE : TILE32;
    for (int l = 0; l < n_layers; l++) {
        if ((st = make_tensor_map(&maps[2 * l], fmt, c->k[l], capacity, box_rows)) != MKV_OK) return fail(st);
        if ((st = make_tensor_map(&maps[2 * l + 1], fmt, c->v[l], capacity, box_rows)) != MKV_OK) return fail(st);
        if ((st = make_tensor_map(&maps[2 * (n_layers + l)], fmt, c->k[l], capacity, pf_rows)) != MKV_OK) return fail(st);
        if ((st = make_tensor_map(&maps[2 * (n_layers + l) + 1], fmt, c->v[l], capacity, pf_rows)) != MKV_OK) return fail(st);
    }
    if (cudaMalloc(&c->maps_dev, maps.size() * sizeof(CUtensorMap)) != cudaSuccess ||
        cudaMalloc(&c->kptrs_dev, n_layers * sizeof(void *)) != cudaSuccess ||
        cudaMalloc(&c->vptrs_dev, n_layers * sizeof(void *)) != cudaSuccess) {
        cudaGetLastError();
        set_error("out of device memory for the cache tables");
        return fail(MKV_ERR_NOMEM);
    }
    if (cudaMemcpy(c->maps_dev, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(c->kptrs_dev, c->k.data(), n_layers * sizeof(void *), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(c->vptrs_dev, c->v.data(), n_layers * sizeof(void *), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaEventCreateWithFlags(&c->ev_snapshot, cudaEventDisableTiming) != cudaSuccess) {
        set_error("setting up the cache tables failed: %s", cudaGetErrorString(cudaGetLastError()));
        return fail(MKV_ERR_CUDA);
    }
    if ((st = ensure_scratch(c, 2u * (size_t)ctx->sm_count)) != MKV_OK) return fail(st);
    if (cudaMalloc(&c->qr, (size_t)MKV_MAX_VERIFY * 16 * 256 * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        set_error("out of device memory for the query scratch");
        return fail(MKV_ERR_NOMEM);
    }
    *out = reinterpret_cast<mkv_cache *>(c);
    return MKV_OK;
}

mkv_status mkv_cache_create(mkv_ctx *h, mkv_fmt fmt, int n_layers, uint32_t context, uint32_t shard_first,
                            uint32_t shard_tokens, mkv_cache **out) {
    return cache_create_common(h, fmt, n_layers, context, shard_first, shard_tokens, 0, out);
}

mkv_status mkv_cache_create_ring(mkv_ctx *h, mkv_fmt fmt, int n_layers, uint32_t context, uint32_t ring_rows, mkv_cache **out) {
    if (ring_rows == 0) {
        set_error("ring_rows must not be 0");
        return MKV_ERR_INVALID;
    }
    return cache_create_common(h, fmt, n_layers, context, 0, 0, ring_rows, out);
}

int mkv_checks_enabled(void) {
#ifdef MKV_CHECKS
    return 1;
#else
    return 0;
#endif
}

mkv_status mkv_cache_check_guards(mkv_cache *h, uint64_t *bad_bytes) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || !bad_bytes) {
        set_error("null cache or result pointer");
        return MKV_ERR_INVALID;
    }
    *bad_bytes = 0;
#ifdef MKV_CHECKS
    mkv_status st = use_device(c->ctx);
    if (st != MKV_OK) return st;
    MKV_CUDA(cudaStreamSynchronize(c->ctx->stream));
    MKV_CUDA(cudaStreamSynchronize(c->ctx->copy_stream));
    std::vector<unsigned char> host(2 * GUARD);
    for (const auto &g : c->guarded) {
        char *p = static_cast<char *>(g.first);
        MKV_CUDA(cudaMemcpy(host.data(), p - GUARD, GUARD, cudaMemcpyDeviceToHost));
        MKV_CUDA(cudaMemcpy(host.data() + GUARD, p + g.second, GUARD, cudaMemcpyDeviceToHost));
        for (unsigned char b : host) *bad_bytes += b != CANARY;
    }
#endif
    return MKV_OK;
}

mkv_status mkv_checks_touch_guard(mkv_cache *h) {
#ifdef MKV_CHECKS
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || c->guarded.empty()) {
        set_error("no guarded buffer");
        return MKV_ERR_INVALID;
    }
    mkv_status st = use_device(c->ctx);
    if (st != MKV_OK) return st;
    MKV_CUDA(cudaMemset(static_cast<char *>(c->guarded[0].first) + c->guarded[0].second + 7, 0, 3));
    return MKV_OK;
#else
    (void)h;
    set_error("not a checked build");
    return MKV_ERR_UNSUPPORTED;
#endif
}

void mkv_cache_destroy(mkv_cache *h) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c) return;
    cudaSetDevice(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    cudaStreamSynchronize(c->ctx->copy_stream);
    for (void *p : c->k) guard_free(c, p);
    for (void *p : c->v) guard_free(c, p);
    if (c->maps_dev) cudaFree(c->maps_dev);
    if (c->kptrs_dev) cudaFree(c->kptrs_dev);
    if (c->vptrs_dev) cudaFree(c->vptrs_dev);
    guard_free(c, c->part_ml);
    guard_free(c, c->part_o);
    if (c->qr) cudaFree(c->qr);
    if (c->ev_snapshot) cudaEventDestroy(c->ev_snapshot);
    Ctx *ctx = c->ctx;
    delete c;
    if (--ctx->live_caches == 0 && ctx->closing) ctx_free(ctx);
}

mkv_status mkv_cache_buffers(mkv_cache *h, int layer, void **k_dev, void **v_dev) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || layer < 0 || layer >= c->n_layers) {
        set_error("bad cache or layer");
        return MKV_ERR_INVALID;
    }
    if (k_dev) *k_dev = c->k[layer];
    if (v_dev) *v_dev = c->v[layer];
    return MKV_OK;
}

uint32_t mkv_cache_len(const mkv_cache *h) { return h ? reinterpret_cast<const Cache *>(h)->len : 0; }

mkv_status mkv_cache_set_len(mkv_cache *h, uint32_t len) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c) return MKV_ERR_INVALID;
    const uint32_t end = c->ring ? c->context : c->shard_first + c->capacity; // a ring's rows are reused by later positions
    if (len > end) {
        set_error("length %u beyond the end of the cache %u", len, end);
        return MKV_ERR_CAPACITY;
    }
    c->len = len;
    c->note_write(0); // the host wrote the buffers itself
    return MKV_OK;
}

uint64_t mkv_cache_device_bytes(const mkv_cache *h) {
    const Cache *c = reinterpret_cast<const Cache *>(h);
    if (!c) return 0;
    return 2ull * c->n_layers * c->buf_bytes + c->scratch_pieces * 32ull * 258ull * 4ull +
           2ull * c->n_layers * (sizeof(CUtensorMap) + sizeof(void *));
}

void mkv_rope_table(int32_t pos, uint32_t ntok, float *out) {
    // M/engine.rs:108-114: iterative theta, f32 libm
    const float scale = powf(1e7f, -2.0f / 64.0f);
    for (uint32_t t = 0; t < ntok; t++) {
        float th = (float)(pos + (int32_t)t);
        float *o = out + (size_t)t * 64;
        for (int i = 0; i < 32; i++) {
            o[i] = cosf(th);
            o[32 + i] = sinf(th);
            th *= scale;
        }
    }
}

// which: 1 = the K rows only, 2 = the V rows only, 3 = both. The rows count as valid once their V half is written
// (the reference dispatches the K writer, then the V writer, M/quad.rs:116-117).
static mkv_status append_common(Cache *c, int layer0, int n_layers, uint32_t pos, uint32_t ntok, const float *k,
                                const float *v, const float *tab, uint32_t which = 3u) {
    if (!c || !k || !v) {
        set_error("null argument");
        return MKV_ERR_INVALID;
    }
    if (ntok < 1 || ntok > (uint32_t)MKV_CTX_MAX) {
        set_error("ntok %u outside [1, %d]", ntok, MKV_CTX_MAX);
        return MKV_ERR_INVALID;
    }
    if (((uintptr_t)k & 15u) || ((uintptr_t)v & 15u) || ((uintptr_t)tab & 15u)) {
        set_error("k, v and the rope table must be 16-byte aligned");
        return MKV_ERR_INVALID;
    }
    const uint64_t end = (uint64_t)pos + ntok;
    const uint32_t shard_end = c->shard_first + c->capacity;
    if (end > (uint64_t)c->context) {
        set_error("rows [%u, %u) do not fit the context of %u rows", pos, (uint32_t)end, c->context);
        return MKV_ERR_CAPACITY;
    }
    if (c->ring && ntok > c->ring) {
        set_error("a ring cache of %u rows cannot take %u rows in one call", c->ring, ntok);
        return MKV_ERR_CAPACITY;
    }
    {
        // rows between the valid length and pos that this cache holds would become valid without ever having been written
        const uint32_t gap_lo = c->ring ? c->len : std::max(c->len, c->shard_first);
        const uint32_t gap_hi = c->ring ? pos : std::min(pos, shard_end);
        if (gap_hi > gap_lo) {
            set_error("rows up to %u are valid, an append at %u would leave a gap (mkv_cache_set_len declares rows the host wrote itself)",
                      c->len, pos);
            return MKV_ERR_STATE;
        }
    }
    mkv_status st = use_device(c->ctx);
    if (st != MKV_OK) return st;
    st = launch_append(c->ctx, c->fmt, c->kptrs_dev + layer0, c->vptrs_dev + layer0, n_layers, (size_t)ntok * ROW,
                       c->shard_first, c->capacity, c->ring, pos, ntok, k, v, tab, which);
    if (st != MKV_OK) return st;
    if (which & 2u) {
        c->len = c->ring ? (uint32_t)end : (uint32_t)std::min<uint64_t>(end, shard_end);
        if (c->len < c->shard_first) c->len = c->shard_first;
    }
    c->note_write(pos);
    return MKV_OK;
}

mkv_status mkv_append(mkv_cache *h, int layer, uint32_t pos, uint32_t ntok, const float *k, const float *v, const float *tab) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || layer < 0 || layer >= c->n_layers) {
        set_error("bad cache or layer %d", layer);
        return MKV_ERR_INVALID;
    }
    return append_common(c, layer, 1, pos, ntok, k, v, tab);
}

mkv_status mkv_append_layers(mkv_cache *h, uint32_t pos, uint32_t ntok, const float *k, const float *v, const float *tab) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c) {
        set_error("null cache");
        return MKV_ERR_INVALID;
    }
    return append_common(c, 0, c->n_layers, pos, ntok, k, v, tab);
}

mkv_status mkv_truncate(mkv_cache *h, uint32_t new_len, int scrub) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c) {
        set_error("null cache");
        return MKV_ERR_INVALID;
    }
    if (new_len > c->len) {
        set_error("cannot truncate to %u: only %u rows are valid", new_len, c->len);
        return MKV_ERR_STATE;
    }
    if (scrub && c->ring) {
        set_error("a ring cache has no scrub: its rows are reused by later positions");
        return MKV_ERR_UNSUPPORTED;
    }
    const uint32_t old = c->len;
    c->len = std::max(new_len, std::min(c->shard_first, old));
    if (scrub && old > c->len) {
        c->note_write(0);
        mkv_status st = use_device(c->ctx);
        if (st != MKV_OK) return st;
        const size_t off = (size_t)(c->len - c->shard_first) * ROW * c->elem;
        const size_t nb = (size_t)(old - c->len) * ROW * c->elem;
        for (int l = 0; l < c->n_layers; l++) {
            MKV_CUDA(cudaMemsetAsync((char *)c->k[l] + off, 0, nb, c->ctx->stream));
            MKV_CUDA(cudaMemsetAsync((char *)c->v[l] + off, 0, nb, c->ctx->stream));
        }
    }
    return MKV_OK;
}

mkv_status mkv_attn_verify(mkv_cache *h, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok, const float *q, float *out) {
    return verify_common(reinterpret_cast<Cache *>(h), layer, first_pos, pos, ntok, q, out, false);
}

mkv_status mkv_attn_verify_window(mkv_cache *h, int layer, uint32_t window, const float *sinks, uint32_t pos, uint32_t ntok,
                                  const float *q, float *out) {
    Cache *c = reinterpret_cast<Cache *>(h);
    VerifyItem it;
    mkv_status st = fill_item(c, layer, 0, pos, ntok, q, out, false, &it);
    if (st != MKV_OK) return st;
    if ((st = apply_window(c, &it, window, sinks)) != MKV_OK) return st;
    if ((st = use_device(c->ctx)) != MKV_OK) return st;
    plan_items(c->ctx, &it, 1);
    Cache *cc[1] = {c};
    if ((st = place_scratch(cc, &it, 1)) != MKV_OK) return st;
    return launch_verify(c->ctx, c->fmt, &it, 1, false, &c->maps_host[2 * layer], &c->maps_host[2 * layer + 1]);
}

mkv_status mkv_attn_step(mkv_cache *h, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok, const mkv_step_in *in,
                         float *ag, void *ag16) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || !in) {
        set_error("null cache or inputs");
        return MKV_ERR_INVALID;
    }
    if (!in->qf_dev || !in->kb_dev || !in->vb_dev || !in->q_norm_dev || !in->k_norm_dev || !in->rope_tab_dev || (!ag && !ag16)) {
        set_error("mkv_attn_step needs qf, kb, vb, both norm weights, the rope table and at least one output");
        return MKV_ERR_INVALID;
    }
    if (((uintptr_t)in->qf_dev & 15u) || ((uintptr_t)ag & 15u) || ((uintptr_t)ag16 & 7u)) {
        set_error("qf and ag must be 16-byte aligned, ag16 8-byte aligned");
        return MKV_ERR_INVALID;
    }
    if (!c->whole) {
        set_error("mkv_attn_step works on an unsharded cache: the gate follows the merge of all shards");
        return MKV_ERR_UNSUPPORTED;
    }
    if (!(in->eps > 0.0f)) {
        set_error("eps must be positive");
        return MKV_ERR_INVALID;
    }
    // the same checks as an append of these rows followed by a verify over them
    VerifyItem it;
    const uint32_t len_before = c->len;
    const uint64_t end = (uint64_t)pos + ntok;
    if (layer < 0 || layer >= c->n_layers || ntok < 1 || ntok > MKV_MAX_VERIFY || end > (uint64_t)c->context) {
        set_error("layer %d, rows [%u, %llu) outside the cache (layers %d, context %u, at most %d rows a step)", layer, pos,
                  (unsigned long long)end, c->n_layers, c->context, MKV_MAX_VERIFY);
        return end > (uint64_t)c->context ? MKV_ERR_CAPACITY : MKV_ERR_INVALID;
    }
    if (c->len < pos) {
        set_error("rows up to %u are valid, the step would leave a gap before %u", c->len, pos);
        return MKV_ERR_STATE;
    }
    c->len = (uint32_t)end; // the rows this call writes count as valid for its own attention
    c->note_write(pos); // (a note that outlives a failed call only makes later launches more careful)
    // Everything that can refuse the call comes before the first launch; the length goes back on every failure.
    // fill_item wants an output pointer for its checks; the f16 one serves when there is no f32 output
    mkv_status st = fill_item(c, layer, first_pos, pos, ntok, c->qr, ag ? ag : static_cast<float *>(ag16), false, &it);
    // a ring cache holds only the last `ring` positions: the keys of the step must fit it (as in mkv_attn_verify)
    if (st == MKV_OK && c->ring) st = apply_window(c, &it, 0, nullptr);
    if (st == MKV_OK) st = use_device(c->ctx);
    Cache *cc[1] = {c};
    if (st == MKV_OK) {
        plan_items(c->ctx, &it, 1);
        st = place_scratch(cc, &it, 1);
    }
    it.out = ag;
    it.gate = in->qf_dev;
    it.out16 = ag16;
    if (st == MKV_OK)
        st = launch_step_prep(c->ctx, c->fmt, in->qf_dev, in->kb_dev, in->vb_dev, in->q_norm_dev, in->k_norm_dev,
                              in->rope_tab_dev, in->eps, c->qr, c->k[layer], c->v[layer], c->shard_first, c->capacity, c->ring, pos,
                              ntok);
    if (st != MKV_OK) { // nothing was written: the rows of the step are not valid
        c->len = len_before;
        return st;
    }
    return launch_verify(c->ctx, c->fmt, &it, 1, false, &c->maps_host[2 * layer], &c->maps_host[2 * layer + 1]);
}

mkv_status mkv_attn_verify_partial(mkv_cache *h, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok, const float *q,
                                   float *rec) {
    return verify_common(reinterpret_cast<Cache *>(h), layer, first_pos, pos, ntok, q, rec, true);
}

mkv_status mkv_combine_shards(mkv_ctx *h, const float *recs, int n_shards, uint32_t ntok, float *out) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx || !recs || !out || n_shards < 1 || ntok < 1 || ntok > MKV_MAX_VERIFY) {
        set_error("bad argument to mkv_combine_shards");
        return MKV_ERR_INVALID;
    }
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    return launch_combine_shards(ctx, recs, n_shards, ntok, out);
}

// ---- peer exchange of shard records (one process per GPU, CUDA IPC) ----------------------------------------------

mkv_status mkv_exchange_create(mkv_ctx *h, int rank, int world, mkv_exchange **out) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx || !out || world < 1 || world > MAX_PEERS || rank < 0 || rank >= world) {
        set_error("mkv_exchange_create: 1 <= world <= %d and 0 <= rank < world", MAX_PEERS);
        return MKV_ERR_INVALID;
    }
    *out = nullptr;
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    Exchange *ex = new (std::nothrow) Exchange();
    if (!ex) return MKV_ERR_NOMEM;
    ex->ctx = ctx;
    ex->rank = rank;
    ex->world = world;
    ex->mailbox_bytes = 2u * (size_t)world * SLOT_WORDS * sizeof(unsigned long long);
    if (cudaMalloc(&ex->mailbox, ex->mailbox_bytes) != cudaSuccess || cudaMalloc(&ex->push_dev, sizeof(PushInfo)) != cudaSuccess) {
        cudaGetLastError();
        set_error("out of device memory for the exchange mailbox");
        delete ex;
        return MKV_ERR_NOMEM;
    }
    MKV_CUDA(cudaMemset(ex->mailbox, 0, ex->mailbox_bytes));
    *out = reinterpret_cast<mkv_exchange *>(ex);
    return MKV_OK;
}

mkv_status mkv_exchange_handle(mkv_exchange *h, void *handle_out) {
    Exchange *ex = reinterpret_cast<Exchange *>(h);
    if (!ex || !handle_out) return MKV_ERR_INVALID;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    mkv_status st = use_device(ex->ctx);
    if (st != MKV_OK) return st;
    cudaIpcMemHandle_t hd;
    MKV_CUDA(cudaIpcGetMemHandle(&hd, ex->mailbox));
    memcpy(handle_out, &hd, sizeof hd);
    return MKV_OK;
}

mkv_status mkv_exchange_connect(mkv_exchange *h, const void *handles) {
    Exchange *ex = reinterpret_cast<Exchange *>(h);
    if (!ex || !handles || ex->connected) {
        set_error("mkv_exchange_connect: null argument or already connected");
        return MKV_ERR_INVALID;
    }
    mkv_status st = use_device(ex->ctx);
    if (st != MKV_OK) return st;
    for (int d = 0; d < ex->world; d++) {
        if (d == ex->rank) {
            ex->peer_base[d] = ex->mailbox;
            continue;
        }
        cudaIpcMemHandle_t hd;
        memcpy(&hd, static_cast<const char *>(handles) + 64 * (size_t)d, sizeof hd);
        bool absent = true; // an all-zero handle = a rank that never joined: nothing is sent to it, its flag never comes
        for (size_t i = 0; i < sizeof hd; i++) absent &= reinterpret_cast<const unsigned char *>(&hd)[i] == 0;
        if (absent) {
            ex->peer_base[d] = nullptr;
            continue;
        }
        MKV_CUDA(cudaIpcOpenMemHandle(&ex->peer_base[d], hd, cudaIpcMemLazyEnablePeerAccess));
    }
    PushInfo pi;
    memset(&pi, 0, sizeof pi);
    pi.world = (uint32_t)ex->world;
    for (int p = 0; p < 2; p++) {
        pi.inbox[p] = reinterpret_cast<const unsigned long long *>(ex->mailbox) + (size_t)p * ex->world * SLOT_WORDS;
        for (int d = 0; d < ex->world; d++) {
            unsigned char *base = static_cast<unsigned char *>(ex->peer_base[d]);
            if (!base) continue;
            pi.slot[p][d] = reinterpret_cast<unsigned long long *>(base) + ((size_t)p * ex->world + ex->rank) * SLOT_WORDS;
        }
    }
    MKV_CUDA(cudaMemcpy(ex->push_dev, &pi, sizeof pi, cudaMemcpyHostToDevice));
    ex->connected = true;
    return MKV_OK;
}

void mkv_exchange_destroy(mkv_exchange *h) {
    Exchange *ex = reinterpret_cast<Exchange *>(h);
    if (!ex) return;
    cudaSetDevice(ex->ctx->device);
    cudaStreamSynchronize(ex->ctx->stream);
    for (int d = 0; d < ex->world; d++)
        if (ex->connected && d != ex->rank && ex->peer_base[d]) cudaIpcCloseMemHandle(ex->peer_base[d]);
    if (ex->mailbox) cudaFree(ex->mailbox);
    if (ex->push_dev) cudaFree(ex->push_dev);
    delete ex;
}

mkv_status mkv_attn_verify_exchange(mkv_cache *hc, mkv_exchange *hx, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                                    const float *q, float *out) {
    Cache *c = reinterpret_cast<Cache *>(hc);
    Exchange *ex = reinterpret_cast<Exchange *>(hx);
    if (!c || !ex || !ex->connected || ex->ctx != c->ctx) {
        set_error("mkv_attn_verify_exchange: cache and connected exchange of one context needed");
        return MKV_ERR_INVALID;
    }
    if ((uintptr_t)out & 15u) {
        set_error("out must be 16-byte aligned");
        return MKV_ERR_INVALID;
    }
    VerifyItem it;
    // partial mode: the merged rows are this shard's record; they go to the mailboxes and `out` gets the merge of all ranks
    mkv_status st = fill_item(c, layer, first_pos, pos, ntok, q, out, true, &it);
    if (st != MKV_OK) return st;
    if ((st = use_device(c->ctx)) != MKV_OK) return st;
    plan_items(c->ctx, &it, 1);
    Cache *cc[1] = {c};
    if ((st = place_scratch(cc, &it, 1)) != MKV_OK) return st;
    if (++ex->epoch == 0u) ++ex->epoch; // never 0: a cleared mailbox must not look like a delivery
    const uint32_t epoch = ex->epoch;   // every rank makes the same calls, so the call number agrees everywhere
    it.push = ex->push_dev;
    it.push_world = (uint32_t)ex->world;
    it.push_epoch = epoch;
    return launch_verify(c->ctx, c->fmt, &it, 1, false, &c->maps_host[2 * layer], &c->maps_host[2 * layer + 1]);
}

mkv_status mkv_attn_verify_batch(mkv_ctx *h, const mkv_verify_item *items, int n) {
    Ctx *ctx = reinterpret_cast<Ctx *>(h);
    if (!ctx || !items || n < 1 || n > Ctx::SLOT_ITEMS) {
        set_error("bad argument to mkv_attn_verify_batch (1 <= n <= %d)", Ctx::SLOT_ITEMS);
        return MKV_ERR_INVALID;
    }
    std::vector<VerifyItem> its((size_t)n);
    std::vector<Cache *> caches((size_t)n);
    mkv_fmt fmt = MKV_F16;
    for (int i = 0; i < n; i++) {
        Cache *c = reinterpret_cast<Cache *>(items[i].cache);
        if (!c || c->ctx != ctx) {
            set_error("item %d: cache missing or of another context", i);
            return MKV_ERR_INVALID;
        }
        if (i == 0) fmt = c->fmt;
        else if (c->fmt != fmt) {
            set_error("item %d: all caches of a batch must have one format", i);
            return MKV_ERR_INVALID;
        }
        mkv_status st = fill_item(c, items[i].layer, items[i].first_pos, items[i].pos, items[i].ntok, items[i].q_dev,
                                  items[i].out_dev, false, &its[i]);
        if (st != MKV_OK) return st;
        if (c->ring && (st = apply_window(c, &its[i], 0, nullptr)) != MKV_OK) return st;
        caches[i] = c;
    }
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    plan_items(ctx, its.data(), n);
    if ((st = place_scratch(caches.data(), its.data(), n)) != MKV_OK) return st;
    return launch_verify(ctx, fmt, its.data(), n, true, nullptr, nullptr);
}

mkv_status mkv_attn_prefill(mkv_cache *h, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok, const void *qv,
                            int q_is_f16, float *out) {
    const float *q = static_cast<const float *>(qv);
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || !q || !out || layer < 0 || layer >= c->n_layers) {
        set_error("bad argument to mkv_attn_prefill");
        return MKV_ERR_INVALID;
    }
    if (c->ring) {
        set_error("not available on a ring cache");
        return MKV_ERR_UNSUPPORTED;
    }
    if (ntok < 1 || ntok > 4096) {
        set_error("ntok %u outside [1, 4096]", ntok);
        return MKV_ERR_INVALID;
    }
    if (((uintptr_t)q & 15u) || ((uintptr_t)out & 15u)) {
        set_error("q and out must be 16-byte aligned");
        return MKV_ERR_INVALID;
    }
    if (!c->whole) {
        set_error("prefill attention runs on unsharded caches");
        return MKV_ERR_UNSUPPORTED;
    }
    const uint64_t end = (uint64_t)pos0 + ntok;
    if (end > c->capacity) {
        set_error("rows [%u, %u) do not fit the cache of %u rows", pos0, (uint32_t)end, c->capacity);
        return MKV_ERR_CAPACITY;
    }
    if (first_pos > pos0) {
        set_error("first_pos %u > pos0 %u", first_pos, pos0);
        return MKV_ERR_INVALID;
    }
    if (c->len < end) {
        set_error("reads rows up to %u but only %u are valid: append the block first", (uint32_t)end, c->len);
        return MKV_ERR_STATE;
    }
    mkv_status st = use_device(c->ctx);
    if (st != MKV_OK) return st;
    if (c->fmt == MKV_F16) {
        // MKV_PREFILL=mma selects the warp-MMA kernel (kept as the measured baseline of the tcgen05 kernel)
        static const bool use_mma = [] { const char *e = getenv("MKV_PREFILL"); return e && strcmp(e, "mma") == 0; }();
        if (use_mma && q_is_f16) {
            set_error("the warp-MMA baseline kernel (MKV_PREFILL=mma) takes f32 queries only");
            return MKV_ERR_UNSUPPORTED;
        }
        return use_mma ? launch_prefill_f16_mma(c->ctx, c, layer, first_pos, pos0, ntok, q, out)
                       : launch_prefill_f16_tc(c->ctx, c, layer, first_pos, pos0, ntok, qv, q_is_f16 != 0, out);
    }
    if (q_is_f16) {
        set_error("f16 queries go with the f16 cache (q_f16 + attn_fa_mx); the f32 cache's attn_fa / attn_fd4 read f32 queries");
        return MKV_ERR_UNSUPPORTED;
    }
    // f32 cache: groups of up to 4 tokens through the f32 verify kernel (the reference's attn_fd4 also reads
    // K/V once per 4 tokens, W/ops.wgsl:694-699), one ragged batch per <= SLOT_ITEMS groups
    uint32_t done = 0;
    while (done < ntok) {
        const uint32_t left = ntok - done;
        const int groups = (int)std::min<uint32_t>((left + 3) / 4, Ctx::SLOT_ITEMS);
        std::vector<VerifyItem> its((size_t)groups);
        std::vector<Cache *> caches((size_t)groups, c);
        for (int g = 0; g < groups; g++) {
            const uint32_t t = done + 4u * g;
            const uint32_t nt = std::min<uint32_t>(4, ntok - t);
            st = fill_item(c, layer, first_pos, pos0 + t, nt, q + (size_t)t * 4096, out + (size_t)t * 4096, false, &its[g]);
            if (st != MKV_OK) return st;
        }
        plan_items(c->ctx, its.data(), groups);
        if ((st = place_scratch(caches.data(), its.data(), groups)) != MKV_OK) return st;
        if ((st = launch_verify(c->ctx, c->fmt, its.data(), groups, true, nullptr, nullptr)) != MKV_OK) return st;
        done += 4u * groups;
    }
    return MKV_OK;
}

// ---- snapshot / restore -------------------------------------------------------------------------------------

// rows of [0, p) this cache holds: [r0, r1) in global positions
static void held_rows(const Cache *c, uint32_t p, uint32_t *r0, uint32_t *r1) {
    const uint32_t end = c->shard_first + c->capacity;
    *r0 = std::min(c->shard_first, p);
    *r1 = std::min(p, end);
    if (*r1 < *r0) *r1 = *r0;
}

size_t mkv_snapshot_bytes(const mkv_cache *h, uint32_t p) {
    const Cache *c = reinterpret_cast<const Cache *>(h);
    if (!c) return 0;
    uint32_t r0, r1;
    held_rows(c, p, &r0, &r1);
    return 2ull * c->n_layers * (size_t)(r1 - r0) * ROW * c->elem;
}

mkv_status mkv_snapshot(mkv_cache *h, uint32_t p, void *dst, size_t cap, size_t *written) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || (!dst && mkv_snapshot_bytes(h, p) != 0)) {
        set_error("null argument");
        return MKV_ERR_INVALID;
    }
    if (c->ring) {
        set_error("not available on a ring cache");
        return MKV_ERR_UNSUPPORTED;
    }
    {
        const uint32_t upto = std::min(p, c->shard_first + c->capacity); // the rows of [0, p) held here
        if (upto > c->shard_first && upto > c->len) {
            set_error("snapshot of %u rows but only %u are valid", p, c->len);
            return MKV_ERR_STATE;
        }
    }
    const size_t need = mkv_snapshot_bytes(h, p);
    if (cap < need) {
        set_error("snapshot needs %zu bytes, buffer has %zu", need, cap);
        return MKV_ERR_INVALID;
    }
    Ctx *ctx = c->ctx;
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    uint32_t r0, r1;
    held_rows(c, p, &r0, &r1);
    const size_t nb = (size_t)(r1 - r0) * ROW * c->elem;
    const size_t off = (size_t)(r0 - c->shard_first) * ROW * c->elem;
    // the copies start after what is already enqueued on the compute stream
    MKV_CUDA(cudaEventRecord(ctx->ev_compute, ctx->stream));
    MKV_CUDA(cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_compute, 0));
    char *d = static_cast<char *>(dst);
    if (nb > 0)
        for (int l = 0; l < c->n_layers; l++) {
            MKV_CUDA(cudaMemcpyAsync(d, (const char *)c->k[l] + off, nb, cudaMemcpyDeviceToHost, ctx->copy_stream));
            d += nb;
            MKV_CUDA(cudaMemcpyAsync(d, (const char *)c->v[l] + off, nb, cudaMemcpyDeviceToHost, ctx->copy_stream));
            d += nb;
        }
    MKV_CUDA(cudaEventRecord(c->ev_snapshot, ctx->copy_stream));
    c->snapshot_pending = true;
    // later appends must not overwrite rows still being copied out
    MKV_CUDA(cudaEventRecord(ctx->ev_copy, ctx->copy_stream));
    MKV_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_copy, 0));
    if (written) *written = need;
    return MKV_OK;
}

mkv_status mkv_snapshot_wait(mkv_cache *h) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c) return MKV_ERR_INVALID;
    if (c->snapshot_pending) {
        mkv_status st = use_device(c->ctx);
        if (st != MKV_OK) return st;
        MKV_CUDA(cudaEventSynchronize(c->ev_snapshot));
        c->snapshot_pending = false;
    }
    return MKV_OK;
}

mkv_status mkv_restore(mkv_cache *h, uint32_t p, const void *src, size_t bytes) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || (!src && bytes != 0)) {
        set_error("null argument");
        return MKV_ERR_INVALID;
    }
    if (c->ring) {
        set_error("not available on a ring cache");
        return MKV_ERR_UNSUPPORTED;
    }
    const uint32_t end = c->shard_first + c->capacity;
    if (p > c->context) {
        set_error("restore of %u rows into a context of %u", p, c->context);
        return MKV_ERR_CAPACITY;
    }
    (void)end;
    const size_t need = mkv_snapshot_bytes(h, p);
    if (bytes != need) {
        set_error("restore payload is %zu bytes, %u rows of this cache are %zu", bytes, p, need);
        return MKV_ERR_FORMAT;
    }
    Ctx *ctx = c->ctx;
    mkv_status st = use_device(ctx);
    if (st != MKV_OK) return st;
    uint32_t r0, r1;
    held_rows(c, p, &r0, &r1);
    const size_t nb = (size_t)(r1 - r0) * ROW * c->elem;
    const size_t off = (size_t)(r0 - c->shard_first) * ROW * c->elem;
    MKV_CUDA(cudaEventRecord(ctx->ev_compute, ctx->stream));
    MKV_CUDA(cudaStreamWaitEvent(ctx->copy_stream, ctx->ev_compute, 0));
    const char *s = static_cast<const char *>(src);
    if (nb > 0)
        for (int l = 0; l < c->n_layers; l++) {
            MKV_CUDA(cudaMemcpyAsync((char *)c->k[l] + off, s, nb, cudaMemcpyHostToDevice, ctx->copy_stream));
            s += nb;
            MKV_CUDA(cudaMemcpyAsync((char *)c->v[l] + off, s, nb, cudaMemcpyHostToDevice, ctx->copy_stream));
            s += nb;
        }
    MKV_CUDA(cudaEventRecord(ctx->ev_copy, ctx->copy_stream));
    MKV_CUDA(cudaStreamWaitEvent(ctx->stream, ctx->ev_copy, 0));
    c->len = std::max(r1, std::min(c->shard_first, p));
    c->note_write(0);
    return MKV_OK;
}

mkv_status mkv_host_alloc(size_t bytes, void **out) {
    if (!out) return MKV_ERR_INVALID;
    *out = nullptr;
    if (cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        set_error("cudaHostAlloc of %zu bytes failed", bytes);
        return MKV_ERR_NOMEM;
    }
    return MKV_OK;
}

void mkv_host_free(void *p) {
    if (p) cudaFreeHost(p);
}

// ---- the reference's dispatch form --------------------------------------------------------------------------

mkv_status mkv_dispatch(mkv_cache *h, int layer, const char *op, const uint32_t u[8], const void *in0, const void *in1,
                        void *out) {
    Cache *c = reinterpret_cast<Cache *>(h);
    if (!c || !op || !u) {
        set_error("null argument");
        return MKV_ERR_INVALID;
    }
    const bool f16 = c->fmt == MKV_F16;
    auto is = [&](const char *a) { return strcmp(op, a) == 0; };
    // P{n, rows, f0, f1, step_a, step_o, flag, extra} (W/ops.wgsl:4)
    const uint32_t n = u[0], rows = u[1], f0 = u[2], f1 = u[3], step_a = u[4], step_o = u[5], flag = u[6], extra = u[7];
    float scale;
    memcpy(&scale, &f0, 4);
    if (is("kv_rope") || is("kv_rope2") || is("rope") || is("rope2")) {
        const bool compact = op[0] == 'k';
        if (compact != f16) {
            set_error("%s is the writer of the %s cache (M/engine.rs:100-105)", op, compact ? "f16" : "f32");
            return MKV_ERR_INVALID;
        }
        if (n != 256 || step_a != 256 || step_o != 256 || extra % 512 != 0 || rows % 2 != 0 || rows == 0) {
            set_error("%s: only the KV writer form [256, 2*ntok, 0,0, 256,256, flag, pos*512] is built", op);
            return MKV_ERR_UNSUPPORTED;
        }
        const bool multi = is("kv_rope2") || is("rope2");
        if (multi ? flag != 2 : rows != 2) {
            set_error("%s: rows per token must be 2", op);
            return MKV_ERR_UNSUPPORTED;
        }
        const uint32_t ntok = rows / 2, pos = extra / 512;
        if (!in0 || !in1 || layer < 0 || layer >= c->n_layers) {
            set_error("%s: missing binding or bad layer", op);
            return MKV_ERR_INVALID;
        }
        // the K rows only; the rows become valid with the V writer that follows (M/quad.rs:116-117)
        return append_common(c, layer, 1, pos, ntok, (const float *)in0, (const float *)in0, (const float *)in1, 1u);
    }
    if (is("kv_copy") || is("copy")) {
        const bool compact = op[0] == 'k';
        if (compact != f16) {
            set_error("%s is the writer of the %s cache (M/engine.rs:100-105)", op, compact ? "f16" : "f32");
            return MKV_ERR_INVALID;
        }
        if (n == 0 || n % 512 != 0 || extra % 512 != 0) {
            set_error("%s: only whole positions are written (n and extra multiples of 512)", op);
            return MKV_ERR_UNSUPPORTED;
        }
        const uint32_t ntok = n / 512, pos = extra / 512;
        if (!in0 || layer < 0 || layer >= c->n_layers) {
            set_error("%s: missing binding or bad layer", op);
            return MKV_ERR_INVALID;
        }
        return append_common(c, layer, 1, pos, ntok, (const float *)in0, (const float *)in0, nullptr, 2u);
    }
    if (is("q_dmx") || is("attn_fd_combine")) return MKV_OK; // fused into the attention entry
    if (is("q_f16")) {
        // W/fa_mx.wgsl:313-319: n packed words = 2 n values, qr f32 -> qh f16 (the input of attn_fa_mx)
        if (!in0 || !out || n == 0 || ((uintptr_t)in0 & 15u) || ((uintptr_t)out & 15u) || n % 4u != 0) {
            set_error("q_f16: in0 = qr (f32), out = qh (f16), both 16-byte aligned, n a multiple of 4 words");
            return MKV_ERR_INVALID;
        }
        mkv_status st = use_device(c->ctx);
        if (st != MKV_OK) return st;
        return launch_q_f16(c->ctx, (const float *)in0, out, n);
    }
    if (is("attn_fa_mx") || is("attn_fa") || is("attn_fd4") || (is("attn_fd") && step_o > 4u)) {
        // The prefill forms (uniforms of M/engine.rs:915-927, dispatch list M/engine.rs:1215-1241): tokens
        // [step_a, step_a + T) of the block that starts at position n - 1, T = 64 for attn_fa_mx / attn_fa (one
        // dispatch per split of chunks: the call for the first chunk, step_o = 0, does all chunks and the others are
        // no-ops, as is the attn_fd_combine that follows), 8 for attn_fd4, step_o for attn_fd in its batch mode.
        // in0 = qh (f16) for attn_fa_mx, qr (f32) otherwise, the whole block's [nb][4096]; out = att [nb][4096].
        if (fabsf(scale - SCALE) > 0.f) {
            set_error("%s: scale %g, only 1/16 is built", op, scale);
            return MKV_ERR_UNSUPPORTED;
        }
        const bool fa = is("attn_fa_mx") || is("attn_fa"), mx = is("attn_fa_mx");
        if (mx && !f16) {
            set_error("attn_fa_mx runs on the f16 cache only (M/engine.rs:1215)");
            return MKV_ERR_INVALID;
        }
        if (fa && step_o != 0u) return MKV_OK; // a later split of the same group
        const uint32_t T = fa ? 64u : (is("attn_fd4") ? 8u : step_o);
        if (n == 0 || !in0 || !out) return MKV_ERR_INVALID;
        const size_t qoff = (size_t)step_a * 4096u;
        const void *qg = mx ? (const void *)((const __half *)in0 + qoff) : (const void *)((const float *)in0 + qoff);
        return mkv_attn_prefill(h, layer, extra, n - 1u + step_a, T, qg, mx ? 1 : 0, (float *)out + qoff);
    }
    if (is("attn_dmx1") || is("attn_dmx2") || is("attn_fd") || is("attn_fd2h")) {
        if (fabsf(scale - SCALE) > 0.f) {
            set_error("%s: scale %g, only 1/16 is built", op, scale);
            return MKV_ERR_UNSUPPORTED;
        }
        uint32_t ntok, first = extra;
        if (is("attn_dmx1") || is("attn_dmx2")) {
            ntok = f1; // uniform [pos+1, chunks, scale, ntok, 0, 0, chunk, 0] (M/quad.rs:286)
            if (!f16) {
                set_error("%s runs on the f16 cache only (M/dmx.rs:2)", op);
                return MKV_ERR_INVALID;
            }
            if (ntok < 1 || ntok > (is("attn_dmx1") ? 2u : 4u)) return MKV_ERR_INVALID;
        } else if (is("attn_fd2h")) {
            ntok = 2;
        } else {
            ntok = step_o > 0 ? step_o : 1; // decode: one token per grid z; here one call per token group
        }
        (void)rows;
        (void)step_a;
        (void)flag;
        if (n == 0) return MKV_ERR_INVALID;
        return mkv_attn_verify(h, layer, first, n - 1, ntok, (const float *)in0, (float *)out);
    }
    set_error("dispatch of '%s' is outside the KV path", op);
    return MKV_ERR_UNSUPPORTED;
}

} // extern "C"
