/* mechta_kv.h — C ABI of the B200 KV-cache / attention path that stands in for the KV operators of
 * ssomenzi/mechta (reference paths below: M/ = engine/crates/mechta/src/, W/ = M/wgsl/).
 *
 * The reference has no FFI for this path: its boundary is a fixed set of compute dispatches over named
 * buffers with an 8-word uniform P{n, rows, f0, f1, step_a, step_o, flag, extra} (W/ops.wgsl:4). Each entry
 * point below replaces one group of those dispatches and says which. A Rust `-sys` crate binds exactly
 * these symbols; mkv_dispatch() additionally accepts the reference's own (kernel name, uniform) form.
 *
 * Conventions
 *  - Every call returns an mkv_status; nothing aborts. mkv_last_error() gives the text of the last failure
 *    on the calling thread.
 *  - One mkv_ctx = one CUDA device + the caller's compute stream (+ a copy stream of its own). Calls on a ctx come from one
 *    host thread at a time (the reference engine is single-threaded, engine/crates/api/src/lib.rs:46) and are
 *    stream-ordered: they return once the work is enqueued, except where "blocks" is written.
 *  - Pointers named *_dev are device pointers on the ctx's device, borrowed for the call; *_host are host
 *    pointers (pinned memory makes the copies asynchronous).
 *  - Shapes are the reference's: 16 query heads, 2 KV heads, head_dim 256, scale 1/16; one cache position is
 *    512 elements of K and 512 of V, element (pos, kvh, d) at pos*512 + kvh*256 + d (W/ops.wgsl:165).
 *  - Positions are global token positions. A cache may hold only a contiguous shard [shard_first,
 *    shard_first + capacity) of the sequence (sequence sharding over several GPUs, one process each).
 *  - There is no CPU fallback: without a usable CUDA device every compute call fails with MKV_ERR_CUDA.
 */
#ifndef MECHTA_KV_H
#define MECHTA_KV_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct mkv_ctx mkv_ctx;
typedef struct mkv_cache mkv_cache;

typedef enum {
    MKV_OK = 0,
    MKV_ERR_INVALID = 1,     /* bad argument (null, ntok out of range, misaligned pointer, unknown op) */
    MKV_ERR_CAPACITY = 2,    /* position range outside the cache (the reference asserts pos + K < ctx, M/quad.rs:278) */
    MKV_ERR_CUDA = 3,        /* a CUDA call failed or no device */
    MKV_ERR_NOMEM = 4,       /* device or host allocation failed */
    MKV_ERR_UNSUPPORTED = 5, /* valid in the reference but not built here */
    MKV_ERR_STATE = 6,       /* reads rows that were never appended or were rolled back */
    MKV_ERR_FORMAT = 7,      /* snapshot / root file does not match the cache */
    MKV_ERR_IO = 8           /* file system error (root files) */
} mkv_status;

/* M/engine.rs:49-68 KvFormat */
typedef enum { MKV_F16 = 0, MKV_F32 = 1 } mkv_fmt;

enum {
    MKV_HQ = 16, MKV_HKV = 2, MKV_D = 256, MKV_GROUP = 8, MKV_ROW = 512,
    MKV_MAX_VERIFY = 4,      /* K of M/quad.rs: tokens per verify step */
    MKV_REC = 258,           /* one partial record [m, l, acc[256]] (W/ops.wgsl:389-391, M/dmx.rs:111) */
    MKV_CTX_MIN = 4096, MKV_CTX_MAX = 262144 /* M/engine.rs:24-25 */
};

const char *mkv_strerror(mkv_status s);
const char *mkv_last_error(void);
/* "mechta-kv <version> sm_100a" */
const char *mkv_version(void);

/* ---- context ------------------------------------------------------------------------------------------
 * Replaces gpu::Gpu's device/queue for this path (engine/crates/gpu/src/lib.rs:60-139). `stream` is a
 * cudaStream_t to run on (borrowed; e.g. the caller's current stream); NULL is the legacy default stream. */
mkv_status mkv_ctx_create(int device, void *stream, mkv_ctx **out);
void mkv_ctx_destroy(mkv_ctx *ctx);
/* blocks until everything enqueued on both streams has finished */
mkv_status mkv_sync(mkv_ctx *ctx);
/* number of this library's kernels launched on the ctx since creation (for launch accounting) */
uint64_t mkv_launch_count(const mkv_ctx *ctx);
/* Kernel timing with CUDA events on the compute stream, off by default. While on, every attention core
 * kernel (verify / prefill) is bracketed by two events; mkv_prof_read blocks on the last one and returns
 * the summed milliseconds and the number of launches since the last read, then clears them. Mirrors the
 * reference's per-dispatch GPU timestamps of "attn.core" (M/engine.rs:1274-1295). on = 0 switches it off;
 * on > 0 switches it on and creates that many event pairs ahead of time (more are created as needed). */
mkv_status mkv_prof_enable(mkv_ctx *ctx, int on);
mkv_status mkv_prof_read(mkv_ctx *ctx, double *core_ms, uint64_t *core_launches);

/* ---- cache --------------------------------------------------------------------------------------------
 * Replaces the per-layer buffers kc[il], vc[il] (M/engine.rs:493-494,602-603): n_layers x (K, V), each
 * [capacity][2][256] of f16 or f32, zero-filled (wgpu zero-initialises; the tail tile of the attention
 * reads rows past the valid length and masks them, M/dmx.rs:53,60-64).
 * context_tokens: the sequence's context, by the reference's rule a multiple of 1024 in [4096, 262144]
 * (M/engine.rs:28-33). shard_tokens = 0: this cache holds the whole context (shard_first must be 0). Otherwise
 * it holds the rows [shard_first, shard_first + shard_tokens) only, both multiples of 64 (one shard of a
 * sequence-sharded context; appends of other rows are skipped, attention goes through the _partial entry).
 * A ctx destroyed before its caches stays alive until the last of them is destroyed. */
mkv_status mkv_cache_create(mkv_ctx *ctx, mkv_fmt fmt, int n_layers, uint32_t context_tokens,
                            uint32_t shard_first, uint32_t shard_tokens, mkv_cache **out);
void mkv_cache_destroy(mkv_cache *c);
/* device pointers of a layer's K and V buffers (for tests and for hosts that fill the cache themselves) */
mkv_status mkv_cache_buffers(mkv_cache *c, int layer, void **k_dev, void **v_dev);
/* rows currently valid: the global position after the last appended row (0 when empty) */
uint32_t mkv_cache_len(const mkv_cache *c);
/* declare rows [.., len) valid without appending (after the host filled the buffers itself, or restore) */
mkv_status mkv_cache_set_len(mkv_cache *c, uint32_t len);
/* M/memcheck.rs:14-20 need_bytes minus its fixed part: K and V of n_layers + the reference's partials */
uint64_t mkv_need_bytes(uint32_t ctx_tokens, mkv_fmt fmt, int n_layers);
/* bytes this library allocates on the device for such a cache (buffers + its own split-K scratch) */
uint64_t mkv_cache_device_bytes(const mkv_cache *c);

/* ---- append: replaces kv_rope2 / kv_rope + kv_copy (W/kv.wgsl:19-42) and rope2 / rope + copy
 * (W/ops.wgsl:141-162,275-286), dispatched at M/quad.rs:116-117, M/engine.rs:1213-1214.
 * k_dev = `kn` f32 [ntok][2][256] (after the K RMSNorm), v_dev = `vb` f32 [ntok][512],
 * rope_tab_dev = f32 [ntok][64] = [cos 0..31 | sin 0..31] per token (mkv_rope_table), or NULL when K is
 * already rotated. Token t goes to global position pos + t; rows outside this cache's shard are skipped.
 * Afterwards the valid length is pos + ntok (rows beyond it, e.g. refused drafts, are forgotten).
 * pos may not lie beyond the valid length: rows in between would count as valid without having been written
 * (MKV_ERR_STATE; a host that fills rows itself declares them with mkv_cache_set_len first).
 * Products and the sum/difference of the rotation are rounded separately (no FMA); f16 stores round to
 * nearest even. 1 <= ntok, pos + ntok <= context. */
mkv_status mkv_append(mkv_cache *c, int layer, uint32_t pos, uint32_t ntok, const float *k_dev,
                      const float *v_dev, const float *rope_tab_dev);
/* the same for every layer in one launch: k_dev/v_dev/rope as above with a leading [n_layers] axis on
 * k and v (the table is shared by the layers) */
mkv_status mkv_append_layers(mkv_cache *c, uint32_t pos, uint32_t ntok, const float *k_dev,
                             const float *v_dev, const float *rope_tab_dev);
/* M/engine.rs:108-114 rope_table, on the host: out[ntok][64] for positions pos..pos+ntok-1 */
void mkv_rope_table(int32_t pos, uint32_t ntok, float *out_host);

/* ---- rollback: the reference has no kernel for it; the session simply continues at a smaller pos
 * (M/session.rs:385-411, M/engine.rs:703-705). new_len <= current length. Rows >= new_len stay in memory
 * until overwritten and are never visible to later reads. scrub != 0 also zeroes them (deterministic
 * snapshots of the whole buffer). */
mkv_status mkv_truncate(mkv_cache *c, uint32_t new_len, int scrub);

/* ---- decode / verify attention: replaces q_dmx + attn_dmx1/attn_dmx2 + attn_fd_combine (M/dmx.rs:19-141,
 * M/quad.rs:122-124) for the f16 cache, and attn_fd / attn_fd2h + attn_fd_combine (W/ops.wgsl:325-538,
 * M/quad.rs:129-130, M/engine.rs:133-142) for the f32 cache and the MTP window.
 * q_dev = `qr` f32 [ntok][16][256] after RoPE; out_dev = `att` f32 [ntok][16][256]. Token t (at pos + t) sees
 * keys first_pos <= key < pos + 1 + t, which includes the rows this step appended. 1 <= ntok <= 4.
 * Requires pos + ntok <= valid length and an unsharded cache. */
mkv_status mkv_attn_verify(mkv_cache *c, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                           const float *q_dev, float *out_dev);

/* Sequence-sharded form. Each shard computes, over the keys it holds, the un-normalised record
 * rec_dev = f32 [64][258], row = tok*16 + head, [M, tot, acc[256]] — the reference's partial format
 * (W/ops.wgsl:389-391) with one record per row; rows that see no key here get M = -3e38, tot = 0.
 * Records of all shards are gathered by the host (NCCL all-gather) and merged by mkv_combine_shards,
 * which is attn_fd_combine's arithmetic (W/ops.wgsl:529-537) over shards instead of blocks. */
mkv_status mkv_attn_verify_partial(mkv_cache *c, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                                   const float *q_dev, float *rec_dev);
mkv_status mkv_combine_shards(mkv_ctx *ctx, const float *recs_dev /*[n_shards][64][258]*/, int n_shards,
                              uint32_t ntok, float *out_dev /*[ntok][16][256]*/);

/* The same exchange without a collective library and without a second kernel: the CTAs of the attention kernel that
 * merge its split-K pieces store each row of the rank's record straight into every rank's mailbox over NVLink (plain
 * peer stores, no multicast; every value as one 8-byte word that also carries the call number, so a value that shows the
 * current call number is the value: no flag and no fence behind the data), wait (bounded) for the same row of every
 * other rank in their own mailbox and write the merged row: one launch per layer. One process per GPU; the mailboxes
 * are shared by CUDA IPC:
 *   mkv_exchange_create on every rank -> mkv_exchange_handle (64 bytes) -> the host gathers the handles of all ranks
 *   in rank order -> mkv_exchange_connect(handles[world][64]).
 * Every rank then makes the same sequence of mkv_attn_verify_exchange calls (same layer, positions and q): the call
 * number is the epoch the words carry. out_dev = f32 [ntok][16][256], final (merged over all shards) on every rank.
 * A rank whose handle is all zeroes counts as absent: nothing is sent to it, and since its rows never arrive the
 * bounded wait of the merging CTAs (about two seconds) runs out; the output is then left untouched and mkv_sync
 * reports MKV_ERR_CUDA (status word), after which the context is usable again. out_dev must be 16-byte aligned.
 * No counterpart in the reference (one GPU); the arithmetic is attn_fd_combine's (W/ops.wgsl:529-537). */
typedef struct mkv_exchange mkv_exchange;
mkv_status mkv_exchange_create(mkv_ctx *ctx, int rank, int world, mkv_exchange **out);
mkv_status mkv_exchange_handle(mkv_exchange *ex, void *handle_out_64_bytes);
mkv_status mkv_exchange_connect(mkv_exchange *ex, const void *handles /*[world][64] bytes, rank order*/);
void mkv_exchange_destroy(mkv_exchange *ex);
mkv_status mkv_attn_verify_exchange(mkv_cache *c, mkv_exchange *ex, int layer, uint32_t first_pos, uint32_t pos,
                                    uint32_t ntok, const float *q_dev, float *out_dev);

/* Verify attention without any allocation by the library. No counterpart in the reference (which allocates
 * all its buffers once at start-up, M/engine.rs:204-252): this is for hosts that cannot let a library call
 * cudaMalloc — all device memory already belongs to their own planner, or the call comes from a place where
 * allocating is not allowed. Same result as mkv_attn_verify on an f16 cache, but the caller owns the cache:
 * k_dev / v_dev are f16 buffers [capacity_tokens][2][256] (16-byte aligned), q_dev / out_dev f32 [ntok][16][256],
 * `stream` a cudaStream_t (NULL = legacy default stream), `device` the CUDA device all of them live on.
 * The split-K pieces go to a fixed array inside the library image (5,284,096 bytes on every GPU that loads
 * the library, held until the process exits) with room for 160 pieces = one CTA per SM up to 160 SMs; a launch
 * that would need more fails with MKV_ERR_CAPACITY. The first call on a device looks up the array's device
 * address, opts the kernel into its shared memory and clears the header (a blocking cudaMemset): make that
 * first call before any stream capture begins. All calls share the array, which keeps the previous call's
 * contents (the counter is cleared on the stream before each launch): calls whose kernels may overlap on the
 * GPU, e.g. on two streams, race on it. Calls cudaMalloc / cudaFree nowhere.
 * Rows of the caller's buffers past pos + ntok need not be initialised: the kernel reads up to the next multiple
 * of 64 rows but zeroes the V rows no token sees before it uses the tile, and masked scores are replaced, so a
 * NaN or infinity left there does not reach the output. The caller's current CUDA device is the same after the
 * call as before it. The entry point has no context object; it may be called from several host threads (its
 * once-per-device set-up is guarded by a mutex), but calls that overlap on the GPU still share the one array.
 * Every wait inside the kernel is bounded; one that runs out sets a status word in the array instead of hanging:
 * mkv_static_status waits for `stream` (blocks), returns the word in *status_out and clears it; a non-zero word
 * also makes it return MKV_ERR_CUDA, and the outputs of the calls since the last check are then not valid. */
mkv_status mkv_attn_verify_static(int device, void *stream, const void *k_dev, const void *v_dev,
                                  uint32_t capacity_tokens, uint32_t first_pos, uint32_t pos, uint32_t ntok,
                                  const float *q_dev, float *out_dev);
mkv_status mkv_static_status(int device, void *stream, uint32_t *status_out);

/* Ragged batch: n independent (cache, layer, position) verify steps in one launch pair; every cache must
 * belong to `ctx`. Each item behaves exactly as one mkv_attn_verify call. */
typedef struct {
    mkv_cache *cache;
    int32_t layer;
    uint32_t first_pos, pos, ntok;
    const float *q_dev; /* [ntok][16][256] */
    float *out_dev;     /* [ntok][16][256] */
} mkv_verify_item;
mkv_status mkv_attn_verify_batch(mkv_ctx *ctx, const mkv_verify_item *items, int n);

/* Cache variants of the reference's second model (engine/crates/mechta/src/flint.rs:22-26,
 * wgsl/flint_attn.wgsl:1-8), as options of the same kernels:
 *  - ring cache: `ring_rows` rows per layer, position p lives in row p % ring_rows (flint_attn.wgsl:3,54,79), for
 *    layers that only ever look back a window; ring_rows a multiple of 128, >= 1024. Appends, mkv_attn_step and the
 *    verify calls work on it as long as the keys a call sees plus the rows of its step fit the ring; snapshots,
 *    prefill and shards do not.
 *  - sliding window: token t of a step at `pos` sees keys pos + t - window < key <= pos + t (flint.rs:22-23,
 *    flint_attn.wgsl:82; window 513 there); 0 = no window.
 *  - attention sinks: `sinks_dev` [16], one logit per query head that joins the softmax's maximum and sum and
 *    never the output (flint_attn.wgsl:243-255, as ggml's soft_max with sinks); NULL = none.
 * mkv_attn_verify_window works on ring and on ordinary (unsharded) caches. */
mkv_status mkv_cache_create_ring(mkv_ctx *ctx, mkv_fmt fmt, int n_layers, uint32_t context_tokens, uint32_t ring_rows,
                                 mkv_cache **out);
mkv_status mkv_attn_verify_window(mkv_cache *c, int layer, uint32_t window, const float *sinks_dev, uint32_t pos,
                                  uint32_t ntok, const float *q_dev, float *out_dev);

/* The layer's whole step around the KV path in two launches. Replaces, for the ntok rows of a step, the nine
 * dispatches of engine/crates/mechta/src/quad.rs:113-125: rmsnorm of the query heads and of the key heads
 * (wgsl/ops.wgsl:27-56 with attn_q_norm / attn_k_norm), rope2 of the queries (ops.wgsl:275-286), kv_rope2 and
 * kv_copy into the cache (wgsl/kv.wgsl:19-42), q_dmx, attn_dmx2 or attn_fd, attn_fd_combine, and attn_gate /
 * attn_gate16 (ops.wgsl:171-177, 295-300). Rows [pos, pos + ntok) of the layer are written exactly as mkv_append
 * would write the normalised keys; the result is the gated attention output. Unsharded caches only. */
typedef struct {
    const float *qf_dev;       /* [ntok][16][512]: per head 256 query values, then 256 gate values (output of attn_q) */
    const float *kb_dev;       /* [ntok][2][256]: output of attn_k, before its norm */
    const float *vb_dev;       /* [ntok][512]: output of attn_v */
    const float *q_norm_dev;   /* [256] attn_q_norm.weight */
    const float *k_norm_dev;   /* [256] attn_k_norm.weight */
    const float *rope_tab_dev; /* [ntok][64] as mkv_rope_table */
    float eps;                 /* 1e-6 in the reference (engine.rs:12) */
} mkv_step_in;
/* ag_dev: [ntok][16][256] f32 (attn_gate), ag16_dev: the same values as f16 (attn_gate16); either may be NULL. */
mkv_status mkv_attn_step(mkv_cache *c, int layer, uint32_t first_pos, uint32_t pos, uint32_t ntok, const mkv_step_in *in,
                         float *ag_dev, void *ag16_dev);

/* ---- prefill attention over the cache: replaces q_f16 + attn_fa_mx + attn_fd_combine (W/fa_mx.wgsl:19-115,
 * 313-319), attn_fa and attn_fd4 (W/ops.wgsl:562-651,711-778), dispatched at M/engine.rs:1215-1241.
 * The block's K/V must already be appended (the reference appends all rows first, M/engine.rs:1213-1214).
 * q_dev [ntok][16][256]: f32 (`qr`, q_is_f16 = 0) or f16 (`qh`, the output of the reference's q_f16 pass,
 * q_is_f16 = 1; f16 cache only, as attn_fa_mx); token T sees keys first_pos <= key < pos0 + 1 + T;
 * out f32 [ntok][16][256]. 1 <= ntok <= 4096. */
mkv_status mkv_attn_prefill(mkv_cache *c, int layer, uint32_t first_pos, uint32_t pos0, uint32_t ntok,
                            const void *q_dev, int q_is_f16, float *out_dev);

/* ---- snapshot / restore of the prefix cache ("root"): replaces the KV part of Engine::read_root /
 * write_root (M/engine.rs:782-823). Payload = for each layer in order, K rows [0,p) then V rows [0,p), raw
 * cache bytes (f16 bit patterns or f32), i.e. Root.kv flattened. A shard copies only the rows it holds; its
 * payload then covers [max(0,shard_first), min(p, shard_first+capacity)).
 * The copies run on the ctx's copy stream after the work already enqueued on the compute stream; with pinned
 * host memory the call returns at once. Compute enqueued later waits for a restore; mkv_snapshot_wait blocks
 * until the last snapshot has landed in host memory. */
size_t mkv_snapshot_bytes(const mkv_cache *c, uint32_t p);
mkv_status mkv_snapshot(mkv_cache *c, uint32_t p, void *dst_host, size_t cap, size_t *written);
mkv_status mkv_snapshot_wait(mkv_cache *c);
/* afterwards the valid length is p (on a shard: min(p, end of shard)) */
mkv_status mkv_restore(mkv_cache *c, uint32_t p, const void *src_host, size_t bytes);
/* pinned host staging, so hosts without their own CUDA binding get asynchronous copies */
mkv_status mkv_host_alloc(size_t bytes, void **out);
void mkv_host_free(void *p);

/* ---- the checked build (make -C mechta_b200/csrc checks: libmechta_kv_checks.so, -DMKV_CHECKS). The reference relies
 * on wgpu's bounds checks on every buffer access (engine/crates/shader/src/lib.rs:13-22 keeps them on); here every
 * buffer of a cache (K and V rows of each layer, the split-K pieces) is allocated between two 64 KB runs of a canary
 * byte, and mkv_cache_check_guards counts the canary bytes that changed (blocks on the context's streams).
 * mkv_checks_enabled: 1 in the checked build, 0 in the shipped one, whose check finds nothing to look at and reports 0.
 * mkv_checks_touch_guard: checked build only, for the test of the check itself: overwrites three canary bytes from
 * the host side (a cudaMemset inside the library's own allocation). */
int mkv_checks_enabled(void);
mkv_status mkv_cache_check_guards(mkv_cache *c, uint64_t *bad_bytes);
mkv_status mkv_checks_touch_guard(mkv_cache *c);

/* ---- root files: the KV section of the reference's on-disk prefix cache, "MECHTA-ROOT-1\n"
 * (M/session.rs:92-129): u64 p, u64 n_ssm, u64 n_kv, p x u32 tokens, then length-prefixed f32-word vectors
 * ssm.., conv.., (K, V)... Files written here carry n_ssm = 0; files with DeltaNet states are read and the
 * states skipped. payload = mkv_snapshot's layout. Blocks (host I/O only). */
mkv_status mkv_root_write(const char *path, mkv_fmt fmt, int n_layers, uint32_t p, const uint32_t *tokens,
                          const void *payload_host, size_t payload_bytes);
mkv_status mkv_root_read(const char *path, mkv_fmt fmt, int n_layers, uint32_t *p_out, uint32_t *tokens_out,
                         size_t tokens_cap, void *payload_host, size_t payload_cap, size_t *payload_bytes);
/* M/session.rs:61-66 root_key: FNV-1a 64 of the token ids */
uint64_t mkv_root_key(const uint32_t *tokens, size_t n);

/* ---- the reference's own dispatch form ------------------------------------------------------------------
 * op = the WGSL entry point name, u = its 8-word uniform, in0/in1 = bindings 0 and 1 (device), out = the
 * output binding (device; ignored by the cache writers). Supported: "kv_rope", "kv_rope2", "rope", "rope2"
 * (K writers: in0 = kn, in1 = table, u = [256, rows, 0,0, 256,256, flag, pos*512]), "kv_copy", "copy"
 * (V writer: in0 = vb, u = [n, .., extra = pos*512]), "attn_dmx1", "attn_dmx2", "attn_fd", "attn_fd2h"
 * (in0 = qr f32; u as M/quad.rs:286 / M/engine.rs:629; runs the core AND the combine, out = att),
 * "attn_fd_combine", "q_dmx" (no-ops: fused into the attention entry), and the prefill list of
 * M/engine.rs:1215-1241 with the uniforms of M/engine.rs:915-927: "q_f16" (in0 = qr f32, out = qh f16, u[0] packed
 * words), "attn_fa_mx" (in0 = qh f16) / "attn_fa" (in0 = qr f32) for the 64 tokens from u[4] = step_a of the block
 * at position u[0] - 1 (the dispatch of the first split of chunks, u[5] = 0, computes all chunks; later splits
 * are no-ops), "attn_fd4" (8 tokens from step_a) and "attn_fd" with u[5] = T > 4 (its batch mode); in0 and out are
 * the whole block's buffers [nb][4096]. Anything else: MKV_ERR_UNSUPPORTED. */
mkv_status mkv_dispatch(mkv_cache *c, int layer, const char *op, const uint32_t u[8], const void *in0,
                        const void *in1, void *out);

#ifdef __cplusplus
}
#endif
#endif
