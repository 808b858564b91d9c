//! Safe handles over `mechta-kv-sys` for a host written like the reference engine
//! (engine/crates/mechta/src/engine.rs, quad.rs): a context per device and stream, a cache that owns the per-layer
//! K and V buffers, and the operators of the KV path as methods. All `unsafe` of the path is in this file and in the
//! `-sys` crate, as the reference keeps its one `unsafe` in engine/crates/shader.
//!
//! NOT COMPILED where it was written (no Rust toolchain there). Device memory is not owned here: the engine passes
//! the device addresses of its own buffers (`DevPtr`), exactly the buffers it binds to the WGSL dispatches today.
//!
//! Call order of one 4-token verify step per attention layer (quad.rs:113-125):
//!   cache.append(layer, pos, kn, vb, tab)?;  cache.attn_verify(layer, 0, pos, 4, qr, att)?;
//! and after sampling `cache.truncate(pos + 1 + accepted)?` (session.rs:401). Everything is enqueued on the
//! context's stream; `KvContext::sync` is the only blocking call besides `Root` reads.

use core::ffi::{c_int, c_void};
use core::ptr;
use mechta_kv_sys as sys;
use std::ffi::CStr;
use std::marker::PhantomData;

/// A device address on the context's GPU (a `CUdeviceptr`), borrowed for the duration of a call.
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub struct DevPtr(pub u64);

impl DevPtr {
    pub const NULL: DevPtr = DevPtr(0);
    fn f32(self) -> *const f32 { self.0 as usize as *const f32 }
    fn f32_mut(self) -> *mut f32 { self.0 as usize as *mut f32 }
    fn void(self) -> *const c_void { self.0 as usize as *const c_void }
    fn void_mut(self) -> *mut c_void { self.0 as usize as *mut c_void }
}

/// engine.rs:49-68
#[derive(Clone, Copy, Debug, PartialEq, Eq)]
pub enum KvFormat { F16, F32 }

impl KvFormat {
    fn raw(self) -> sys::mkv_fmt { match self { KvFormat::F16 => sys::MKV_F16, KvFormat::F32 => sys::MKV_F32 } }
    pub fn elem_bytes(self) -> usize { match self { KvFormat::F16 => 2, KvFormat::F32 => 4 } }
}

/// A status other than MKV_OK, with the library's message for it.
#[derive(Debug, Clone)]
pub struct KvError { pub status: i32, pub text: String }

impl std::fmt::Display for KvError {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result { write!(f, "mkv status {}: {}", self.status, self.text) }
}
impl std::error::Error for KvError {}

fn check(status: sys::mkv_status) -> Result<(), KvError> {
    if status == sys::MKV_OK { return Ok(()); }
    // SAFETY: mkv_last_error returns a NUL-terminated string owned by the library, valid until the next failing call on this thread.
    let text = unsafe { CStr::from_ptr(sys::mkv_last_error()) }.to_string_lossy().into_owned();
    Err(KvError { status: status as i32, text })
}

/// One CUDA device + the stream the KV operators run on. Not `Send`: calls on a context come from one thread, as the
/// reference's engine (engine/crates/api/src/lib.rs:46).
pub struct KvContext { raw: *mut sys::mkv_ctx, _not_send: PhantomData<*mut ()> }

impl KvContext {
    /// `stream` is a `cudaStream_t` owned by the caller (null = the legacy default stream).
    pub fn new(device: i32, stream: *mut c_void) -> Result<Self, KvError> {
        let mut raw = ptr::null_mut();
        // SAFETY: `raw` is a valid out-pointer; the library validates the device index.
        check(unsafe { sys::mkv_ctx_create(device as c_int, stream, &mut raw) })?;
        Ok(KvContext { raw, _not_send: PhantomData })
    }
    /// Blocks until everything enqueued has finished; reports a kernel's bounded wait that ran out.
    pub fn sync(&self) -> Result<(), KvError> { check(unsafe { sys::mkv_sync(self.raw) }) }
    pub fn launches(&self) -> u64 { unsafe { sys::mkv_launch_count(self.raw) } }
    /// attn_fd_combine over the records of `n_shards` sequence shards (ops.wgsl:529-537).
    pub fn combine_shards(&self, recs: DevPtr, n_shards: i32, ntok: u32, out: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_combine_shards(self.raw, recs.f32(), n_shards as c_int, ntok, out.f32_mut()) })
    }
}

impl Drop for KvContext {
    fn drop(&mut self) { unsafe { sys::mkv_ctx_destroy(self.raw) } }
}

/// engine.rs:108-114: `[cos 0..31 | sin 0..31]` per position, for positions pos..pos+ntok-1.
pub fn rope_table(pos: i32, ntok: u32) -> Vec<f32> {
    let mut out = vec![0f32; 64 * ntok as usize];
    // SAFETY: `out` has room for ntok * 64 floats.
    unsafe { sys::mkv_rope_table(pos, ntok, out.as_mut_ptr()) };
    out
}

/// memcheck.rs:14-20 without its fixed part.
pub fn need_bytes(ctx_tokens: u32, fmt: KvFormat, n_layers: i32) -> u64 { unsafe { sys::mkv_need_bytes(ctx_tokens, fmt.raw(), n_layers as c_int) } }

/// session.rs:61-66
pub fn root_key(tokens: &[u32]) -> u64 { unsafe { sys::mkv_root_key(tokens.as_ptr(), tokens.len()) } }

/// engine.rs:194-195 `Root`, KV part: rows [0, p) of every attention layer, K then V, raw cache bytes, in pinned host memory.
pub struct Root { pub p: u32, pub fmt: KvFormat, pub n_layers: i32, data: *mut c_void, bytes: usize }

impl Root {
    pub fn payload(&self) -> &[u8] { unsafe { std::slice::from_raw_parts(self.data as *const u8, self.bytes) } }
}
impl Drop for Root {
    fn drop(&mut self) { unsafe { sys::mkv_host_free(self.data) } }
}

/// The per-layer K and V buffers of the attention layers (kc[il], vc[il] of engine.rs:493-494) and their operators.
pub struct KvCache<'c> { raw: *mut sys::mkv_cache, fmt: KvFormat, n_layers: i32, _ctx: PhantomData<&'c KvContext> }

impl<'c> KvCache<'c> {
    /// `context`: a multiple of 1024 in [4096, 262144] (engine.rs:28-33). `shard`: None = the whole context lives here;
    /// Some((first, rows)) = one contiguous shard of a sequence-sharded context.
    pub fn new(ctx: &'c KvContext, fmt: KvFormat, n_layers: i32, context: u32, shard: Option<(u32, u32)>) -> Result<Self, KvError> {
        let (first, rows) = shard.unwrap_or((0, 0));
        let mut raw = ptr::null_mut();
        check(unsafe { sys::mkv_cache_create(ctx.raw, fmt.raw(), n_layers as c_int, context, first, rows, &mut raw) })?;
        Ok(KvCache { raw, fmt, n_layers, _ctx: PhantomData })
    }
    pub fn len(&self) -> u32 { unsafe { sys::mkv_cache_len(self.raw) } }
    pub fn is_empty(&self) -> bool { self.len() == 0 }
    /// kv_rope2 + kv_copy (kv.wgsl:19-42): `kn` f32 [ntok][2][256], `vb` f32 [ntok][512], `tab` f32 [ntok][64] or NULL.
    pub fn append(&mut self, layer: i32, pos: u32, ntok: u32, kn: DevPtr, vb: DevPtr, tab: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_append(self.raw, layer as c_int, pos, ntok, kn.f32(), vb.f32(), tab.f32()) })
    }
    /// Rollback of refused drafts: the next step continues at `new_len` (session.rs:385-411).
    pub fn truncate(&mut self, new_len: u32, scrub: bool) -> Result<(), KvError> {
        check(unsafe { sys::mkv_truncate(self.raw, new_len, scrub as c_int) })
    }
    /// q_dmx + attn_dmx2 + attn_fd_combine (dmx.rs) or attn_fd + combine: `qr`, `att` f32 [ntok][16][256].
    pub fn attn_verify(&mut self, layer: i32, first_pos: u32, pos: u32, ntok: u32, qr: DevPtr, att: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_attn_verify(self.raw, layer as c_int, first_pos, pos, ntok, qr.f32(), att.f32_mut()) })
    }
    /// This shard's un-normalised record [64][258] (ops.wgsl:389-391) for the merge across shards.
    pub fn attn_verify_partial(&mut self, layer: i32, first_pos: u32, pos: u32, ntok: u32, qr: DevPtr, rec: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_attn_verify_partial(self.raw, layer as c_int, first_pos, pos, ntok, qr.f32(), rec.f32_mut()) })
    }
    /// The nine dispatches of quad.rs:113-125 in two launches.
    pub fn attn_step(&mut self, layer: i32, first_pos: u32, pos: u32, ntok: u32, inputs: &sys::mkv_step_in, ag: DevPtr, ag16: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_attn_step(self.raw, layer as c_int, first_pos, pos, ntok, inputs, ag.f32_mut(), ag16.void_mut()) })
    }
    /// q_f16 + attn_fa_mx / attn_fa / attn_fd4 (engine.rs:1215-1241); the block's rows are appended before.
    pub fn attn_prefill(&mut self, layer: i32, first_pos: u32, pos0: u32, ntok: u32, q: DevPtr, q_is_f16: bool, att: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_attn_prefill(self.raw, layer as c_int, first_pos, pos0, ntok, q.void(), q_is_f16 as c_int, att.f32_mut()) })
    }
    /// The reference's own form: WGSL entry point name + its 8-word uniform (ops.wgsl:4).
    pub fn dispatch(&mut self, layer: i32, op: &CStr, uniform: &[u32; 8], in0: DevPtr, in1: DevPtr, out: DevPtr) -> Result<(), KvError> {
        check(unsafe { sys::mkv_dispatch(self.raw, layer as c_int, op.as_ptr(), uniform.as_ptr(), in0.void(), in1.void(), out.void_mut()) })
    }
    /// Engine::read_root, KV part (engine.rs:784-802): rows [0, p) to pinned host memory; blocks until they have landed.
    pub fn read_root(&mut self, p: u32) -> Result<Root, KvError> {
        let bytes = unsafe { sys::mkv_snapshot_bytes(self.raw, p) };
        let mut data = ptr::null_mut();
        check(unsafe { sys::mkv_host_alloc(bytes, &mut data) })?;
        let root = Root { p, fmt: self.fmt, n_layers: self.n_layers, data, bytes };
        let mut written = 0usize;
        check(unsafe { sys::mkv_snapshot(self.raw, p, data, bytes, &mut written) })?;
        check(unsafe { sys::mkv_snapshot_wait(self.raw) })?;
        debug_assert_eq!(written, bytes);
        Ok(root)
    }
    /// Engine::write_root, KV part (engine.rs:804-823). The root must stay alive until the context is synchronised.
    pub fn write_root(&mut self, root: &Root) -> Result<(), KvError> {
        if root.fmt != self.fmt || root.n_layers != self.n_layers {
            return Err(KvError { status: sys::MKV_ERR_FORMAT as i32, text: "root of another format or layer count".into() });
        }
        check(unsafe { sys::mkv_restore(self.raw, root.p, root.data as *const c_void, root.bytes) })
    }
}

impl Drop for KvCache<'_> {
    fn drop(&mut self) { unsafe { sys::mkv_cache_destroy(self.raw) } }
}
