"""Host-side mirror of the reference's KV operators above the C ABI.

Names follow the reference (engine/crates/mechta/src/engine.rs, quad.rs): KvFormat, check_ctx, rope_table,
Root, read_root / write_root, need_bytes; step4-style helpers take `pos` exactly as the reference does (token t of
a call sits at pos + t). PyTorch is used only for device memory and streams; every computation is a call into
libmechta_kv through ctypes with raw pointers.
"""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib
from ._lib import MkvError, check

CTX_DEFAULT, CTX_MIN, CTX_MAX = 65536, 4096, 262144  # engine.rs:23-25
HQ, HKV, D, ROW = 16, 2, 256, 512
K_VERIFY = 4  # quad.rs K


class KvFormat(enum.IntEnum):
    """engine.rs:49-68"""
    F16 = _lib.F16
    F32 = _lib.F32

    @property
    def elem_bytes(self) -> int:
        return 2 if self is KvFormat.F16 else 4

    def data_words(self, n: int) -> int:
        return n if self is KvFormat.F32 else n // 2

    def buffer_bytes_for(self, ctx: int) -> int:
        return 4 * self.data_words(ctx * 512)

    @property
    def torch_dtype(self):
        return torch.float16 if self is KvFormat.F16 else torch.float32


def check_ctx(n: int) -> int:
    """engine.rs:28-33: a multiple of 1024 in [CTX_MIN, CTX_MAX]."""
    if n % 1024 != 0 or not (CTX_MIN <= n <= CTX_MAX):
        raise ValueError(f"context {n}: must be a multiple of 1024 between {CTX_MIN} and {CTX_MAX}")
    return n


def rope_table(pos: int, ntok: int = 1) -> np.ndarray:
    """engine.rs:108-114 for positions pos..pos+ntok-1: [ntok][64] = [cos 0..31 | sin 0..31]."""
    out = np.empty((ntok, 64), np.float32)
    _lib.lib().mkv_rope_table(int(pos), int(ntok), out.ctypes.data_as(C.c_void_p))
    return out


def need_bytes(ctx: int, fmt: KvFormat, n_layers: int = 11) -> int:
    """memcheck.rs:14-20 without BASE_BYTES (10 attention layers + the MTP layer by default)."""
    return int(_lib.lib().mkv_need_bytes(ctx, int(fmt), n_layers))


def root_key(tokens) -> str:
    """session.rs:61-66"""
    t = np.ascontiguousarray(tokens, np.uint32)
    return f"{int(_lib.lib().mkv_root_key(t.ctypes.data_as(C.c_void_p), t.size)):016x}"


@dataclass
class Root:
    """engine.rs:194-195 Root, KV part: rows [0, p) of every attention layer, K then V, raw cache bytes."""
    p: int
    fmt: KvFormat
    n_layers: int
    payload: torch.Tensor  # uint8, pinned host memory


def _ptr(t) -> int:
    if t is None:
        return 0
    assert t.is_contiguous(), "tensors passed to the KV operators must be contiguous"
    return t.data_ptr()


class KvContext:
    """One device + the stream the KV operators run on (mkv_ctx)."""

    def __init__(self, device: int = 0, stream: torch.cuda.Stream | None = None):
        self._h = C.c_void_p()
        self.device = int(device)
        self.stream = stream
        sp = C.c_void_p(stream.cuda_stream) if stream is not None else None
        check(_lib.lib().mkv_ctx_create(self.device, sp, C.byref(self._h)))

    def sync(self) -> None:
        check(_lib.lib().mkv_sync(self._h))

    @property
    def launches(self) -> int:
        return int(_lib.lib().mkv_launch_count(self._h))

    def prof_enable(self, on: int) -> None:
        """0 = off; n > 0 = on, with n event pairs created ahead of time."""
        check(_lib.lib().mkv_prof_enable(self._h, int(on)))

    def prof_read(self) -> tuple[float, int]:
        ms, n = C.c_double(), C.c_uint64()
        check(_lib.lib().mkv_prof_read(self._h, C.byref(ms), C.byref(n)))
        return ms.value, int(n.value)

    def combine_shards(self, recs: torch.Tensor, ntok: int, out: torch.Tensor) -> None:
        """recs [n_shards][64][258] f32 -> out [ntok][16][256] (ops.wgsl:529-537 over shards)."""
        check(_lib.lib().mkv_combine_shards(self._h, _ptr(recs), recs.shape[0], ntok, _ptr(out)))

    def attn_verify_batch(self, items) -> None:
        """items: iterable of (cache, layer, first_pos, pos, q, out); one launch pair for all of them."""
        items = list(items)
        arr = (_lib.VerifyItem * len(items))()
        for i, (cache, layer, first_pos, pos, q, out) in enumerate(items):
            arr[i] = _lib.VerifyItem(cache._h.value, layer, first_pos, pos, q.shape[0], _ptr(q), _ptr(out))
        check(_lib.lib().mkv_attn_verify_batch(self._h, arr, len(items)))

    def close(self) -> None:
        if self._h:
            _lib.lib().mkv_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KvCache:
    """The per-layer K and V buffers of the attention layers and the operators that touch them (mkv_cache)."""

    def __init__(self, ctx: KvContext, fmt: KvFormat, n_layers: int, context: int, shard_first: int = 0,
                 shard_tokens: int = 0, ring: int = 0):
        """context: the sequence's context (check_ctx rule). shard_tokens = 0: the whole context lives here;
        otherwise only rows [shard_first, shard_first + shard_tokens). ring > 0: a ring cache of that many rows,
        position p in row p % ring (flint.rs:24-26)."""
        self.ctx, self.fmt, self.n_layers = ctx, KvFormat(fmt), n_layers
        self.context, self.ring = context, ring
        self.capacity, self.shard_first = (ring or shard_tokens or context), shard_first
        self._h = C.c_void_p()
        if ring:
            check(_lib.lib().mkv_cache_create_ring(ctx._h, int(fmt), n_layers, context, ring, C.byref(self._h)))
        else:
            check(_lib.lib().mkv_cache_create(ctx._h, int(fmt), n_layers, context, shard_first, shard_tokens,
                                              C.byref(self._h)))

    # -- bookkeeping
    def __len__(self) -> int:
        return int(_lib.lib().mkv_cache_len(self._h))

    def set_len(self, n: int) -> None:
        check(_lib.lib().mkv_cache_set_len(self._h, n))

    @property
    def device_bytes(self) -> int:
        return int(_lib.lib().mkv_cache_device_bytes(self._h))

    def buffers(self, layer: int) -> tuple[int, int]:
        k, v = C.c_void_p(), C.c_void_p()
        check(_lib.lib().mkv_cache_buffers(self._h, layer, C.byref(k), C.byref(v)))
        return k.value, v.value

    def buffer_tensors(self, layer: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Zero-copy torch views [capacity][2][256] of a layer's K and V (for tests and synthetic fills)."""
        kp, vp = self.buffers(layer)
        return tuple(_as_tensor(p, self.capacity * ROW, self.fmt.torch_dtype, self.ctx.device).view(self.capacity, HKV, D)
                     for p in (kp, vp))

    # -- operators
    def append(self, layer: int, pos: int, k: torch.Tensor, v: torch.Tensor, tab: torch.Tensor | None) -> None:
        """kv_rope2 + kv_copy (kv.wgsl:19-42): k, v f32 [ntok][2][256]; tab f32 [ntok][64] or None."""
        check(_lib.lib().mkv_append(self._h, layer, pos, k.shape[0], _ptr(k), _ptr(v), _ptr(tab)))

    def append_layers(self, pos: int, k: torch.Tensor, v: torch.Tensor, tab: torch.Tensor | None) -> None:
        """All layers in one launch: k, v f32 [n_layers][ntok][2][256]."""
        check(_lib.lib().mkv_append_layers(self._h, pos, k.shape[1], _ptr(k), _ptr(v), _ptr(tab)))

    def truncate(self, new_len: int, scrub: bool = False) -> None:
        """Rollback of refused drafts: the next step continues at new_len (session.rs:385-411)."""
        check(_lib.lib().mkv_truncate(self._h, new_len, int(scrub)))

    def attn_verify(self, layer: int, first_pos: int, pos: int, q: torch.Tensor, out: torch.Tensor) -> None:
        """q_dmx + attn_dmx2 + attn_fd_combine (dmx.rs) / attn_fd (+combine): q, out f32 [ntok][16][256]."""
        check(_lib.lib().mkv_attn_verify(self._h, layer, first_pos, pos, q.shape[0], _ptr(q), _ptr(out)))

    def attn_verify_window(self, layer: int, window: int, sinks: torch.Tensor | None, pos: int, q: torch.Tensor,
                           out: torch.Tensor) -> None:
        """Verify attention with a sliding window (0 = none) and per-head sinks [16] (None = none), on a ring or an
        ordinary cache (flint.rs:22-26, flint_attn.wgsl:79-82,243-255)."""
        check(_lib.lib().mkv_attn_verify_window(self._h, layer, window, _ptr(sinks), pos, q.shape[0], _ptr(q), _ptr(out)))

    def attn_step(self, layer: int, first_pos: int, pos: int, qf: torch.Tensor, kb: torch.Tensor, vb: torch.Tensor,
                  q_norm: torch.Tensor, k_norm: torch.Tensor, tab: torch.Tensor, out: torch.Tensor | None = None,
                  out16: torch.Tensor | None = None, eps: float = 1e-6) -> None:
        """The layer's step around the KV path in two launches (quad.rs:113-125): rmsnorm of q and k heads, rope2,
        kv_rope2 + kv_copy of rows [pos, pos + ntok), the attention, attn_gate (out, f32) / attn_gate16 (out16, f16).
        qf [ntok][16][512] (query | gate per head), kb [ntok][2][256], vb [ntok][512], norms [256], tab [ntok][64]."""
        inp = _lib.StepIn(_ptr(qf), _ptr(kb), _ptr(vb), _ptr(q_norm), _ptr(k_norm), _ptr(tab), eps)
        check(_lib.lib().mkv_attn_step(self._h, layer, first_pos, pos, qf.shape[0], C.byref(inp),
                                       _ptr(out) if out is not None else None, _ptr(out16) if out16 is not None else None))

    def attn_verify_partial(self, layer: int, first_pos: int, pos: int, q: torch.Tensor, rec: torch.Tensor) -> None:
        """This shard's un-normalised record [64][258] for the step."""
        check(_lib.lib().mkv_attn_verify_partial(self._h, layer, first_pos, pos, q.shape[0], _ptr(q), _ptr(rec)))

    def attn_prefill(self, layer: int, first_pos: int, pos0: int, q: torch.Tensor, out: torch.Tensor) -> None:
        """q_f16 + attn_fa_mx / attn_fa / attn_fd4 (+combine): q [ntok][16][256] f32 (`qr`) or f16 (`qh`, f16 cache only),
        out f32 [ntok][16][256]; the block's K/V appended before."""
        assert q.dtype in (torch.float32, torch.float16)
        check(_lib.lib().mkv_attn_prefill(self._h, layer, first_pos, pos0, q.shape[0], _ptr(q), int(q.dtype == torch.float16),
                                          _ptr(out)))

    def dispatch(self, layer: int, op: str, uniform, in0=None, in1=None, out=None) -> None:
        """The reference's own form: WGSL entry point name + its 8-word uniform (ops.wgsl:4)."""
        u = (C.c_uint32 * 8)(*[int(x) & 0xFFFFFFFF for x in uniform])
        check(_lib.lib().mkv_dispatch(self._h, layer, op.encode(), u, _ptr(in0), _ptr(in1), _ptr(out)))

    # -- prefix cache
    def snapshot_bytes(self, p: int) -> int:
        return int(_lib.lib().mkv_snapshot_bytes(self._h, p))

    def read_root(self, p: int, payload: torch.Tensor | None = None, wait: bool = True) -> Root:
        """Engine::read_root, KV part (engine.rs:784-802): rows [0, p) to pinned host memory."""
        n = self.snapshot_bytes(p)
        if payload is None:
            payload = torch.empty(n, dtype=torch.uint8, pin_memory=True)
        w = C.c_size_t()
        check(_lib.lib().mkv_snapshot(self._h, p, payload.data_ptr(), payload.numel(), C.byref(w)))
        if wait:
            self.snapshot_wait()
        return Root(p, self.fmt, self.n_layers, payload[: w.value])

    def snapshot_wait(self) -> None:
        check(_lib.lib().mkv_snapshot_wait(self._h))

    def write_root(self, root: Root) -> None:
        """Engine::write_root, KV part (engine.rs:804-823)."""
        if root.fmt != self.fmt or root.n_layers != self.n_layers:
            raise MkvError(_lib.ERR_FORMAT, "root of another format or layer count")
        check(_lib.lib().mkv_restore(self._h, root.p, root.payload.data_ptr(), root.payload.numel()))

    def check_guards(self) -> int:
        """Canary bytes around this cache's buffers that were overwritten (always 0 with the shipped library, which has no
        guards; the checked build is `make -C mechta_b200/csrc checks`, selected with MKV_LIB_PATH)."""
        bad = C.c_uint64(0)
        check(_lib.lib().mkv_cache_check_guards(self._h, C.byref(bad)))
        return int(bad.value)

    def close(self) -> None:
        if self._h:
            bad = self.check_guards() if _lib.lib().mkv_checks_enabled() else 0
            _lib.lib().mkv_cache_destroy(self._h)
            self._h = C.c_void_p()
            if bad:
                raise _lib.MkvError(-1, f"{bad} guard bytes around the cache's buffers were overwritten")

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class KvExchange:
    """Mailboxes for the peer exchange of shard records (mkv_exchange): every rank's attention kernel stores its
    record into every rank's mailbox over NVLink, no collective call. `gather_handles(my_handle) -> [bytes] * world`
    is how the 64-byte IPC handles travel between the processes (e.g. torch.distributed.all_gather_object)."""

    def __init__(self, ctx: KvContext, rank: int, world: int, gather_handles=None):
        self.ctx, self.rank, self.world = ctx, rank, world
        self._h = C.c_void_p()
        check(_lib.lib().mkv_exchange_create(ctx._h, rank, world, C.byref(self._h)))
        mine = C.create_string_buffer(64)
        check(_lib.lib().mkv_exchange_handle(self._h, mine))
        handles = [mine.raw] if world == 1 else gather_handles(mine.raw)
        handles = [h if h is not None else bytes(64) for h in handles]  # None = a rank that never joined
        assert len(handles) == world and all(len(h) == 64 for h in handles)
        check(_lib.lib().mkv_exchange_connect(self._h, b"".join(handles)))

    def attn_verify(self, cache: "KvCache", layer: int, first_pos: int, pos: int, q: torch.Tensor, out: torch.Tensor) -> None:
        """Local record -> peer stores into all mailboxes -> merge; `out` is final on every rank."""
        check(_lib.lib().mkv_attn_verify_exchange(cache._h, self._h, layer, first_pos, pos, q.shape[0], _ptr(q), _ptr(out)))

    def close(self) -> None:
        if self._h:
            _lib.lib().mkv_exchange_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def write_root_file(path: str, tokens, root: Root) -> None:
    """session.rs:92-111 (KV section; n_ssm = 0)."""
    t = np.ascontiguousarray(tokens, np.uint32)
    assert t.size == root.p
    check(_lib.lib().mkv_root_write(path.encode(), int(root.fmt), root.n_layers, root.p, t.ctypes.data_as(C.c_void_p),
                                    root.payload.data_ptr(), root.payload.numel()))


def read_root_file(path: str, fmt: KvFormat, n_layers: int, pin: bool = True) -> tuple[np.ndarray, Root]:
    """session.rs:113-129: returns (tokens, Root)."""
    L = _lib.lib()
    p, nbytes = C.c_uint32(), C.c_size_t()
    check(L.mkv_root_read(path.encode(), int(fmt), n_layers, C.byref(p), None, 0, None, 0, C.byref(nbytes)))
    toks = np.empty(p.value, np.uint32)
    payload = torch.empty(nbytes.value, dtype=torch.uint8, pin_memory=pin)
    check(L.mkv_root_read(path.encode(), int(fmt), n_layers, C.byref(p), toks.ctypes.data_as(C.c_void_p), toks.size,
                          payload.data_ptr(), payload.numel(), C.byref(nbytes)))
    return toks, Root(p.value, KvFormat(fmt), n_layers, payload)


def _as_tensor(ptr: int, numel: int, dtype, device: int) -> torch.Tensor:
    """A torch view over device memory owned by the library (no copy)."""
    itemsize = torch.empty((), dtype=dtype).element_size()

    class _Mem:
        pass

    m = _Mem()
    typestr = {torch.float16: "<f2", torch.float32: "<f4", torch.uint8: "|u1"}[dtype]
    m.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 3,
                                  "strides": (itemsize,)}
    return torch.as_tensor(m, device=f"cuda:{device}")
