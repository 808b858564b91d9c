"""The allocation-free verify entry point against the ordinary one.

mkv_attn_verify_static is for hosts that own every byte of device memory themselves, or that call from code
where allocating is off limits: its split-K pieces live in a fixed array inside the library instead of a
cudaMalloc'd scratch. Here it runs through the C ABI on caller-owned K/V buffers, twice in a row (the second call
finds the first call's leftovers in the array), and must agree with mkv_attn_verify and with the CPU oracle within the
f16-cache tolerance, with the caller's rows past the step left uninitialised (poisoned with NaN and infinity here).
This file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from mechta_b200 import _lib, kv, synth

pytestmark = pytest.mark.gpu
TOL = 2e-3  # max|a-b| / max|b|, the f16-cache bar of the other attention tests


def _max_rel(a, b):
    a, b = a.double(), b.double()
    return float((a - b).abs().max() / b.abs().max())


def test_static_scratch_verify_matches_the_allocating_entry_point_twice(oracle):
    assert torch.cuda.is_available(), "this test needs the GPU"
    torch.cuda.set_device(0)
    L = _lib.lib()
    ctx = kv.KvContext(0, torch.cuda.current_stream())
    capacity = 8192
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, capacity)
    kc, vc = oracle.new_cache(0, capacity), oracle.new_cache(0, capacity)
    rows = 6000
    for p in range(0, rows, 2000):
        k, v = synth.normal(301, synth.S_K, p, (2000, 2, 256)), synth.normal(301, synth.S_V, p, (2000, 2, 256))
        tab = kv.rope_table(p, 2000)
        cache.append(0, p, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), torch.from_numpy(tab).cuda())
        oracle.append(0, kc, vc, p, k, v, tab)
    ck, cv = cache.buffer_tensors(0)
    # Caller-owned buffers as a caller has them: uninitialised memory with the valid rows copied in. What lies past the
    # rows a call may see is poisoned on purpose: the kernel reads up to the next multiple of 64 rows and must not let it through.
    own_k = torch.empty(capacity, 2, 256, device="cuda", dtype=torch.float16)
    own_v = torch.empty(capacity, 2, 256, device="cuda", dtype=torch.float16)
    own_k[:rows].copy_(ck[:rows]); own_v[:rows].copy_(cv[:rows])
    stream = torch.cuda.current_stream().cuda_stream

    def poison_from(row):
        own_k[:rows].copy_(ck[:rows]); own_v[:rows].copy_(cv[:rows])
        own_k[row:].fill_(float("nan")); own_v[row:].fill_(float("nan"))
        own_v[row:row + 7].fill_(float("inf"))

    def both(first, pos, ntok, seed):
        poison_from(pos + ntok)
        qh = synth.normal(seed, synth.S_Q, pos, (ntok, 16, 256))
        q = torch.from_numpy(qh).cuda()
        want = torch.empty(ntok, 16, 256, device="cuda")
        got = torch.full((ntok, 16, 256), float("nan"), device="cuda")
        cache.attn_verify(0, first, pos, q, want)
        _lib.check(L.mkv_attn_verify_static(0, C.c_void_p(stream), own_k.data_ptr(), own_v.data_ptr(), capacity, first, pos,
                                            ntok, q.data_ptr(), got.data_ptr()))
        st = C.c_uint32(7)
        _lib.check(L.mkv_static_status(0, C.c_void_p(stream), C.byref(st)))  # blocks; no bounded wait ran out
        assert st.value == 0
        assert torch.isfinite(got).all()
        ref = oracle.attn_ref_f32(0, kc, vc, first, pos, qh)
        return max(_max_rel(got, want), oracle.max_rel(got.cpu().numpy(), ref))

    assert both(0, rows - 4, 4, 1) < TOL
    # second call: other length, window and token count, over whatever the first call left in the array
    assert both(100, 3000, 2, 2) < TOL
    assert both(0, rows - 4, 4, 3) < TOL
    assert both(0, 4093, 3, 4) < TOL  # the step ends exactly on a tile border: no tail rows at all

    # the caller's current device is left as it was (where the box has a second GPU: called with another one current)
    if torch.cuda.device_count() > 1:
        torch.cuda.set_device(1)
        q = torch.from_numpy(synth.normal(5, synth.S_Q, 0, (4, 16, 256))).to("cuda:0")
        got = torch.empty(4, 16, 256, device="cuda:0")
        _lib.check(L.mkv_attn_verify_static(0, C.c_void_p(stream), own_k.data_ptr(), own_v.data_ptr(), capacity, 0, 1000, 4,
                                            q.data_ptr(), got.data_ptr()))
        assert torch.cuda.current_device() == 1
        torch.cuda.set_device(0)
        torch.cuda.synchronize()
    assert torch.cuda.current_device() == 0

    # sizes beyond what the entry point supports are refused, nothing is launched
    q = torch.zeros(4, 16, 256, device="cuda")
    out = torch.empty_like(q)
    st = L.mkv_attn_verify_static(0, C.c_void_p(stream), own_k.data_ptr(), own_v.data_ptr(), capacity, 0, capacity - 2, 4,
                                  q.data_ptr(), out.data_ptr())
    assert st == _lib.ERR_CAPACITY and b"outside a cache" in L.mkv_last_error()
    st = L.mkv_attn_verify_static(0, C.c_void_p(stream), own_k.data_ptr(), own_v.data_ptr(), 262144 + 1024, 0, 10, 4,
                                  q.data_ptr(), out.data_ptr())
    assert st == _lib.ERR_CAPACITY
    st = L.mkv_attn_verify_static(0, C.c_void_p(stream), own_k.data_ptr(), own_v.data_ptr(), capacity, 0, 10, 5,
                                  q.data_ptr(), out.data_ptr())
    assert st == _lib.ERR_INVALID
    cache.close()
    ctx.close()
