"""The allocation-free verify entry point against the ordinary one.

mkv_attn_verify_static is for hosts that own every byte of device memory themselves, or that call from code
where allocating is off limits: its split-K pieces live in a fixed array inside the library instead of a
cudaMalloc'd scratch. Here it runs through the C ABI on caller-owned K/V buffers, twice in a row (the second call
finds the first call's leftovers in the array), and must agree with mkv_attn_verify within the f16-cache tolerance.
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


def test_static_scratch_verify_matches_the_allocating_entry_point_twice():
    assert torch.cuda.is_available(), "this test needs the GPU"
    torch.cuda.set_device(0)
    L = _lib.lib()
    ctx = kv.KvContext(0, torch.cuda.current_stream())
    capacity = 8192
    cache = kv.KvCache(ctx, kv.KvFormat.F16, 1, capacity)
    # caller-owned buffers with the same contents as the library's cache
    rows = 6000
    for p in range(0, rows, 2000):
        k = torch.from_numpy(synth.normal(301, synth.S_K, p, (2000, 2, 256))).cuda()
        v = torch.from_numpy(synth.normal(301, synth.S_V, p, (2000, 2, 256))).cuda()
        cache.append(0, p, k, v, torch.from_numpy(kv.rope_table(p, 2000)).cuda())
    ck, cv = cache.buffer_tensors(0)
    own_k, own_v = ck.clone(), cv.clone()
    stream = torch.cuda.current_stream().cuda_stream

    def both(first, pos, ntok, seed):
        q = torch.from_numpy(synth.normal(seed, synth.S_Q, pos, (ntok, 16, 256))).cuda()
        want = torch.empty(ntok, 16, 256, device="cuda")
        got = torch.full((ntok, 16, 256), float("nan"), device="cuda")
        cache.attn_verify(0, first, pos, q, want)
        _lib.check(L.mkv_attn_verify_static(0, C.c_void_p(stream), own_k.data_ptr(), own_v.data_ptr(), capacity, first, pos,
                                            ntok, q.data_ptr(), got.data_ptr()))
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        return _max_rel(got, want)

    assert both(0, rows - 4, 4, 1) < TOL
    # second call: other length, window and token count, over whatever the first call left in the array
    assert both(100, 3000, 2, 2) < TOL
    assert both(0, rows - 4, 4, 3) < TOL

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
