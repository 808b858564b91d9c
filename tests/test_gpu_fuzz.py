"""Random verify steps against the oracle: cache sizes, positions, token counts, windows (first_pos), layer counts
and accept counts drawn at random, several layers launched back to back without a sync in between (the pattern in
which the kernels overlap their neighbours in the stream)."""
import numpy as np
import pytest
import torch

from mechta_b200 import kv

pytestmark = pytest.mark.gpu
TOL = {0: 2e-3, 1: 1e-5}


def _oracle_views(cache, layer, cap):
    k, v = cache.buffer_tensors(layer)
    if cache.fmt == kv.KvFormat.F16:
        as_np = lambda t: t.view(torch.int16).cpu().numpy().view(np.uint16).reshape(cap, 512).copy()
    else:
        as_np = lambda t: t.cpu().numpy().reshape(cap, 512).copy()
    return as_np(k), as_np(v)


@pytest.mark.parametrize("seed", [11, 12])
def test_random_steps_against_the_oracle(oracle, seed):
    torch.cuda.set_device(0)
    ctx = kv.KvContext(0, torch.cuda.current_stream())
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    rng = np.random.default_rng(seed)
    checked = 0
    for case in range(14):
        fmt = kv.KvFormat(int(rng.integers(0, 2)))
        cap = int(rng.choice([4096, 8192, 20480, 40960, 69632]))
        n_layers = int(rng.integers(1, 4))
        cache = kv.KvCache(ctx, fmt, n_layers, cap)
        pos = int(rng.integers(1, cap - 8))
        g = torch.Generator(device="cuda"); g.manual_seed(1000 * seed + case)
        for l in range(n_layers):
            k, v = cache.buffer_tensors(l)
            k[:pos].normal_(generator=g); v[:pos].normal_(generator=g)
        cache.set_len(pos)
        torch.cuda.synchronize()
        ocs = [_oracle_views(cache, l, cap) for l in range(n_layers)]
        for _ in range(int(rng.integers(1, 4))):
            ntok = int(rng.integers(1, 5))
            if pos + ntok >= cap:
                break
            first = int(rng.integers(0, pos + 1)) if rng.random() < 0.4 else 0
            kn = rng.standard_normal((n_layers, ntok, 2, 256)).astype(np.float32)
            vn = rng.standard_normal((n_layers, ntok, 2, 256)).astype(np.float32)
            q = rng.standard_normal((n_layers, ntok, 16, 256)).astype(np.float32)
            tab = kv.rope_table(pos, ntok)
            outs = torch.empty(n_layers, ntok, 16, 256, device="cuda")
            cache.append_layers(pos, dev(kn), dev(vn), dev(tab))
            dq = dev(q)
            for l in range(n_layers):
                cache.attn_verify(l, first, pos, dq[l], outs[l])
            ctx.sync()
            got = outs.cpu().numpy()
            for l in range(n_layers):
                oracle.append(int(fmt), ocs[l][0], ocs[l][1], pos, kn[l], vn[l], tab)
                want = oracle.attn_ref_f32(int(fmt), ocs[l][0], ocs[l][1], first, pos, q[l])
                err = oracle.max_rel(got[l], want)
                assert err < TOL[int(fmt)], (case, int(fmt), cap, pos, ntok, first, l, err)
                checked += 1
            pos += 1 + int(rng.integers(0, ntok))
            cache.truncate(pos)
        cache.close()
    assert checked > 20
    ctx.close()


def test_f32_cache_on_the_warp_mma_kernel_in_a_child_process():
    """The f32 cache runs on the tcgen05 kernel; MKV_VERIFY32=mma selects the warp-MMA kernel kept as the measured
    baseline (read once per process, so a child process runs the same random steps with it)."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, MKV_VERIFY32="mma")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(root, "tests", "test_gpu_fuzz.py"), "-q", "-x", "-m", "gpu", "-k",
                        "random_steps"], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
