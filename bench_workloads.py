"""Benchmark workloads beside the default line of bench.py. Each `measure_*` returns a dict; bench.py prints them
either as a line of their own (--workload NAME) or under `other_workloads` of the default line.

verify262k  the decode attention kernel alone at the last rows of a 262,144-token context, f16 or f32 cache, 2 layers.
step65k     decode65k with the layer's whole step around the KV path fused (mkv_attn_step): per layer one launch for
            rmsnorm of q and k heads + RoPE + the cache rows, one for attention + merge + output gate, i.e. 20 launches
            per step where the reference's dispatch list has 90; the rows of a layer are written just before its attention.
prefill     Prefix-cache restore + prefill: a 32,768-token f16 snapshot of 10 layers is restored from pinned host
            memory, a 2,048-token block is appended and attends to the prefix and to itself (causal), and 34,816 rows are
            snapshotted back. One step = all of that. Reported: attention TFLOP/s against the tensor peak, copy GB/s.
sessions    32 concurrent sessions with ragged f16 caches (lengths uniform in [1,024, 131,072]), spread over the ranks
            by KV bytes (greedy, longest first), 10 layers, one 4-token verify per session per step with its own accept
            count. No collective: sessions are independent.
longctx     One 262,144-token context with an f32 cache, sequence-sharded in equal contiguous chunks over the ranks; the
            ranks' records are exchanged by the attention kernel itself (peer stores over NVLink) or by an NCCL all-gather.
            Total work is fixed as the ranks grow ("strong"); the line carries the same launch over the unsharded context
            on rank 0 (`strong_ref`), the efficiency against it, the kernel-alone / exchange split and a check of the
            sharded output against the unsharded one on the same rows and queries.
"""
from __future__ import annotations

import json
import os

import numpy as np

N_LAYERS = 10
ROOT = os.path.dirname(os.path.abspath(__file__))


def peaks():
    """(HBM GB/s, sustained bf16 TFLOP/s, which): the measured peaks of this pool's B200s, else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
        except Exception:
            pass
    return 6650.0, 1400.0, "fallback"


def spread(xs):
    xs = sorted(float(x) for x in xs)
    q = lambda f: xs[min(len(xs) - 1, max(0, int(round(f * (len(xs) - 1)))))]
    return {"median": float(np.median(xs)), "p10": q(0.1), "p90": q(0.9), "min": xs[0], "max": xs[-1], "n": len(xs)}


def _env():
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    return world, rank, local


def _reduce(torch, world, x, op="max"):
    if world == 1:
        return float(x)
    import torch.distributed as dist
    t = torch.tensor([float(x)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
    return float(t.item())


def _barrier(torch, world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


# ---------------------------------------------------------------------------------------------------------------------

# dram read + write per launch of verify_f32_tc_kernel at 262,076 tokens, from one ncu capture of this workload
# (1.0744 GB read + 6.5 MB written against 1.0735 GB algorithmic); a constant, not re-measured by the bench
NCU_TRAFFIC_BYTES_VERIFY262K_F32 = 1_080_900_000


def measure_verify262k(ctx, stream, fmt, layers=2, steps=12, warmup=3):
    """The decode attention launch alone at 262,144 tokens: `layers` layers back to back per step, appends in between."""
    import torch
    from mechta_b200 import kv
    context = kv.CTX_MAX
    n = context - 4 * (steps + warmup) - 8
    per_pos = 2048 if fmt == kv.KvFormat.F16 else 4096
    cache = kv.KvCache(ctx, fmt, layers, context)
    g = torch.Generator(device="cuda"); g.manual_seed(9)
    for l in range(layers):
        k, v = cache.buffer_tensors(l)
        k[:n].normal_(generator=g); v[:n].normal_(generator=g)
    cache.set_len(n)
    ctx.sync()
    q = torch.randn(layers, 4, 16, 256, device="cuda", generator=g)
    kn = torch.randn(layers, 4, 2, 256, device="cuda", generator=g)
    vn = torch.randn(layers, 4, 2, 256, device="cuda", generator=g)
    out = torch.empty_like(q)
    tabs = torch.from_numpy(kv.rope_table(n, 4 * (steps + warmup) + 8)).cuda()
    pos, nbytes = n, 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for s in range(warmup + steps):
        if s == warmup:
            e0.record(stream)
        cache.append_layers(pos, kn, vn, tabs[pos - n:pos - n + 4])
        for l in range(layers):
            cache.attn_verify(l, 0, pos, q[l], out[l])
        if s >= warmup:
            nbytes += layers * (pos + 4) * per_pos
        pos += 2
        cache.truncate(pos)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    hbm, _, kind = peaks()
    gbs = nbytes / (ms * 1e-3) / 1e9
    cache.close()
    return {"workload": f"verify262k_{fmt.name.lower()}", "context_tokens": n, "layers": layers, "steps": steps,
            "us_per_launch": 1e3 * ms / (steps * layers), "value": gbs, "unit": "GB/s", "frac": gbs / hbm, "peak": hbm,
            "peak_kind": kind, "kernel": "verify_f16_tc_kernel" if fmt == kv.KvFormat.F16 else "verify_f32_tc_kernel",
            "traffic": None if fmt == kv.KvFormat.F16 else NCU_TRAFFIC_BYTES_VERIFY262K_F32,
            "note": "whole loop: one append launch per step + the attention launches, inputs resident"}


def measure_step65k(ctx, stream, steps, warmup):
    import torch
    from mechta_b200 import kv, synth
    ctx0 = 65536
    cache = kv.KvCache(ctx, kv.KvFormat.F16, N_LAYERS, (ctx0 + 4 * (steps + warmup) + 8 + 1023) // 1024 * 1024)
    g = torch.Generator(device="cuda"); g.manual_seed(7)
    for l in range(N_LAYERS):  # synthetic rows written straight into the buffers
        k, v = cache.buffer_tensors(l)
        k[:ctx0].normal_(generator=g); v[:ctx0].normal_(generator=g)
    cache.set_len(ctx0)
    ctx.sync()
    ring = 8
    qf = torch.randn(ring, N_LAYERS, 4, 16, 512, device="cuda", generator=g)
    kb = torch.randn(ring, N_LAYERS, 4, 2, 256, device="cuda", generator=g)
    vb = torch.randn(ring, N_LAYERS, 4, 512, device="cuda", generator=g)
    qw = 1.0 + 0.1 * torch.randn(N_LAYERS, 256, device="cuda", generator=g)
    kw = 1.0 + 0.1 * torch.randn(N_LAYERS, 256, device="cuda", generator=g)
    tabs = torch.from_numpy(kv.rope_table(ctx0, 4 * (steps + warmup) + 8)).cuda()
    out16 = torch.empty(N_LAYERS, 4, 16, 256, device="cuda", dtype=torch.float16)
    acc = synth.accept_counts(11, steps + warmup)

    def step(s, pos):
        r = s % ring
        tab = tabs[pos - ctx0:pos - ctx0 + 4]
        for l in range(N_LAYERS):
            cache.attn_step(l, 0, pos, qf[r, l], kb[r, l], vb[r, l], qw[l], kw[l], tab, None, out16[l])
        new_len = pos + 1 + int(acc[s])
        cache.truncate(new_len)
        return new_len

    pos = ctx0
    for s in range(warmup):
        pos = step(s, pos)
    torch.cuda.synchronize()
    n0 = ctx.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    total = 0
    e0.record(stream)
    for s in range(warmup, warmup + steps):
        total += N_LAYERS * (pos + 4) * 2048
        pos = step(s, pos)
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    hbm, _, kind = peaks()
    value = total / (ms * 1e-3) / 1e9
    launches = ctx.launches - n0
    cache.close()
    return {"workload": "step65k", "value": value, "unit": "GB/s", "ms_per_step": ms / steps, "steps": steps,
            "frac": value / hbm, "peak": hbm, "peak_kind": kind, "launches_per_step": launches // steps,
            "reference_dispatches_per_step": 9 * N_LAYERS, "gpu_launches": launches,
            "fused": "rmsnorm(q,k) + rope2 + kv_rope2 + kv_copy | attention + merge + attn_gate16, per layer"}


def measure_prefill(ctx, stream, steps, warmup, block=2048):
    import torch
    from mechta_b200 import kv
    prefix = 32768
    cache = kv.KvCache(ctx, kv.KvFormat.F16, N_LAYERS, (prefix + block + 1023) // 1024 * 1024)
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    for p in range(0, prefix, 8192):  # the prefix, written once through the append kernel, then snapshotted
        k = torch.randn(N_LAYERS, 8192, 2, 256, device="cuda", generator=g)
        v = torch.randn(N_LAYERS, 8192, 2, 256, device="cuda", generator=g)
        cache.append_layers(p, k, v, torch.from_numpy(kv.rope_table(p, 8192)).cuda())
    del k, v
    root_snap = cache.read_root(prefix)
    back = torch.empty(cache.snapshot_bytes(prefix + block), dtype=torch.uint8, pin_memory=True)
    # f16 queries, as the configuration states (the reference's q_f16 output)
    q = torch.randn(N_LAYERS, block, 16, 256, device="cuda", generator=g).half()
    kn = torch.randn(N_LAYERS, block, 2, 256, device="cuda", generator=g)
    vn = torch.randn(N_LAYERS, block, 2, 256, device="cuda", generator=g)
    tab = torch.from_numpy(kv.rope_table(prefix, block)).cuda()
    out = torch.empty(N_LAYERS, block, 16, 256, device="cuda")
    flops = 4 * 16 * 256 * sum(prefix + t + 1 for t in range(block)) * N_LAYERS
    ev = lambda: torch.cuda.Event(enable_timing=True)
    t_restore = t_attn = t_snap = t_all = 0.0
    n0 = 0
    for s in range(warmup + steps):
        if s == warmup:
            n0 = ctx.launches
        e = [ev() for _ in range(5)]
        e[0].record(stream)
        cache.truncate(0)
        cache.write_root(root_snap)
        e[1].record(stream)
        cache.append_layers(prefix, kn, vn, tab)
        e[2].record(stream)
        for l in range(N_LAYERS):
            cache.attn_prefill(l, 0, prefix, q[l], out[l])
        e[3].record(stream)
        cache.read_root(prefix + block, payload=back, wait=True)
        e[4].record(stream)
        torch.cuda.synchronize()
        if s >= warmup:
            t_restore += e[0].elapsed_time(e[1]); t_attn += e[2].elapsed_time(e[3])
            t_snap += e[3].elapsed_time(e[4]); t_all += e[0].elapsed_time(e[4])
    _, tf, kind = peaks()
    ach = flops * steps / (t_attn * 1e-3) / 1e12
    res = {"workload": "prefill", "value": ach, "unit": "TFLOP/s", "steps": steps, "ms_per_step": t_all / steps,
           "frac": ach / tf, "peak": tf, "peak_kind": kind, "bound": "tensor", "kernel": "prefill_f16_tc_kernel",
           "prefix_tokens": prefix, "block_tokens": block, "q": "f16", "attn_ms_per_layer": t_attn / steps / N_LAYERS,
           "restore_gbs": root_snap.payload.numel() * steps / (t_restore * 1e-3) / 1e9,
           "snapshot_gbs": back.numel() * steps / (t_snap * 1e-3) / 1e9,
           "e2e": {"value": flops * steps / (t_all * 1e-3) / 1e12, "unit": "TFLOP/s",
                   "h2d_bytes_per_step": root_snap.payload.numel(), "d2h_bytes_per_step": back.numel()},
           "gpu_launches": ctx.launches - n0}
    cache.close()
    return res


def measure_sessions(ctx, stream, world, rank, steps, warmup):
    """The 32 sessions of the multi-session configuration placed on `world` ranks; this rank runs its own."""
    import torch
    from mechta_b200 import kv, synth
    from mechta_b200.sharded import place_sessions
    lens = [int(x) for x in synth.session_lengths(21, 32)]
    mine = place_sessions([n * 2048 * N_LAYERS for n in lens], world)[rank]
    room = 4 * (steps + warmup) + 8
    g = torch.Generator(device="cuda"); g.manual_seed(100 + rank)
    caches, pos = [], []
    for i in mine:
        context = min(kv.CTX_MAX, (lens[i] + room + 1023) // 1024 * 1024)
        context = max(context, kv.CTX_MIN)
        c = kv.KvCache(ctx, kv.KvFormat.F16, N_LAYERS, context)
        for l in range(N_LAYERS):  # synthetic rows written straight into the buffers
            k, v = c.buffer_tensors(l)
            k[:lens[i]].normal_(generator=g); v[:lens[i]].normal_(generator=g)
        c.set_len(lens[i])
        caches.append(c); pos.append(lens[i])
    ctx.sync()
    ns = len(mine)
    q = torch.randn(ns, N_LAYERS, 4, 16, 256, device="cuda", generator=g)
    kn = torch.randn(ns, N_LAYERS, 4, 2, 256, device="cuda", generator=g)
    vn = torch.randn(ns, N_LAYERS, 4, 2, 256, device="cuda", generator=g)
    out = torch.empty(ns, N_LAYERS, 4, 16, 256, device="cuda")
    tabs = [torch.from_numpy(kv.rope_table(pos[j], room)).cuda() for j in range(ns)]
    acc = [synth.accept_counts(50 + i, steps + warmup) for i in mine]

    def step(s):
        nbytes = 0
        for j, c in enumerate(caches):
            o = pos[j] - lens[mine[j]]
            c.append_layers(pos[j], kn[j], vn[j], tabs[j][o:o + 4])
            nbytes += N_LAYERS * (pos[j] + 4) * 2048
        for l in range(N_LAYERS):
            ctx.attn_verify_batch([(caches[j], l, 0, pos[j], q[j, l], out[j, l]) for j in range(ns)])
        for j, c in enumerate(caches):
            pos[j] += 1 + int(acc[j][s])
            c.truncate(pos[j])
        return nbytes

    for s in range(warmup):
        step(s)
    _barrier(torch, world)
    n0 = ctx.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    total = sum(step(s) for s in range(warmup, warmup + steps))
    e1.record(stream)
    _barrier(torch, world)
    ms = _reduce(torch, world, e0.elapsed_time(e1), "max")
    tot_bytes = _reduce(torch, world, total, "sum")
    kvb = _reduce(torch, world, sum(lens[i] for i in mine) * 2048 * N_LAYERS, "max")
    launches = ctx.launches - n0
    for c in caches:
        c.close()
    hbm, _, kind = peaks()
    value = tot_bytes / (ms * 1e-3) / 1e9
    mean_b = sum(lens) * 2048 * N_LAYERS / world
    return {"workload": "sessions", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "ms_per_step": ms / steps,
            "sessions": 32, "lengths": "uniform [1024, 131072], seed 21", "placement": "greedy by KV bytes",
            "imbalance_max_over_mean": kvb / mean_b, "kernel": "verify_f16_tc_kernel (ragged batch, one launch per layer)",
            "frac": value / world / hbm, "peak": hbm, "peak_kind": kind, "gpu_launches": launches}


def fill_rows_by_position(torch, cache, layers, lo, hi, seed, dev, chunk=8192):
    """Seeded N(0,1) K/V rows [lo, hi) through the library's append (RoPE on K). A row's values depend on its global
    position and layer only, whichever cache or rank holds it: whole chunks are drawn and the part inside [lo, hi) used.
    `layers` = the layer indices of the full model this cache's layers stand for."""
    from mechta_b200 import kv
    for p0 in range(lo // chunk * chunk, hi, chunk):
        a, b = max(p0, lo), min(p0 + chunk, hi)
        if b <= a:
            continue
        g = torch.Generator(device=dev)
        ks, vs = [], []
        for l in layers:
            g.manual_seed(seed * 1000003 + l * 4099 + p0 // chunk)
            ks.append(torch.randn(chunk, 2, 256, device=dev, generator=g)[a - p0:b - p0])
            vs.append(torch.randn(chunk, 2, 256, device=dev, generator=g)[a - p0:b - p0])
        k, v = torch.stack(ks).contiguous(), torch.stack(vs).contiguous()
        cache.append_layers(a, k, v, torch.from_numpy(kv.rope_table(a, b - a)).to(dev))


def measure_longctx(ctx, stream, world, rank, local, group, steps, warmup, exchange="p2p", context=0, regions=3):
    """Sequence-sharded decode over an f32 cache (world >= 1; world = 1 is the unsharded context)."""
    import torch
    from mechta_b200 import kv, synth
    from mechta_b200.sharded import ShardedKvCache
    dev = f"cuda:{local}"
    fmt, per_pos = kv.KvFormat.F32, 4096
    context = kv.check_ctx(context or kv.CTX_MAX)
    ctx0 = context - 4 * (steps + warmup) - 8  # the run ends at the last rows of the context
    accepts = synth.accept_counts(11, steps + warmup)
    sharded = ShardedKvCache(ctx, fmt, N_LAYERS, context, group, exchange=exchange) if world > 1 else None
    cache = sharded.cache if sharded else kv.KvCache(ctx, fmt, N_LAYERS, context)
    first = cache.shard_first
    fill_rows_by_position(torch, cache, range(N_LAYERS), first, max(first, min(ctx0, first + cache.capacity)), 100, dev)
    ctx.sync()
    g = torch.Generator(device=dev); g.manual_seed(5)
    ring = 8
    q = torch.randn(ring, N_LAYERS, 4, 16, 256, device=dev, generator=g)
    kn = torch.randn(ring, N_LAYERS, 4, 2, 256, device=dev, generator=g)
    vn = torch.randn(ring, N_LAYERS, 4, 2, 256, device=dev, generator=g)
    tabs = torch.from_numpy(kv.rope_table(ctx0, 4 * (steps + warmup) + 8)).to(dev)
    out = torch.empty(N_LAYERS, 4, 16, 256, device=dev)
    rec = torch.empty(64, 258, device=dev)

    def attn(layer, pos, qq, o):
        if sharded:
            sharded.attn_verify(layer, 0, pos, qq, o)
        else:
            cache.attn_verify(layer, 0, pos, qq, o)

    def one_step(s, pos, kernel_only=False):
        r = s % ring
        cache.append_layers(pos, kn[r], vn[r], tabs[pos - ctx0:pos - ctx0 + 4])
        for l in range(N_LAYERS):
            if kernel_only and sharded:
                cache.attn_verify_partial(l, 0, pos, q[r, l], rec)  # this shard's record, nothing exchanged
            else:
                attn(l, pos, q[r, l], out[l])
        new_len = pos + 1 + int(accepts[s])
        cache.truncate(min(new_len, len(cache)))
        return new_len

    def region(kernel_only=False):
        cache.truncate(min(ctx0, len(cache)))
        pos = ctx0
        for s in range(warmup):
            pos = one_step(s, pos, kernel_only)
        _barrier(torch, world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        nbytes = 0
        e0.record(stream)
        for s in range(warmup, warmup + steps):
            nbytes += N_LAYERS * (pos + 4) * per_pos
            pos = one_step(s, pos, kernel_only)
        e1.record(stream)
        _barrier(torch, world)
        return _reduce(torch, world, e0.elapsed_time(e1), "max"), nbytes

    n0 = ctx.launches
    times = []
    for _ in range(regions):
        ms, nbytes = region()
        times.append(ms)
    launches = (ctx.launches - n0) // regions
    sp = spread([t / steps for t in times])
    ms = sp["median"] * steps
    value = nbytes / (ms * 1e-3) / 1e9
    hbm, _, kind = peaks()
    res = {"workload": "longctx", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "ms_per_step": ms / steps,
           "ms_per_step_spread": sp, "scaling": "strong", "context_tokens": ctx0, "cache": "f32", "layers": N_LAYERS,
           "kernel": "verify_f32_tc_kernel", "frac_per_gpu": value / world / hbm, "peak": hbm, "peak_kind": kind,
           "exchange": ("none (one GPU)" if world == 1 else
                        "rows of the record pushed peer to peer over NVLink and merged by the attention kernel's own CTAs"
                        if exchange == "p2p" else "NCCL all-gather of records + merge kernel"),
           "gpu_launches_per_region": launches}
    if world > 1:
        ms_k, _ = region(kernel_only=True)
        res["split_us_per_layer"] = {"kernel_alone": 1e3 * ms_k / steps / N_LAYERS,
                                     "with_exchange": 1e3 * ms / steps / N_LAYERS,
                                     "exchange": 1e3 * (ms - ms_k) / steps / N_LAYERS,
                                     "note": "kernel alone = the same loop with mkv_attn_verify_partial (this shard's record, "
                                             "nothing sent or awaited); max over ranks"}
        # strong-scaling reference and output check: layer 0 of the same rows, unsharded, on rank 0
        cache.truncate(min(ctx0, len(cache)))
        cache.append_layers(ctx0, kn[0], vn[0], tabs[0:4])
        attn(0, ctx0, q[0, 0], out[0])
        torch.cuda.synchronize()
        check, strong_ref = None, None
        if rank == 0:
            whole = kv.KvCache(ctx, fmt, 1, context)
            fill_rows_by_position(torch, whole, [0], 0, ctx0, 100, dev)
            whole.append_layers(ctx0, kn[0, 0:1], vn[0, 0:1], tabs[0:4])
            o1 = torch.empty(4, 16, 256, device=dev)
            for _ in range(3):
                whole.attn_verify(0, 0, ctx0, q[0, 0], o1)
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 20
            g0.record(stream)
            for _ in range(reps):
                whole.attn_verify(0, 0, ctx0, q[0, 0], o1)
            g1.record(stream)
            torch.cuda.synchronize()
            us1 = 1e3 * g0.elapsed_time(g1) / reps
            strong_ref = {"n_gpus": 1, "us_per_layer": us1, "value": (ctx0 + 4) * per_pos / (us1 * 1e-6) / 1e9, "unit": "GB/s",
                          "note": "the same attention launch over the unsharded context on rank 0, one layer"}
            a, b = out[0].double(), o1.double()
            max_rel = float((a - b).abs().max() / b.abs().max())
            check = {"what": "sharded output of layer 0 against the unsharded launch on the same rows and queries",
                     "max_rel": max_rel, "bar": 1e-5, "ok": bool(max_rel < 1e-5 and bool(torch.isfinite(a).all()))}
            whole.close()
        _barrier(torch, world)
        res["strong_ref"] = strong_ref
        res["check"] = check
        if strong_ref:
            res["strong_efficiency"] = strong_ref["us_per_layer"] * 1e-3 * N_LAYERS / (world * ms / steps)
    if sharded:
        sharded.close()
    else:
        cache.close()
    return res
