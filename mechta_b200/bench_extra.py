"""Benchmark workloads beyond the two default bench lines.

prefill   Prefix-cache restore + prefill: a 32,768-token f16 snapshot of 10 layers is restored from pinned host
          memory, a 2,048-token block is appended and attends to the prefix and to itself (causal), and 34,816 rows are
          snapshotted back. One step = all of that. Reported: attention TFLOP/s against the tensor peak, copy GB/s.
step65k   decode65k with the layer's whole step around the KV path fused (mkv_attn_step): per layer one launch for
          rmsnorm of q and k heads + RoPE + the cache rows, one for attention + merge + output gate, i.e. 20 launches
          per step where the reference's dispatch list has 90.
sessions  32 concurrent sessions with ragged f16 caches (lengths uniform in [1,024, 131,072]), spread over the ranks
          by KV bytes (greedy, longest first), 10 layers, one 4-token verify per session per step with its own accept
          count. No collective: sessions are independent.
"""
from __future__ import annotations

import json
import os

import numpy as np

N_LAYERS = 10


def _peaks(root):
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


def run(args, workload):
    if workload == "prefill":
        return run_prefill(args)
    if workload == "step65k":
        return run_step(args)
    return run_sessions(args)


def run_step(args):
    import torch
    from mechta_b200 import kv, synth
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    steps, warmup, ctx0 = args.steps, args.warmup, 65536
    with torch.cuda.stream(stream):
        ctx = kv.KvContext(0, stream)
        cache = kv.KvCache(ctx, kv.KvFormat.F16, N_LAYERS, (ctx0 + 4 * (steps + warmup) + 8 + 1023) // 1024 * 1024)
        g = torch.Generator(device="cuda"); g.manual_seed(7)
        for l in range(N_LAYERS):  # synthetic rows written straight into the buffers
            k, v = cache.buffer_tensors(l)
            k[:ctx0].normal_(generator=g); v[:ctx0].normal_(generator=g)
        cache.set_len(ctx0)
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
        hbm, _, kind = _peaks(root)
        value = total / (ms * 1e-3) / 1e9
        line = {"metric": "kv_read_gbps", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
                "data": "synthetic",
                "config": {"workload": "step65k", "layers": N_LAYERS, "context_tokens": ctx0, "verify_tokens": 4, "cache": "f16",
                           "fused": "rmsnorm(q,k) + rope2 + kv_rope2 + kv_copy | attention + merge + attn_gate16",
                           "launches_per_step": (ctx.launches - n0) // steps, "reference_dispatches_per_step": 9 * N_LAYERS},
                "roofline": {"bound": "hbm", "kernel": "verify_f16_tc_kernel", "achieved": value, "peak": hbm, "peak_kind": kind,
                             "unit": "GB/s", "frac": value / hbm, "traffic": None},
                "gpu_launches": ctx.launches - n0}
        print(json.dumps(line), flush=True)
        cache.close()


def run_prefill(args):
    import torch
    from mechta_b200 import kv
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    steps, warmup = min(args.steps, 20), min(args.warmup, 3)
    prefix, block = 32768, 2048
    with torch.cuda.stream(stream):
        ctx = kv.KvContext(0, stream)
        cache = kv.KvCache(ctx, kv.KvFormat.F16, N_LAYERS, prefix + block)
        g = torch.Generator(device="cuda"); g.manual_seed(3)
        for p in range(0, prefix, 8192):  # the prefix, written once through the append kernel, then snapshotted
            k = torch.randn(N_LAYERS, 8192, 2, 256, device="cuda", generator=g)
            v = torch.randn(N_LAYERS, 8192, 2, 256, device="cuda", generator=g)
            cache.append_layers(p, k, v, torch.from_numpy(kv.rope_table(p, 8192)).cuda())
        root_snap = cache.read_root(prefix)
        back = torch.empty(cache.snapshot_bytes(prefix + block), dtype=torch.uint8, pin_memory=True)
        q = torch.randn(N_LAYERS, block, 16, 256, device="cuda", generator=g)
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
        hbm, tf, kind = _peaks(root)
        ach = flops * steps / (t_attn * 1e-3) / 1e12
        line = {
            "metric": "prefill_attn_tflops", "value": ach, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": t_all / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16",
            "data": "synthetic",
            "config": {"workload": "prefill", "layers": N_LAYERS, "prefix_tokens": prefix, "block_tokens": block, "cache": "f16"},
            "roofline": {"bound": "tensor", "kernel": "prefill attention", "achieved": ach, "peak": tf, "peak_kind": kind,
                         "unit": "TFLOP/s", "frac": ach / tf, "traffic": None},
            "attn_ms_per_layer": t_attn / steps / N_LAYERS,
            "restore_gbs": root_snap.payload.numel() * steps / (t_restore * 1e-3) / 1e9,
            "snapshot_gbs": back.numel() * steps / (t_snap * 1e-3) / 1e9,
            "e2e": {"value": flops * steps / (t_all * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": root_snap.payload.numel(), "d2h_bytes_per_step": back.numel()},
            "gpu_launches": ctx.launches - n0,
        }
        print(json.dumps(line), flush=True)
        cache.close()


def run_sessions(args):
    import torch
    from mechta_b200 import kv, synth
    from mechta_b200.sharded import place_sessions
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    dev = f"cuda:{local}"
    stream = torch.cuda.Stream(device=dev)
    steps, warmup = min(args.steps, 200), args.warmup
    lens = [int(x) for x in synth.session_lengths(21, 32)]
    mine = place_sessions([n * 2048 * N_LAYERS for n in lens], world)[rank]
    room = 4 * (steps + warmup) + 8
    with torch.cuda.stream(stream):
        ctx = kv.KvContext(local, stream)
        g = torch.Generator(device=dev); g.manual_seed(100 + rank)
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
        ns = len(mine)
        q = torch.randn(ns, N_LAYERS, 4, 16, 256, device=dev, generator=g)
        kn = torch.randn(ns, N_LAYERS, 4, 2, 256, device=dev, generator=g)
        vn = torch.randn(ns, N_LAYERS, 4, 2, 256, device=dev, generator=g)
        out = torch.empty(ns, N_LAYERS, 4, 16, 256, device=dev)
        tabs = [torch.from_numpy(kv.rope_table(pos[j], room)).to(dev) for j in range(ns)]
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
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        n0 = ctx.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        total = sum(step(s) for s in range(warmup, warmup + steps))
        e1.record(stream)
        torch.cuda.synchronize()
        ms, tot_bytes, kvb = e0.elapsed_time(e1), float(total), float(sum(lens[i] for i in mine) * 2048 * N_LAYERS)
        if world > 1:
            t = torch.tensor([ms, 0.0, 0.0], device=dev, dtype=torch.float64)
            dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
            u = torch.tensor([tot_bytes], device=dev, dtype=torch.float64); dist.all_reduce(u)
            w = torch.tensor([kvb], device=dev, dtype=torch.float64); dist.all_reduce(w, op=dist.ReduceOp.MAX)
            ms, tot_bytes, kvb = float(t[0]), float(u[0]), float(w[0])
        if rank == 0:
            hbm, _, kind = _peaks(root)
            value = tot_bytes / (ms * 1e-3) / 1e9
            mean_b = sum(lens) * 2048 * N_LAYERS / world
            line = {"metric": "kv_read_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
                    "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16",
                    "data": "synthetic",
                    "config": {"workload": "sessions", "sessions": 32, "layers": N_LAYERS, "lengths": "uniform [1024, 131072], seed 21",
                               "placement": "greedy by KV bytes", "imbalance_max_over_mean": kvb / mean_b},
                    "roofline": {"bound": "hbm", "kernel": "verify_f16_kernel (ragged batch)", "achieved": value / world, "peak": hbm,
                                 "peak_kind": kind, "unit": "GB/s", "frac": value / world / hbm, "traffic": None},
                    "gpu_launches": ctx.launches - n0}
            print(json.dumps(line), flush=True)
        for c in caches:
            c.close()
    if world > 1:
        dist.destroy_process_group()
