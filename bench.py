"""Benchmark of the KV-cache / attention hot path.

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

The default line, at every N: decode65k, the steady-state decode configuration. 10 attention layers, f16 cache at
65,536 tokens, one 4-token verify step = append of the 4 new rows (one launch for all layers' rows), verify attention
per layer, rollback of the refused drafts (accepted count uniform in 0..3 from a fixed seed). With N > 1 every rank
runs its own session of that shape (sessions are independent: no collective on the data path, "weak" scaling) and
the value is the sum over the ranks. The line also carries, under `other_workloads`, short measurements of the
other configurations: at N = 1 the same kernel at 262,144 tokens (f16 and f32 cache), the 32-session batch, the
fused layer step and the prefix-restore + prefill configuration; at N > 1 the sequence-sharded 262,144-token
context (f32 cache, "strong" scaling, with its own reference, efficiency and output check) and the 32 sessions
spread over the ranks. --workload longctx|sessions|prefill|step65k prints one of those as a line of its own.

One JSON line is printed by rank 0. `value` = algorithmic KV bytes read by the attention of all ranks per second
of the whole step loop (append + attention + merge + rollback), inputs already in HBM: the K steps are timed
`regions` times from the same starting state and the line reports the median region (all of them under
`repeats`). `e2e` = the same loop driven through the public API from pinned host buffers with the step's result
read back every step. The reference arm (--impl reference) times the CPU restatement of the reference's kernels
(the reference is Rust + wgpu/Vulkan and does not build here) on all host cores, on a bounded sample of the same
workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_LAYERS = 10
KV_BYTES_F16, KV_BYTES_F32 = 2048, 4096  # K + V bytes per position per layer
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of verify_f16_tc_kernel at the decode65k shape, from an ncu
# capture of that kernel (134.6 MB read + 4.2 MB written: split-K pieces and the output)
NCU_TRAFFIC_BYTES_DECODE65K = 138_800_000
REGIONS = 5


def decode65k_config(world: int) -> dict:
    """`config` of the default line, the same for this repository's arm and for the reference arm."""
    return {"workload": "decode65k", "layers": N_LAYERS, "context_tokens": 65536, "verify_tokens": 4, "cache": "f16",
            "accept": "uniform 0..3 per step from a fixed seed",
            "append": "the 4 new rows of all layers in one launch per step, then one attention launch per layer "
                      "(other_workloads.step65k writes each layer's rows just before its attention)",
            "parallelism": "single GPU" if world == 1 else
                           f"{world} independent sessions of this shape, one per GPU, no collective on the data path",
            "l2": "inputs larger than L2: every layer's K+V exceeds 126 MB and 9 other layers are read between reuses"}


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with NVML while a timed region runs (read-only)."""

    def __init__(self, index: int, period: float = 0.01):
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4,
                 "hw_power_brake": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                try:
                    r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------------------------
# the reference arm: CPU restatement of the reference's kernels on the host cores
# ------------------------------------------------------------------------------------------------------------------

def host_cache(oracle, fmt, rows, seed):
    """One layer of seeded K/V rows appended through the oracle's writers (RoPE on K)."""
    from mechta_b200 import synth
    kc, vc = oracle.new_cache(fmt, rows + 64), oracle.new_cache(fmt, rows + 64)
    for p in range(0, rows, 4096):
        n = min(4096, rows - p)
        oracle.append(fmt, kc, vc, p, synth.normal(seed, synth.S_K, p, (n, 2, 256)), synth.normal(seed, synth.S_V, p, (n, 2, 256)),
                      oracle.rope_tables(p, n))
    return kc, vc


def cpu_layer_step(oracle, fmt, kc, vc, pos, seed, step):
    """One layer of one verify step on the CPU: append 4 rows, attention of 4 tokens, (rollback is a length)."""
    from mechta_b200 import synth
    k = synth.normal(seed, synth.S_KNEW, step, (4, 2, 256))
    v = synth.normal(seed, synth.S_VNEW, step, (4, 2, 256))
    q = synth.normal(seed, synth.S_Q, step, (4, 16, 256))
    tab = oracle.rope_tables(pos, 4)
    t0 = time.perf_counter()
    oracle.append(fmt, kc, vc, pos, k, v, tab)
    oracle.attn_ref_f32(fmt, kc, vc, 0, pos, q)
    return time.perf_counter() - t0


def run_reference(args):
    """--impl reference: the oracle (a port: the reference has no CPU path and does not build here).

    A step is one layer of one verify step (append 4 rows + attention of 4 tokens) over the last `window`
    positions of the context; the window is the whole context when K such steps fit the time budget, else it
    is cut so that warm-up + K steps end within about 15 seconds. Bytes are counted for the window actually read.
    All host cores are used whatever OMP_NUM_THREADS the launcher exported."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from mechta_b200 import synth
    from oracle import oracle
    oracle.build()
    cores = oracle.use_all_cores()
    workload = args.workload or "decode65k"
    if workload == "longctx":
        fmt, ctx_len, per_pos = 1, 262144 - 4 * (args.steps + args.warmup) - 8, KV_BYTES_F32
    else:
        workload, fmt, ctx_len, per_pos = "decode65k", 0, 65536, KV_BYTES_F16
    kc, vc = host_cache(oracle, fmt, ctx_len + (args.steps + args.warmup) + 8, 7)
    pos = ctx_len
    t1 = cpu_layer_step(oracle, fmt, kc, vc, pos, 7, 0)          # untimed: sizes the window
    t1 = min(t1, cpu_layer_step(oracle, fmt, kc, vc, pos, 7, 1))
    budget = 15.0
    frac = min(1.0, budget / max(t1 * (args.steps + args.warmup), 1e-9))
    window = max(4096, int(ctx_len * frac) // 128 * 128)

    def step(s, pos):
        k = synth.normal(7, synth.S_KNEW, s, (4, 2, 256))
        v = synth.normal(7, synth.S_VNEW, s, (4, 2, 256))
        q = synth.normal(7, synth.S_Q, s, (4, 16, 256))
        tab = oracle.rope_tables(pos, 4)
        first = max(0, pos + 4 - window)
        t0 = time.perf_counter()
        oracle.append(fmt, kc, vc, pos, k, v, tab)
        oracle.attn_ref_f32(fmt, kc, vc, first, pos, q)
        return time.perf_counter() - t0, (pos + 4 - first) * per_pos

    for s in range(args.warmup):
        step(s, pos)
    t, nbytes = 0.0, 0
    for s in range(args.steps):
        dt, nb = step(args.warmup + s, pos)
        t += dt
        nbytes += nb
        pos += 1
    gbs = nbytes / t / 1e9
    sample = (f"{args.steps} layer-steps of {workload} over the last {window} of {ctx_len} positions "
              f"(1 of {N_LAYERS} layers per step), OpenMP on {cores} threads")
    line = {
        "impl": "reference", "metric": "kv_read_gbps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps, "higher_is_better": True,
        "scaling": "weak" if workload == "decode65k" else "strong", "vs_baseline": None,
        "dtype": "f32 math over an %s cache" % ("f16" if fmt == 0 else "f32"), "data": "synthetic",
        "config": decode65k_config(max(1, args.gpus)) if workload == "decode65k" else
                  {"workload": workload, "context_tokens": ctx_len, "layers": N_LAYERS, "verify_tokens": 4, "cache": "f32"},
        "reference_sample": {"window_tokens": window, "context_tokens": ctx_len,
                             "note": "a step of this arm is one layer-step (1 of the 10 layers) over the sampled window, on the "
                                     "host cores of one process whatever --gpus says"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------------------

class StepInputs:
    """A ring of distinct step inputs on the device (q, new k, new v for all layers) and the RoPE tables of every
    position the run can reach, so that the device-resident loop touches no host memory."""

    def __init__(self, torch, device, seed, ring, pos0, max_pos):
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        self.ring = ring
        self.q = torch.randn(ring, N_LAYERS, 4, 16, 256, device=device, generator=g)
        self.k = torch.randn(ring, N_LAYERS, 4, 2, 256, device=device, generator=g)
        self.v = torch.randn(ring, N_LAYERS, 4, 2, 256, device=device, generator=g)
        from mechta_b200 import kv
        self.pos0 = pos0
        self.tab = torch.from_numpy(kv.rope_table(pos0, max_pos - pos0 + 8)).to(device)

    def tab_at(self, pos):
        return self.tab[pos - self.pos0: pos - self.pos0 + 4]


def fill_cache(torch, cache, rows, seed, device, first=0, chunk=8192):
    """Seeded N(0,1) K/V rows [first, first+rows) for every layer through the library's own append (RoPE on K)."""
    from mechta_b200 import kv
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    for p in range(first, first + rows, chunk):
        n = min(chunk, first + rows - p)
        k = torch.randn(cache.n_layers, n, 2, 256, device=device, generator=g)
        v = torch.randn(cache.n_layers, n, 2, 256, device=device, generator=g)
        tab = torch.from_numpy(kv.rope_table(p, n)).to(device)
        cache.append_layers(p, k, v, tab)


def dist_setup():
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        group = dist.group.WORLD
    return world, rank, local, group


def barrier_sync(torch, world):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(torch, world, x: float) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(torch, world, x: float) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def run_decode65k(args):
    """The default line: decode65k on every rank (one independent session per GPU)."""
    import torch
    import bench_workloads as bw
    from mechta_b200 import kv, synth

    world, rank, local, group = dist_setup()
    dev = f"cuda:{local}"
    stream = torch.cuda.Stream(device=dev)
    steps, warmup = args.steps, args.warmup
    fmt, ctx0, per_pos = kv.KvFormat.F16, 65536, KV_BYTES_F16
    context = min(kv.CTX_MAX, 65536 + 1024 * ((4 * (steps + warmup) + 8 + 1023) // 1024 + 1))
    accepts = synth.accept_counts(11 + rank, steps + warmup)
    others = []

    with torch.cuda.stream(stream):
        ctx = kv.KvContext(local, stream)
        cache = kv.KvCache(ctx, fmt, N_LAYERS, context)
        fill_cache(torch, cache, ctx0, 100 + rank, dev)
        inp = StepInputs(torch, dev, 5 + rank, 8, ctx0, ctx0 + 4 * (steps + warmup) + 8)
        out = torch.empty(N_LAYERS, 4, 16, 256, device=dev)
        ctx.sync()

        def one_step(s, pos):
            r = s % inp.ring
            cache.append_layers(pos, inp.k[r], inp.v[r], inp.tab_at(pos))
            for l in range(N_LAYERS):
                cache.attn_verify(l, 0, pos, inp.q[r, l], out[l])
            new_len = pos + 1 + int(accepts[s])
            cache.truncate(new_len)
            return new_len

        def bytes_of_step(pos):
            # algorithmic KV bytes: rows [0, pos + 4) of K and V per layer
            return N_LAYERS * (pos + 4) * per_pos

        # ---- device-resident loop: warm-up, then the K timed steps, REGIONS times from the same starting state
        # (no per-kernel events inside a region)
        pos = ctx0
        for s in range(warmup):
            pos = one_step(s, pos)
        pos_timed = pos
        region_ms, launches, total_bytes = [], 0, 0
        with ClockSampler(local) as clk:
            for reg in range(REGIONS):
                cache.truncate(pos_timed)
                pos = pos_timed
                barrier_sync(torch, world)
                n0 = ctx.launches
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                total_bytes = 0
                e0.record(stream)
                for s in range(warmup, warmup + steps):
                    total_bytes += bytes_of_step(pos)
                    pos = one_step(s, pos)
                e1.record(stream)
                barrier_sync(torch, world)
                region_ms.append(max_over_ranks(torch, world, e0.elapsed_time(e1)))
                launches = ctx.launches - n0
        clocks = clk.summary()
        rep = bw.spread([t / steps for t in region_ms])
        ms = rep["median"] * steps
        all_bytes = sum_over_ranks(torch, world, float(total_bytes))
        all_launches = int(sum_over_ranks(torch, world, float(launches)))

        # ---- the same steps once more with one pair of CUDA events per step around its 10 attention launches
        # (nothing else runs between them): the dominant kernel's average launch duration for the roofline.
        # A pair per launch would add its own few microseconds to every short kernel.
        prof_steps = min(steps, 200)
        core_ms, core_bytes = 0.0, 0
        for rep_i in range(max(1, min(REGIONS, 200 // max(prof_steps, 1)))):
            cache.truncate(pos_timed)
            pos = pos_timed
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(prof_steps)]
            for i, s in enumerate(range(warmup, warmup + prof_steps)):
                core_bytes += N_LAYERS * (pos + 4) * per_pos
                r = s % inp.ring
                cache.append_layers(pos, inp.k[r], inp.v[r], inp.tab_at(pos))
                pairs[i][0].record(stream)
                for l in range(N_LAYERS):
                    cache.attn_verify(l, 0, pos, inp.q[r, l], out[l])
                pairs[i][1].record(stream)
                pos = pos + 1 + int(accepts[s])
                cache.truncate(pos)
            torch.cuda.synchronize()
            core_ms += sum(a.elapsed_time(b) for a, b in pairs)
            core_n = N_LAYERS * prof_steps * (rep_i + 1)

        # ---- end to end through the public API from pinned host buffers
        e2e_steps = min(steps, 200)
        # one pinned staging row per step: q | k | v | rope table, so that a step's inputs travel in one copy
        nq, nk, nt_ = N_LAYERS * 4 * 16 * 256, N_LAYERS * 4 * 2 * 256, 4 * 64
        hin = torch.empty(inp.ring, nq + 2 * nk + nt_).pin_memory()
        hin[:, :nq + 2 * nk].normal_()
        hout = torch.empty(N_LAYERS, 4, 16, 256).pin_memory()
        din = torch.empty(nq + 2 * nk + nt_, device=dev)
        dq = din[:nq].view(N_LAYERS, 4, 16, 256)
        dk = din[nq:nq + nk].view(N_LAYERS, 4, 2, 256)
        dv = din[nq + nk:nq + 2 * nk].view(N_LAYERS, 4, 2, 256)
        dtab = din[nq + 2 * nk:].view(4, 64)

        # the host keeps the rope table rows of the positions ahead (they depend on the position only), so that a step
        # starts with one small host copy into its staging row instead of computing sines while the GPU waits
        e2e_tab = kv.rope_table(ctx0, 4 * (e2e_steps + min(warmup, 5)) + 8)
        hin_np = hin.numpy()

        def e2e_step(s, pos):
            r = s % inp.ring
            hin_np[r, nq + 2 * nk:] = e2e_tab[pos - ctx0:pos - ctx0 + 4].reshape(-1)
            din.copy_(hin[r], non_blocking=True)
            cache.append_layers(pos, dk, dv, dtab)
            for l in range(N_LAYERS):
                cache.attn_verify(l, 0, pos, dq[l], out[l])
            hout.copy_(out, non_blocking=True)
            stream.synchronize()  # the host reads the step's result before it can sample and accept
            new_len = pos + 1 + int(accepts[s])
            cache.truncate(new_len)
            return new_len

        cache.truncate(ctx0)
        pos = ctx0
        for s in range(min(warmup, 5)):
            pos = e2e_step(s, pos)
        pos_e2e = pos
        e2e_ms, e2e_bytes = [], 0
        for reg in range(REGIONS):
            cache.truncate(pos_e2e)
            pos = pos_e2e
            barrier_sync(torch, world)
            f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e2e_bytes = 0
            f0.record(stream)
            for s in range(e2e_steps):
                e2e_bytes += bytes_of_step(pos)
                pos = e2e_step(s, pos)
            f1.record(stream)
            barrier_sync(torch, world)
            e2e_ms.append(max_over_ranks(torch, world, f0.elapsed_time(f1)))
        e2e_rep = bw.spread([t / e2e_steps for t in e2e_ms])
        e2e_all_bytes = sum_over_ranks(torch, world, float(e2e_bytes))
        h2d = hin[0].numel() * 4
        d2h = hout.numel() * 4
        cache.close()
        del hin, hout, din, inp

        value = all_bytes / (ms * 1e-3) / 1e9
        e2e_value = e2e_all_bytes / (e2e_rep["median"] * e2e_steps * 1e-3) / 1e9
        peak, peak_kind = measured_peaks()
        core_us = 1e3 * core_ms / max(core_n, 1)
        achieved = (core_bytes / max(core_n, 1)) / (core_us * 1e-6) / 1e9 if core_n else 0.0
        core_us_max = max_over_ranks(torch, world, core_us)

        # ---- the other configurations, short runs outside the timed regions above
        if not args.no_other:
            short = max(5, min(steps, 20))
            def guarded(fn, *a, **k):
                try:
                    others.append(fn(*a, **k))
                except Exception as e:  # a workload that does not fit or fails must not take the headline with it
                    others.append({"workload": getattr(fn, "__name__", "?"), "error": f"{type(e).__name__}: {e}"[:300]})
                torch.cuda.empty_cache()
            if world == 1:
                guarded(bw.measure_verify262k, ctx, stream, kv.KvFormat.F16)
                guarded(bw.measure_verify262k, ctx, stream, kv.KvFormat.F32)
                guarded(bw.measure_sessions, ctx, stream, 1, 0, min(short, 10), 3)
                guarded(bw.measure_step65k, ctx, stream, 3 * short, 5)
                guarded(bw.measure_prefill, ctx, stream, 3, 1)
            else:
                guarded(bw.measure_longctx, ctx, stream, world, rank, local, group, short, 3, args.exchange)
                guarded(bw.measure_sessions, ctx, stream, world, rank, short, 3)

        cpu = None
        if rank == 0 and world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline("decode65k", int(fmt), ctx0, per_pos)

        if rank == 0:
            kernel = "verify_f16_kernel" if os.environ.get("MKV_VERIFY") == "mma" else "verify_f16_tc_kernel"
            line = {
                "metric": "kv_read_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
                "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": decode65k_config(world),
                "capacity_tokens": context,
                "hbm_frac_of_8TBps_nominal": value / 8000.0 / world,
                "repeats": {"regions": REGIONS, "ms_per_step": rep,
                            "note": "the K timed steps run `regions` times from the same starting state; "
                                    "ms_per_step and value are the median region, max over ranks per region"},
                "attn_core_us_per_layer": core_us_max,
                "roofline": {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                             "unit": "GB/s", "frac": achieved / peak, "launches_timed": core_n,
                             "traffic": NCU_TRAFFIC_BYTES_DECODE65K,
                             "traffic_note": "dram read + write per launch from the committed ncu capture, not re-measured here"},
                "cpu_baseline": cpu,
                "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "steps": e2e_steps, "ms_per_step": e2e_rep["median"], "ms_per_step_spread": e2e_rep},
                "gpu_launches": all_launches,
                "clocks": clocks,
                "other_workloads": others,
            }
            print(json.dumps(line), flush=True)
        ctx.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_other(args, workload):
    """--workload NAME: one of the other configurations as a line of its own."""
    import torch
    import bench_workloads as bw
    from mechta_b200 import kv
    world, rank, local, group = dist_setup()
    stream = torch.cuda.Stream(device=f"cuda:{local}")
    with torch.cuda.stream(stream):
        ctx = kv.KvContext(local, stream)
        if workload == "longctx":
            r = bw.measure_longctx(ctx, stream, world, rank, local, group, min(args.steps, 200), args.warmup, args.exchange,
                                   args.context)
            metric, dtype, scaling = "kv_read_gbps", "f32", "strong"
        elif workload == "sessions":
            r = bw.measure_sessions(ctx, stream, world, rank, min(args.steps, 200), args.warmup)
            metric, dtype, scaling = "kv_read_gbps", "f16", "strong"
        elif workload == "step65k":
            r = bw.measure_step65k(ctx, stream, args.steps, args.warmup)
            metric, dtype, scaling = "kv_read_gbps", "f16", "weak"
        elif workload == "verify262k":
            r = bw.measure_verify262k(ctx, stream, kv.KvFormat.F32 if args.f32 else kv.KvFormat.F16, steps=min(args.steps, 50))
            metric, dtype, scaling = "kv_read_gbps", "f32" if args.f32 else "f16", "weak"
        else:
            r = bw.measure_prefill(ctx, stream, min(args.steps, 20), min(args.warmup, 3), args.block)
            metric, dtype, scaling = "prefill_attn_tflops", "f16", "weak"
        if rank == 0:
            frac = r.get("frac", r.get("frac_per_gpu"))
            line = {"metric": metric, "value": r["value"], "unit": r["unit"], "n_gpus": world, "steps": r.get("steps", args.steps),
                    "warmup": args.warmup, "ms_per_step": r.get("ms_per_step"), "higher_is_better": True, "scaling": scaling,
                    "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": {"workload": r["workload"]},
                    "roofline": {"bound": r.get("bound", "hbm"), "kernel": r.get("kernel"), "achieved": r["value"] / (world if "frac_per_gpu" in r else 1),
                                 "peak": r.get("peak"), "peak_kind": r.get("peak_kind"), "unit": r["unit"], "frac": frac, "traffic": r.get("traffic")},
                    "gpu_launches": r.get("gpu_launches", r.get("gpu_launches_per_region")), "detail": r}
            if "e2e" in r:
                line["e2e"] = r["e2e"]
            print(json.dumps(line), flush=True)
        ctx.close()
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def cpu_baseline(workload, fmt, ctx0, per_pos):
    """The oracle timed on this host's cores on a bounded sample: layer-steps of the same workload."""
    from oracle import oracle
    oracle.build()
    cores = oracle.use_all_cores()
    max_steps = 400
    kc, vc = host_cache(oracle, fmt, ctx0 + max_steps + 8, 7)  # every step moves on one position and appends 4 rows
    pos, t, n, nbytes = ctx0, 0.0, 0, 0
    cpu_layer_step(oracle, fmt, kc, vc, pos, 7, 0)  # warm
    while t < 10.0 and n < max_steps:
        t += cpu_layer_step(oracle, fmt, kc, vc, pos, 7, n + 1)
        nbytes += (pos + 4) * per_pos
        pos += 1
        n += 1
    return {"value": nbytes / t / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{n} layer-steps of {workload} (1 of {N_LAYERS} layers per step), {t:.1f} s",
            "ms_per_layer_step": 1e3 * t / n}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None,
                    choices=[None, "decode65k", "longctx", "prefill", "sessions", "step65k", "verify262k"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other", action="store_true", help="skip the short runs of the other configurations")
    ap.add_argument("--f32", action="store_true", help="verify262k only: the f32 cache")
    ap.add_argument("--block", type=int, default=2048, help="prefill only: tokens of the prefill block (default 2048)")
    ap.add_argument("--context", type=int, default=0, help="longctx only: context tokens (default 262144); smaller for profiling")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"], help="how shard records travel between ranks")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
        return
    workload = args.workload or "decode65k"
    if workload == "decode65k":
        run_decode65k(args)
    else:
        run_other(args, workload)


if __name__ == "__main__":
    main()
