"""Timeline of the decode attention kernel inside a chain of launches, and the per-launch time of that chain.

    make -C mechta_b200/csrc measure                       # builds mechta_b200/libmechta_kv_measure.so (-DMKV_MEASURE)
    python -m mechta_b200.trace_timeline --context 65536   # timeline + microseconds per launch
    python -m mechta_b200.trace_timeline --context 262144 --no-trace   # stock library, per-launch time only

The measurement build makes every CTA of verify_f16_tc_kernel record %globaltimer at its start, after
griddepcontrol.wait, at each batch of MMAs, when its piece is written, in the merge and at its exit. The loop is
the benchmark's: per step one append of 4 rows to all layers, then one verify launch per layer, nothing between
the launches. Times are medians over the CTAs of one launch, in microseconds from the launch's first CTA start.
"""
from __future__ import annotations

import argparse
import ctypes as C
import os

import numpy as np

# one uint64 per name, in the order of struct VtTrace in csrc/verify_tc.cu
NAMES = (["launch", "cta", "sm", "nt", "ticket", "start", "wait_done", "q_ready", "piece", "exit", "fin_ticket", "fin_seen",
          "fin_merged", "fin_loads", "fin_max", "fin_summed", "t0_scores", "t0_scaled", "t0_votes", "t0_reduced", "t0_moved", "t0_weights"]
         + [f"st_issued{i}" for i in range(8)] + [f"softmax_done{i}" for i in range(8)] + [f"ot_issued{i}" for i in range(8)])
COL = {n: i for i, n in enumerate(NAMES)}
FIELDS = len(NAMES)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--context", type=int, default=65536)
    ap.add_argument("--layers", type=int, default=10)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--no-trace", action="store_true", help="use the stock library: per-launch time only")
    args = ap.parse_args()

    import torch
    from mechta_b200 import _lib
    if not args.no_trace:
        so = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libmechta_kv_measure.so")
        if not os.path.exists(so):
            raise SystemExit("build the trace library first: make -C mechta_b200/csrc measure")
        _lib.SO_PATH = so
    from mechta_b200 import kv

    torch.cuda.set_device(0)
    st = torch.cuda.Stream()
    n, nl = args.context, args.layers
    with torch.cuda.stream(st):
        ctx = kv.KvContext(0, st)
        lib = _lib.lib()
        cache = kv.KvCache(ctx, kv.KvFormat.F16, nl, min(kv.CTX_MAX, n + 1024))
        n = min(n, cache.capacity - 64)
        for l in range(nl):
            k, v = cache.buffer_tensors(l)
            k.normal_(); v.normal_()
        cache.set_len(n)
        ctx.sync()  # the rows are in place: later launches may load them early
        q = torch.randn(nl, 4, 16, 256, device="cuda")
        out = torch.empty_like(q)
        kn = torch.randn(nl, 4, 2, 256, device="cuda")
        vn = torch.randn(nl, 4, 2, 256, device="cuda")
        pos = n

        def step(pos):
            cache.append_layers(pos, kn, vn, torch.from_numpy(kv.rope_table(pos, 4)).cuda())
            for l in range(nl):
                cache.attn_verify(l, 0, pos, q[l], out[l])
            cache.truncate(pos + 2)
            return pos + 2

        for _ in range(5):
            pos = step(pos)
        torch.cuda.synchronize()
        buf = np.zeros((65536, FIELDS), dtype=np.uint64)
        if not args.no_trace:
            lib.mkv_trace_read.restype = C.c_int
            lib.mkv_trace_read(buf.ctypes.data_as(C.c_void_p), 65536)  # drop the warm-up records
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(st)
        for _ in range(args.steps):
            pos = step(pos)
        e1.record(st)
        torch.cuda.synchronize()
        print(f"context {n}: {1e3 * e0.elapsed_time(e1) / (args.steps * nl):.2f} us per launch (append included), "
              f"{n * 2048 * args.steps * nl / e0.elapsed_time(e1) / 1e6:.0f} GB/s")
        if args.no_trace:
            return
        cnt = lib.mkv_trace_read(buf.ctypes.data_as(C.c_void_p), 65536)
        r = buf[:cnt].astype(np.int64)
        launches = sorted(set(r[:, COL["launch"]].tolist()))
        prev_t0 = None
        for la in launches[-4:]:
            x = r[r[:, COL["launch"]] == la]
            t0 = x[:, COL["start"]].min()
            us = lambda name, rows=x: (rows[:, COL[name]] - t0) / 1e3
            med = lambda name, rows=x: float(np.median(us(name, rows)))
            period = (t0 - prev_t0) / 1e3 if prev_t0 is not None else float("nan")
            prev_t0 = t0
            nt = int(np.bincount(x[:, COL["nt"]]).argmax())
            full = x[x[:, COL["nt"]] == nt]
            last = f"ot_issued{min(nt, 8) - 1}"
            print(f"launch (ticket base {la}): {len(x)} CTAs, period {period:.2f}")
            print(f"  start med {med('start'):.2f} max {us('start').max():.2f} | wait returns med {med('wait_done'):.2f} | "
                  f"Q ready med {med('q_ready'):.2f} | first S^T med {med('st_issued0', full):.2f} | "
                  f"last O^T med {med(last, full):.2f} max {us(last, full).max():.2f} | last piece {us('piece').max():.2f} | "
                  f"exit med {med('exit'):.2f} max {us('exit').max():.2f}")
            m = x[x[:, COL["ticket"]] >= len(x) - min(len(x), 64)]  # the last arrivals merge
            if len(m):
                print(f"  {len(m)} merging CTAs: ticket med {med('fin_ticket', m):.2f} max {us('fin_ticket', m).max():.2f} | "
                      f"all pieces published med {med('fin_seen', m):.2f} max {us('fin_seen', m).max():.2f} | "
                      f"loads issued med {med('fin_loads', m):.2f} max {us('fin_loads', m).max():.2f} | maximum known med {med('fin_max', m):.2f} | "
                      f"pieces summed med {med('fin_summed', m):.2f} | merged med {med('fin_merged', m):.2f} max {us('fin_merged', m).max():.2f}")
            print("  first tile: scores seen %.2f | read and scaled %.2f | votes %.2f | maxima reduced %.2f | references moved %.2f | "
                  "weights start %.2f" % tuple(med(n, full) for n in ("t0_scores", "t0_scaled", "t0_votes", "t0_reduced", "t0_moved", "t0_weights")))
            for title, stem in (("S^T issued", "st_issued"), ("softmax done", "softmax_done"), ("O^T issued", "ot_issued")):
                print(f"  {title:13s}", " ".join(f"{med(stem + str(j), full):6.2f}" for j in range(min(nt, 8))))


if __name__ == "__main__":
    main()
