"""Benchmark workloads beyond the two default bench lines: prefix restore + prefill, and ragged sessions."""
from __future__ import annotations


def run(args, workload):
    raise SystemExit(f"workload {workload!r} is not wired into bench.py yet")
