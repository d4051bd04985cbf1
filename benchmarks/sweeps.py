#!/usr/bin/env python
"""The reference's three published sweeps, on this library.

    python benchmarks/sweeps.py [--sweep batched|single|causal|all] [--csv out.csv] [--quick]

Shapes and dtype follow the reference's ``sweep_all_unified``
(benchmarks/benchmark_colsum.py:289-424 and 757-801): fp16;
batched non-causal H=16 S=1024 D=64 over the batch size; single-sample non-causal
H=16 D=64 over the sequence length; causal H=32 Q=128 D=128 over the key length.
Latency is reported two ways: per call by CUDA events over back-to-back calls
(device time), and the reference's way -- host clock around call + synchronize
(benchmark_colsum.py:42-56).  Peak memory is ``torch.cuda.max_memory_allocated``
around one call (benchmark_colsum.py:59-71), inputs included.  One CSV row per point.
"""

from __future__ import annotations

import argparse
import csv
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

import flash_colsum_b200 as fc  # noqa: E402

SWEEPS = {
    # name: (list of points, builder)
    "batched": [dict(B=b, H=16, Sq=1024, Sk=1024, D=64, causal=False) for b in (8, 16, 32, 64, 128, 256, 512, 1024)],
    "single": [dict(B=1, H=16, Sq=s, Sk=s, D=64, causal=False)
               for s in (4096, 8192, 16384, 32768, 65536, 131072, 262144)],
    "causal": [dict(B=1, H=32, Sq=128, Sk=k, D=128, causal=True)
               for k in (16384, 32768, 65536, 131072, 262144)],
}


def run_point(pt, warmup, iters):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(pt["B"], pt["H"], pt["Sq"], pt["D"], generator=g, device=dev).half()
    k = torch.randn(pt["B"], pt["H"], pt["Sk"], pt["D"], generator=g, device=dev).half()
    call = lambda: fc.flash_colsum(q, k, is_causal=pt["causal"])  # noqa: E731
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        call()
    e1.record()
    torch.cuda.synchronize()
    device_ms = e0.elapsed_time(e1) / iters
    t0 = time.perf_counter()
    for _ in range(iters):
        call()
        torch.cuda.synchronize()
    host_ms = (time.perf_counter() - t0) * 1e3 / iters
    torch.cuda.reset_peak_memory_stats()
    out = call()
    torch.cuda.synchronize()
    peak_gib = torch.cuda.max_memory_allocated() / 2 ** 30
    flop = 4.0 * pt["B"] * pt["H"] * pt["Sq"] * pt["Sk"] * pt["D"]
    row_sum = float(out.sum(dim=1).mean().item())
    assert fc.device_status() == 0
    return {**pt, "device_ms": device_ms, "host_sync_ms": host_ms, "eff_tflops": flop / device_ms / 1e9,
            "peak_mem_gib": peak_gib, "row_sum": row_sum}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", default="all", choices=["all"] + sorted(SWEEPS))
    ap.add_argument("--csv", default=None)
    ap.add_argument("--quick", action="store_true", help="skip the two largest points of every sweep")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    rows = []
    for name in (sorted(SWEEPS) if args.sweep == "all" else [args.sweep]):
        pts = SWEEPS[name][:-2] if args.quick else SWEEPS[name]
        for pt in pts:
            big = pt["B"] * pt["H"] * pt["Sq"] * pt["Sk"] > 3e10
            r = run_point(pt, warmup=2 if big else 10, iters=3 if big else 50)
            r["sweep"] = name
            rows.append(r)
            print(f"{name:8s} B={pt['B']:5d} H={pt['H']} Sq={pt['Sq']:7d} Sk={pt['Sk']:7d} D={pt['D']:3d} "
                  f"device {r['device_ms']:10.3f} ms  host+sync {r['host_sync_ms']:10.3f} ms  "
                  f"{r['eff_tflops']:7.1f} TFLOP/s  peak {r['peak_mem_gib']:.2f} GiB  rowsum {r['row_sum']:.5f}",
                  flush=True)
    if args.csv:
        with open(args.csv, "w", newline="") as f:
            wr = csv.DictWriter(f, fieldnames=["sweep", "B", "H", "Sq", "Sk", "D", "causal", "device_ms",
                                               "host_sync_ms", "eff_tflops", "peak_mem_gib", "row_sum"])
            wr.writeheader()
            wr.writerows(rows)


if __name__ == "__main__":
    main()
