#!/usr/bin/env python
"""The reference's three published sweeps, on this library.

    python benchmarks/sweeps.py [--sweep batched|single|causal|causal_short|configs|all] [--csv out.csv] [--quick]
                                [--with-reference] [--label TEXT]

Shapes and dtype follow the reference's ``sweep_all_unified``
(benchmarks/benchmark_colsum.py:289-424 and 757-801): fp16;
batched non-causal H=16 S=1024 D=64 over the batch size; single-sample non-causal
H=16 D=64 over the sequence length; causal H=32 Q=128 D=128 over the key length (and,
as `causal_short`, the same shape from 1024 to 8192 keys, below the reference's axis).
Latency is reported two ways: per call by CUDA events over back-to-back calls (device time; the median of five
groups of calls), and the reference's way -- host clock around call + synchronize
(benchmark_colsum.py:42-56).  Peak memory is ``torch.cuda.max_memory_allocated``
around one call (benchmark_colsum.py:59-71), inputs included.  One CSV row per point.

``--with-reference`` times, on the same GPU and the same inputs, what the reference's own
benchmark puts side by side (benchmark_colsum.py:199-286): its Triton ``flash_colsum`` and its
materialising ``naive_colsum``, both imported unmodified from an install of the reference in
``baseline/_ref`` (``python -m pip install --no-index --no-build-isolation --no-deps --target
baseline/_ref <checkout>``).  Points whose score matrix would not fit are evaluated in chunks of
batch entries or query rows, as the reference's benchmark does past its first out-of-memory
point (benchmark_colsum.py:74-196), and flagged.  These are baseline legs: nothing under
``flash_colsum_b200/`` imports the reference.  ``ref_triton_rel_l2`` is the distance of the
reference kernel's result from this library's; it is large where the reference's kernels differ
from ``naive_colsum`` (its causal kernel contracts 64 of 128 head dimensions, its non-causal
kernels do not mask ragged keys, its results are fp16).
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
    # the same causal shape below the reference's axis: decode-time calls, bound by launch and ramp
    "causal_short": [dict(B=1, H=32, Sq=128, Sk=k, D=128, causal=True) for k in (1024, 2048, 4096, 8192)],
    # the configurations the headline numbers are quoted on (fp16 here; the long-context one is
    # bf16 with outlier keys in the benchmark proper)
    "configs": [dict(B=8, H=16, Sq=2048, Sk=2048, D=64, causal=False),
                dict(B=32, H=16, Sq=577, Sk=577, D=64, causal=False, cls_len=1),
                dict(B=1, H=32, Sq=128, Sk=4096, D=128, causal=True),
                dict(B=1, H=32, Sq=512, Sk=131072, D=128, causal=True)],
}

SCORE_BUDGET_BYTES = 8 << 30     # largest score matrix the materialising baseline forms in one piece


def load_reference():
    """(flash_colsum, naive_colsum) of the reference installed in baseline/_ref."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flash_colsum")):
        raise SystemExit("--with-reference needs an install of the reference in baseline/_ref (see the docstring)")
    if ref_dir not in sys.path:
        sys.path.append(ref_dir)
    from flash_colsum import flash_colsum as ref_flash, naive_colsum as ref_naive
    return ref_flash, ref_naive


def time_device(call, warmup, iters):
    """Device time of one call: back-to-back calls in up to five groups, each group bracketed by CUDA
    events, the median of the groups' means (one mean over all calls would carry any one-off stall of
    the launching thread that lets the queue run dry)."""
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    groups = min(5, iters)
    per = max(1, iters // groups)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(groups + 1)]
    marks[0].record()
    for g in range(groups):
        for _ in range(per):
            out = call()
        marks[g + 1].record()
    torch.cuda.synchronize()
    means = sorted(marks[g].elapsed_time(marks[g + 1]) / per for g in range(groups))
    return means[groups // 2], out


def naive_in_pieces(ref_naive, q, k, causal, cls_len):
    """The reference's materialising baseline; when the fp32 score matrix exceeds the budget it is
    formed for a few batch entries, or a few hundred query rows, at a time.  Returns (fn, chunked)."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    rows = Sq if cls_len is None else min(cls_len, Sq)
    if B * H * rows * Sk * 4 <= SCORE_BUDGET_BYTES:
        return (lambda: ref_naive(q, k, is_causal=causal, cls_len=cls_len)), False
    per_entry = H * rows * Sk * 4
    if per_entry <= SCORE_BUDGET_BYTES:
        step = max(1, SCORE_BUDGET_BYTES // per_entry)

        def by_batch():
            return torch.cat([ref_naive(q[b:b + step], k[b:b + step], is_causal=causal, cls_len=cls_len)
                              for b in range(0, B, step)], dim=0)
        return by_batch, True
    if causal:
        raise SystemExit("no chunked form for causal points of this size")
    step = max(1, SCORE_BUDGET_BYTES // (H * Sk * 4))

    def by_rows():   # one sample: the reference's function on a few thousand query rows at a time
        acc = torch.zeros(B, Sk, dtype=torch.float32, device=q.device)
        for r0 in range(0, rows, step):
            r1 = min(rows, r0 + step)
            acc += ref_naive(q[:, :, r0:r1], k).float() * ((r1 - r0) / rows)
        return acc
    return by_rows, True



def run_point(pt, warmup, iters, reference=None):
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(pt["B"], pt["H"], pt["Sq"], pt["D"], generator=g, device=dev).half()
    k = torch.randn(pt["B"], pt["H"], pt["Sk"], pt["D"], generator=g, device=dev).half()
    cls_len = pt.get("cls_len")
    call = lambda: fc.flash_colsum(q, k, is_causal=pt["causal"], cls_len=cls_len)  # noqa: E731
    device_ms, _ = time_device(call, warmup, iters)
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
    row = {**pt, "cls_len": cls_len, "device_ms": device_ms, "host_sync_ms": host_ms,
           "eff_tflops": flop / device_ms / 1e9, "peak_mem_gib": peak_gib, "row_sum": row_sum}
    if reference is not None:
        ref_flash, ref_naive = reference
        few = max(1, iters // 5)
        try:
            ms, ref_out = time_device(lambda: ref_flash(q, k, is_causal=pt["causal"], cls_len=cls_len),
                                      min(warmup, 3), few)
            row["ref_triton_ms"] = ms
            row["ref_triton_rel_l2"] = float(((ref_out.float() - out).norm() / out.norm()).item())
            del ref_out
        except Exception as exc:     # the Triton kernels could not compile or run this point
            row["ref_triton_ms"] = None
            row["ref_note"] = f"triton: {type(exc).__name__}"
        try:
            fn, chunked = naive_in_pieces(ref_naive, q, k, pt["causal"], cls_len)
            ms, naive_out = time_device(fn, 1, max(1, few // 2))
            row["ref_naive_ms"] = ms
            row["ref_naive_chunked"] = chunked
            row["ours_rel_l2_vs_naive"] = float(((naive_out.float() - out).norm() / out.norm()).item())
            del naive_out
        except (RuntimeError, SystemExit) as exc:
            row["ref_naive_ms"] = None
            row["ref_note"] = (row.get("ref_note", "") + f" naive: {type(exc).__name__}").strip()
        torch.cuda.empty_cache()
    return row


FIELDS = ["sweep", "B", "H", "Sq", "Sk", "D", "causal", "cls_len", "device_ms", "host_sync_ms", "eff_tflops",
          "peak_mem_gib", "row_sum", "ref_triton_ms", "ref_triton_rel_l2", "ref_naive_ms", "ref_naive_chunked",
          "ours_rel_l2_vs_naive", "ref_note"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", default="all", choices=["all"] + sorted(SWEEPS))
    ap.add_argument("--csv", default=None)
    ap.add_argument("--quick", action="store_true", help="skip the two largest points of every sweep")
    ap.add_argument("--with-reference", action="store_true",
                    help="also time the reference's Triton kernels and materialising baseline (baseline/_ref)")
    ap.add_argument("--label", default="", help="text for the CSV's header line (the commit that produced it)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("needs a CUDA device")
    reference = load_reference() if args.with_reference else None
    rows = []
    for name in (sorted(SWEEPS) if args.sweep == "all" else [args.sweep]):
        pts = SWEEPS[name][:-2] if args.quick and name not in ("configs", "causal_short") else SWEEPS[name]
        for pt in pts:
            big = pt["B"] * pt["H"] * pt["Sq"] * pt["Sk"] > 3e10
            r = run_point(pt, warmup=2 if big else 10, iters=3 if big else 50, reference=reference)
            r["sweep"] = name
            rows.append(r)
            ref = ""
            if reference is not None:
                fmt = lambda v: "     n/a" if v is None else f"{v:10.3f}"  # noqa: E731
                ref = (f"  | reference: triton {fmt(r.get('ref_triton_ms'))} ms, naive {fmt(r.get('ref_naive_ms'))} ms"
                       f"{' (chunked)' if r.get('ref_naive_chunked') else ''}")
            print(f"{name:8s} B={pt['B']:5d} H={pt['H']} Sq={pt['Sq']:7d} Sk={pt['Sk']:7d} D={pt['D']:3d} "
                  f"device {r['device_ms']:10.3f} ms  host+sync {r['host_sync_ms']:10.3f} ms  "
                  f"{r['eff_tflops']:7.1f} TFLOP/s  peak {r['peak_mem_gib']:.2f} GiB  rowsum {r['row_sum']:.5f}{ref}",
                  flush=True)
    if args.csv:
        with open(args.csv, "w", newline="") as f:
            f.write(f"# benchmarks/sweeps.py on {torch.cuda.get_device_name()}; {args.label}\n")
            wr = csv.DictWriter(f, fieldnames=FIELDS, extrasaction="ignore")
            wr.writeheader()
            wr.writerows(rows)


if __name__ == "__main__":
    main()
