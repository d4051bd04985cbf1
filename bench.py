#!/usr/bin/env python
"""Benchmark of the attention column mean on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one `flash_colsum` call over one batch of seeded synthetic input.
At one GPU the workload is the batched non-causal headline shape (B=8, H=16,
S=2048, D=64, fp16).  At N GPUs each rank runs that shape on its own batch shard
(weak scaling, no collective: the output is batch-sharded), and the JSON line
also carries the long-context causal shape (131072 keys, 512 suffix queries,
D=128, bf16) with its 32 heads split over the ranks and one NCCL all-reduce of
the fp32 per-key partials (strong scaling) under "causal_long_context", and the reference's
batched sweep shape (B=128 H=16 S=1024 per GPU), which takes the single-pass cluster kernel,
next to the two-pass kernels on the same inputs under "short_key_axis", and a point of the
reference's causal sweep (H=32 Q=128 K=65536 D=128), which is bound by HBM, under "causal_suffix",
the CLIP-style CLS call (B=32 H=16 S=577, cls_len=1; bound by HBM) under "cls_prefix" and the
decode-suffix call (H=32 Q=128 K=4096 D=128; bound by latency: the one-kernel cluster form, with the
three-kernel form timed beside it) under "causal_short".  The
long-context leg carries a "parity" object: its result against a materialising fp32 evaluation
of all heads (every rank evaluates its own heads, the sums meet in one NCCL all-reduce).

Prints ONE JSON line on rank 0.  `--impl reference` times the CPU restatement of
the reference's materialising implementation on the host cores instead.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

from flash_colsum_b200.inputs import WORKLOADS, Workload, make_inputs  # noqa: E402

METRIC = "colsum_effective_tflops"
UNIT = "TFLOP/s"
WORKLOAD_LABEL = "c2: non-causal B=8 H=16 S=2048 D=64 fp16 per GPU"
L2_FLUSH_BYTES = 256 << 20


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"tflops": float(p["bf16_tflops"]), "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


def load_traffic(kernel: str):
    """DRAM bytes per launch of `kernel` from the committed ncu summary, if any."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f).get(kernel)


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


def time_steps(fn, steps, warmup, flush_buf, barrier=None):
    """Per-step CUDA-event timing with an untimed L2 flush before every step."""
    for _ in range(warmup):
        flush_buf.zero_()
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush_buf.zero_()
        starts[i].record()
        fn()
        ends[i].record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    return [s.elapsed_time(e) for s, e in zip(starts, ends)]


def cpu_implementation():
    """The materialising CPU implementation to time: the reference's own ``naive_colsum`` when an
    install of the reference sits in baseline/_ref (flash_colsum/baselines.py:13-78, unmodified),
    else this repository's restatement of it under oracle/."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref_dir, "flash_colsum")):
        try:
            if ref_dir not in sys.path:
                sys.path.append(ref_dir)
            from flash_colsum.baselines import naive_colsum
            return naive_colsum, "reference", "naive_colsum of the reference installed in baseline/_ref"
        except Exception:
            pass
    from oracle.naive_colsum import naive_colsum_torch
    return naive_colsum_torch, "port", "CPU restatement of naive_colsum (oracle/naive_colsum.py)"


def cpu_port_tflops(w: Workload, budget_s: float, batch_entries: int):
    """The CPU implementation of the reference on a bounded sample of `w`."""
    fn, kind, what = cpu_implementation()
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    sample = Workload(w.name + "_sample", min(batch_entries, w.B), w.H, w.Sq, w.Sk, w.D, w.dtype,
                      w.is_causal, w.cls_len, w.key_outliers, w.key_is_query, w.seed)
    q, k = make_inputs(sample)
    q, k = q.float(), k.float()
    fn(q, k, is_causal=w.is_causal, cls_len=w.cls_len)   # warm-up
    times = []
    t_end = time.perf_counter() + budget_s
    while True:
        t0 = time.perf_counter()
        fn(q, k, is_causal=w.is_causal, cls_len=w.cls_len)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() > t_end or len(times) >= 50:
            break
    best = statistics.median(times)
    return {"value": sample.flop / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": kind,
            "sample": (f"{what}: {sample.B} of {w.B} batch entries of {w.name} in fp32, "
                       f"median of {len(times)} calls of {best * 1e3:.1f} ms; host has "
                       f"{os.cpu_count()} logical cores")}, best, sample


def reference_gpu_same_box(w: Workload, steps: int):
    """The reference's own Triton `flash_colsum` (flash_colsum/ops.py:13) on this box's GPU, from
    the install in baseline/_ref: context for the CPU figure, not part of it.  Returns a dict with
    `ms_per_call` and `value`, or with `unavailable`."""
    try:
        if not torch.cuda.is_available():
            return {"unavailable": "no CUDA device"}
        ref_dir = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_dir, "flash_colsum")):
            return {"unavailable": "no install of the reference in baseline/_ref"}
        if ref_dir not in sys.path:
            sys.path.append(ref_dir)
        from flash_colsum import flash_colsum as ref_flash_colsum
        dev = torch.device("cuda", 0)
        q, k = (t.to(dev) for t in make_inputs(w))
        flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
        for _ in range(3):
            ref_flash_colsum(q, k, is_causal=w.is_causal, cls_len=w.cls_len)
        torch.cuda.synchronize()
        n = max(3, min(steps, 20))
        t = time_steps(lambda: ref_flash_colsum(q, k, is_causal=w.is_causal, cls_len=w.cls_len), n, 1, flush)
        ms = sum(t) / len(t)
        return {"what": "reference Triton flash_colsum on cuda:0, same inputs, L2 flushed per call",
                "ms_per_call": ms, "value": w.flop / (ms * 1e-3) / 1e12, "unit": UNIT, "steps": n}
    except Exception as exc:   # Triton could not compile or run here
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS["c2"]
    fn, kind, what = cpu_implementation()
    # all host cores, also under torchrun (which exports OMP_NUM_THREADS=1 to its ranks)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    sample = Workload("c2_sample", 1, w.H, w.Sq, w.Sk, w.D, w.dtype, seed=w.seed)
    q, k = make_inputs(sample)
    q, k = q.float(), k.float()
    for _ in range(max(1, min(args.warmup, 2))):
        fn(q, k)
    times = []
    # one step = one batch entry on the host cores; bounded so that the run ends in minutes
    t_stop = time.perf_counter() + 120.0
    for _ in range(args.steps):
        t0 = time.perf_counter()
        fn(q, k)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() > t_stop:
            break
    mean_s = sum(times) / len(times)
    value = sample.flop / mean_s / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": mean_s * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD_LABEL, "flop_count": "4*B*H*Sq*Sk*D (two passes)",
                   "step": "one batch entry (B=1) of the workload per step, fp32 on the host cores",
                   "l2": "host run"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
                         "sample": f"1 of 8 batch entries per step, {what} in fp32"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if not args.no_gpu_reference:
        line["reference_gpu_same_box"] = reference_gpu_same_box(w, args.steps)
    print(json.dumps(line), flush=True)


def kernel_only(args, fc, _cabi, dev, flush_buf, peaks):
    """Device passes of one workload, per-pass durations; one JSON line."""
    w = WORKLOADS[args.workload]
    if args.batch > 0 or args.keys > 0 or args.queries > 0 or args.heads > 0:
        sq = args.queries or (w.Sq if w.is_causal or not args.keys else args.keys)
        w = Workload(w.name, args.batch or w.B, args.heads or w.H, sq,
                     args.keys or w.Sk, w.D, w.dtype, w.is_causal, w.cls_len,
                     w.key_outliers, w.key_is_query, w.seed)
    g = torch.Generator(device=dev).manual_seed(w.seed)
    q = torch.randn(w.B, w.H, w.Sq, w.D, generator=g, device=dev).to(w.torch_dtype)
    k = torch.randn(w.B, w.H, w.Sk, w.D, generator=g, device=dev).to(w.torch_dtype)

    target = torch.zeros(w.Sk, dtype=torch.float32, device=dev) if args.accumulate else None

    def call():
        if target is not None:   # the entry head-sharded ranks call: adds into a buffer that may be peer-mapped
            return fc.ops._flash_colsum_causal(q, k, 1.0 / w.D ** 0.5, accumulate_into=target)
        return fc.flash_colsum(q, k, is_causal=w.is_causal, cls_len=w.cls_len)

    if args.two_pass:
        _cabi.set_single_pass(_cabi.SINGLE_PASS_NEVER)
    _cabi.set_profiling(True)
    for _ in range(args.warmup):
        flush_buf.zero_()
        call()
    torch.cuda.synchronize()
    rows = []
    for _ in range(args.steps):
        if not args.no_l2_flush:
            flush_buf.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call()
        e1.record()
        torch.cuda.synchronize()
        rows.append((e0.elapsed_time(e1),) + _cabi.last_pass_ms())
    _cabi.set_profiling(False)
    n = len(rows)
    total, st, mg, col = (sum(r[i] for r in rows) / n for i in range(4))
    rows_used = w.rows_averaged
    print(json.dumps({
        "workload": w.name, "B": w.B, "H": w.H, "Sq": w.Sq, "Sk": w.Sk, "D": w.D, "dtype": w.dtype,
        "causal": w.is_causal, "cls_len": w.cls_len, "steps": n, "ms_per_call": total,
        "stats_ms": st, "merge_ms": mg, "colsum_ms": col,
        "tflops_nominal": w.flop / (total * 1e-3) / 1e12,
        "tflops_rows_used": w.flop_rows_used / (total * 1e-3) / 1e12,
        "min_bytes_gbs": w.min_bytes / (total * 1e-3) / 1e9,
        "frac_of_tensor_peak": w.flop / (total * 1e-3) / 1e12 / peaks["tflops"],
        "plan": _cabi.plan_info(w.B, w.H, rows_used, w.Sk, w.is_causal),
        "status": fc.device_status()}), flush=True)


def long_context_parity(q5, k5, w5, out5, world, rank, dev, dist, used_peer, nccl_call):
    """The head-sharded long-context result against a materialising fp32 evaluation of ALL heads:
    every rank evaluates its own heads (two at a time), the un-normalised sums meet in one NCCL
    all-reduce, rank 0 compares.  With the in-kernel peer-memory reduce, also that result
    against the NCCL all-reduce of the same partials."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        h_local, Sq, Sk, D = q5.shape[1], q5.shape[2], k5.shape[2], q5.shape[3]
        acc = torch.zeros(Sk, dtype=torch.float64, device=dev)
        vis = (torch.arange(Sk, device=dev)[None, :] <= (Sk - Sq + torch.arange(Sq, device=dev))[:, None])
        for h0 in range(0, h_local, 2):
            s = torch.matmul(q5[0, h0:h0 + 2].float(), k5[0, h0:h0 + 2].float().transpose(-1, -2)) / D ** 0.5
            s.masked_fill_(~vis, float("-inf"))
            acc += torch.softmax(s, dim=-1).sum(dim=(0, 1), dtype=torch.float64)
            del s
        if dist is not None:
            dist.all_reduce(acc)
        want = acc / (w5.H * Sq)
        got = out5.reshape(-1).double()
        res = {"vs": "fp32 materialised, all heads", "n_gpus": world,
               "rel_l2": float(((got - want).norm() / want.norm()).item()),
               "max_abs": float(((got - want).abs().max() / want.max()).item()),
               "max_abs_unit": "fraction of the largest column mean", "tolerance": 1e-3}
        if used_peer:
            via_nccl = nccl_call().reshape(-1).double()
            res["peer_reduce_vs_nccl_all_reduce"] = {
                "rel_l2": float(((got - via_nccl).norm() / via_nccl.norm()).item()),
                "max_abs": float(((got - via_nccl).abs().max() / via_nccl.max()).item())}
        # only rank 0's figures are printed; with the peer-memory reduce only rank 0 holds the result
        return res
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def small_call_leg(fc, _cabi, w, q, k, steps, flush_buf, barrier, max_over_ranks, peaks):
    """One of the short calls through the public operator: ms per call (L2 flushed before each),
    back-to-back issue rate, and the library's own event times of the device passes."""
    call = lambda: fc.flash_colsum(q, k, is_causal=w.is_causal, cls_len=w.cls_len)
    t = time_steps(call, steps, 3, flush_buf, barrier)
    ms = max_over_ranks(sum(t) / len(t))
    # back to back, no flush: what a caller issuing many such calls sees (host-bound if above the kernel time)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(200):
        call()
    e1.record()
    torch.cuda.synchronize()
    b2b = e0.elapsed_time(e1) / 200
    _cabi.set_profiling(True)
    rows = []
    for _ in range(max(5, steps)):
        flush_buf.zero_()
        call()
        rows.append(_cabi.last_pass_ms())
    _cabi.set_profiling(False)
    st, mg, col = (sum(r[i] for r in rows) / len(rows) for i in range(3))
    return ms, b2b, st, mg, col


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-budget-s", type=float, default=12.0)
    ap.add_argument("--skip-long-context", action="store_true")
    ap.add_argument("--no-gpu-reference", action="store_true",
                    help="reference arm: do not also time the reference's Triton kernels on the GPU")
    ap.add_argument("--nccl-reduce", action="store_true",
                    help="reduce the head-sharded partials with an NCCL all-reduce instead of peer-memory atomics")
    ap.add_argument("--kernel-only", action="store_true",
                    help="time only the device passes of --workload (used for ncu captures)")
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--batch", type=int, default=0, help="override the batch size (kernel-only mode)")
    ap.add_argument("--keys", type=int, default=0, help="override the key length (kernel-only mode)")
    ap.add_argument("--two-pass", action="store_true",
                    help="kernel-only mode: never take the single-pass kernel (time the two streaming passes)")
    ap.add_argument("--accumulate", action="store_true",
                    help="kernel-only mode, causal workloads: call the accumulate entry (combined adds) instead")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (kernel-only mode)")
    ap.add_argument("--queries", type=int, default=0, help="override the query length (kernel-only mode, causal workloads)")
    ap.add_argument("--no-l2-flush", action="store_true",
                    help="kernel-only mode: do not write the 256 MiB buffer between calls (inputs stay in L2)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3

    if args.impl == "reference":
        run_reference_arm(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import flash_colsum_b200 as fc
    from flash_colsum_b200 import _cabi
    from flash_colsum_b200.sharded import flash_colsum_head_sharded, shard_range

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    peaks = load_peaks()
    flush_buf = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)

    if args.kernel_only:
        kernel_only(args, fc, _cabi, dev, flush_buf, peaks)
        return

    # ------------------------------------------------------------ headline workload
    w = WORKLOADS["c2"]
    wr = Workload(w.name, w.B, w.H, w.Sq, w.Sk, w.D, w.dtype, seed=w.seed + rank)   # this rank's batch shard
    q_host, k_host = make_inputs(wr)
    q_host, k_host = q_host.pin_memory(), k_host.pin_memory()
    q, k = q_host.to(dev), k_host.to(dev)
    plan = _cabi.plan_info(w.B, w.H, w.Sq, w.Sk, False)
    launches_per_call = 2 + (1 if plan["nsplit"] > 1 else 0)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    times = time_steps(lambda: fc.flash_colsum(q, k), args.steps, args.warmup, flush_buf, barrier)
    clocks = sampler.stop() if rank == 0 else None
    ms_local = sum(times) / len(times)
    ms_step = max_over_ranks(ms_local)
    value = w.flop * world / (ms_step * 1e-3) / 1e12
    assert fc.device_status() == 0, "a device-side wait expired during the timed region"

    # per-kernel durations (events recorded by the library around each pass)
    _cabi.set_profiling(True)
    stats_ms, col_ms = [], []
    for _ in range(max(5, min(args.steps, 50))):
        flush_buf.zero_()
        fc.flash_colsum(q, k)
        a, _, c = _cabi.last_pass_ms()
        stats_ms.append(a)
        col_ms.append(c)
    _cabi.set_profiling(False)
    col_avg = sum(col_ms) / len(col_ms)
    stats_avg = sum(stats_ms) / len(stats_ms)
    pass_flop = w.flop / 2.0
    # the two kernels do equal halves of the work; the statistics pass is the longer one
    achieved = pass_flop / (stats_avg * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": "colsum_stream_kernel<64, statistics pass>",
        "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved / peaks["tflops"],
        "peak_source": f"{peaks['source']} bf16 burst", "traffic": load_traffic("stats_pass_c2"),
        "traffic_source": ("constant from profiles/dram_traffic.json: one ncu capture of this kernel at "
                           "batch 2 of the same shape, scaled by 4 to the batch of 8 (the traffic is the "
                           "inputs once per pass and grows with the batch)"),
        "launch_ms": stats_avg, "flop_per_launch": pass_flop,
        "other_kernels": {"column pass": {"launch_ms": col_avg,
                                          "achieved": pass_flop / (col_avg * 1e-3) / 1e12,
                                          "traffic": load_traffic("colsum_pass_c2")}},
    }

    # ------------------------------------------------------------ end to end from host memory
    def e2e_step():
        # pinned host tensors in, host tensor out: copies of batch entries overlap the compute
        return fc.flash_colsum_host(q_host, k_host, device=dev)

    e2e_times = []
    for i in range(3 + max(5, min(args.steps // 2, 30))):
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        e2e_step()
        torch.cuda.synchronize()
        if i >= 3:
            e2e_times.append((time.perf_counter() - t0) * 1e3)
    e2e_ms = max_over_ranks(sum(e2e_times) / len(e2e_times))
    e2e = {"value": w.flop * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": int(q_host.numel() * 2 + k_host.numel() * 2),
           "d2h_bytes_per_step": int(w.B * w.Sk * 4)}

    # ------------------------------------------------------------ long-context causal, heads sharded
    long_ctx = None
    if not args.skip_long_context:
        w5 = WORKLOADS["c5"]
        lo, hi = shard_range(w5.H, world, rank)
        g = torch.Generator(device=dev).manual_seed(1234)
        # generated on the device: 1 GiB of keys per 32 heads; same distribution as the CPU generator
        q5 = torch.randn(1, hi - lo, w5.Sq, w5.D, generator=g, device=dev, dtype=torch.float32)
        k5 = torch.randn(1, hi - lo, w5.Sk, w5.D, generator=g, device=dev, dtype=torch.float32)
        k5 *= (torch.rand(w5.Sk, generator=g, device=dev) * 1.5 + 0.5)[None, None, :, None]
        q5, k5 = q5.to(torch.bfloat16), k5.to(torch.bfloat16)

        peer = None
        reduce_kind = "single GPU"
        if world > 1:
            reduce_kind = "one NCCL all-reduce of (1,131072) fp32"
            if not args.nccl_reduce:
                try:
                    from flash_colsum_b200.sharded import PeerAccumulator
                    peer = PeerAccumulator(w5.Sk, dev, dst=0)
                    reduce_kind = ("column-pass atomics into rank 0's peer-mapped (1,131072) fp32 buffer over "
                                   "NVLink; the target alternates between two buffers, rank 0 clears the next one "
                                   "inside its kernels; the last CTA of every rank's column pass posts a flag on rank "
                                   "0, which alone waits (release/acquire flags in peer memory: no collective, no "
                                   "all-to-all barrier, no kernel of its own on the other ranks)")
                except Exception as exc:   # symmetric memory not available: keep the collective
                    peer = None
                    reduce_kind += f" (peer-memory path unavailable: {type(exc).__name__})"

        def long_step():
            return flash_colsum_head_sharded(q5, k5, w5.H, is_causal=True, peer=peer)

        t5 = time_steps(long_step, max(5, min(args.steps // 2, 30)), 3, flush_buf, barrier)
        ms5 = max_over_ranks(sum(t5) / len(t5))
        breakdown5 = None
        if world > 1:
            # where the time of a sharded call goes: this rank's kernels alone (local output), and the
            # device barrier alone
            n_b = max(5, min(args.steps // 2, 30))
            t_loc = time_steps(lambda: fc.ops._flash_colsum_causal(q5, k5, 1.0 / w5.D ** 0.5, h_norm=w5.H), n_b, 3,
                               flush_buf, barrier)
            bd = {"local_kernels_ms": max_over_ranks(sum(t_loc) / len(t_loc))}
            if peer is not None:
                # the flags of a call with nothing to add, issued by one-warp kernels (rank 0 still clears
                # the next buffer); inside a real call they ride in the column pass
                def nothing_to_add(target, clear_next, signals):
                    if signals is not None:
                        return False
                    if clear_next is not None:
                        clear_next.zero_()
                    return True
                t_bar = time_steps(lambda: peer.reduce(nothing_to_add), n_b, 3, flush_buf, barrier)
                bd["flags_alone_ms"] = max_over_ranks(sum(t_bar) / len(t_bar))
            breakdown5 = bd
        out5 = long_step()
        torch.cuda.synchronize()
        parity5 = long_context_parity(q5, k5, w5, out5, world, rank, dev, dist, peer is not None,
                                      lambda: flash_colsum_head_sharded(q5, k5, w5.H, is_causal=True, peer=None))
        long_ctx = {"workload": "c5: causal H=32 Q=512 K=131072 D=128 bf16, outlier keys",
                    "parallelism": f"heads sharded over {world} GPU(s); reduce: {reduce_kind}",
                    "scaling": "strong", "ms_per_call": ms5, "value": w5.flop / (ms5 * 1e-3) / 1e12,
                    "unit": UNIT, "frac_of_peak": w5.flop / (ms5 * 1e-3) / 1e12 / peaks["tflops"],
                    "row_sum_on_rank0": float(out5.sum().item()), "parity": parity5, "breakdown": breakdown5}
        del q5, k5
    assert fc.device_status() == 0

    # ------------------------------------------------------------ short key axis (single-pass kernel)
    # the reference's batched sweep shape (benchmarks/benchmark_colsum.py:289: H=16 S=1024 D=64),
    # B=128 per GPU; takes the single-pass cluster kernel, timed next to the two passes
    short_keys = None
    if not args.skip_long_context:
        ws_ = Workload("batched_s1024", 128, 16, 1024, 1024, 64, "fp16", seed=5 + rank)
        g = torch.Generator(device=dev).manual_seed(ws_.seed)
        qs = torch.randn(ws_.B, ws_.H, ws_.Sq, ws_.D, generator=g, device=dev).to(ws_.torch_dtype)
        ks = torch.randn(ws_.B, ws_.H, ws_.Sk, ws_.D, generator=g, device=dev).to(ws_.torch_dtype)
        n_short = max(5, min(args.steps // 4, 20))
        t_single = time_steps(lambda: fc.flash_colsum(qs, ks), n_short, 3, flush_buf, barrier)
        _cabi.set_single_pass(_cabi.SINGLE_PASS_NEVER)
        t_double = time_steps(lambda: fc.flash_colsum(qs, ks), n_short, 3, flush_buf, barrier)
        _cabi.set_single_pass(_cabi.SINGLE_PASS_AUTO)
        ms_single = max_over_ranks(sum(t_single) / len(t_single))
        ms_double = max_over_ranks(sum(t_double) / len(t_double))
        short_keys = {"workload": "batched non-causal B=128 H=16 S=1024 D=64 fp16 per GPU (inputs 512 MiB)",
                      "kernel": "colsum_single_pass_kernel, clusters of 4" if _cabi.single_pass_applies(
                          ws_.B, ws_.H, ws_.Sk) else "two passes",
                      "ms_per_call": ms_single, "value": ws_.flop * world / (ms_single * 1e-3) / 1e12,
                      "unit": UNIT, "two_pass_ms_per_call": ms_double}
        del qs, ks
    assert fc.device_status() == 0

    # ------------------------------------------------------------ causal suffix queries (short-query column pass)
    # a point of the reference's causal sweep (benchmarks/benchmark_colsum.py:289: H=32 Q=128 D=128):
    # one sweep over the keys per pass, so the bound is HBM -- reported against the copy bandwidth
    suffix = None
    if not args.skip_long_context:
        wq = Workload("causal_q128", 1, 32, 128, 65536, 128, "fp16", is_causal=True, seed=9 + rank)
        g = torch.Generator(device=dev).manual_seed(wq.seed)
        qq = torch.randn(wq.B, wq.H, wq.Sq, wq.D, generator=g, device=dev).to(wq.torch_dtype)
        kq = torch.randn(wq.B, wq.H, wq.Sk, wq.D, generator=g, device=dev).to(wq.torch_dtype)
        n_q = max(5, min(args.steps // 4, 20))
        t_q = time_steps(lambda: fc.flash_colsum(qq, kq, is_causal=True), n_q, 3, flush_buf, barrier)
        ms_q = max_over_ranks(sum(t_q) / len(t_q))
        key_bytes = 2 * kq.numel() * 2      # the keys are read once per pass
        suffix = {"workload": "causal H=32 Q=128 K=65536 D=128 fp16 per GPU (keys 512 MiB)",
                  "ms_per_call": ms_q, "value": wq.flop * world / (ms_q * 1e-3) / 1e12, "unit": UNIT,
                  "roofline": {"bound": "hbm", "achieved": key_bytes / (ms_q * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                               "unit": "GB/s", "frac": key_bytes / (ms_q * 1e-3) / 1e9 / peaks["hbm_gbs"],
                               "bytes": "the keys twice (once per phase of the one-kernel form, or once per streaming pass); the whole call"}}
        del qq, kq
    assert fc.device_status() == 0

    # ------------------------------------------------------------ CLS prefix (C3) and decode suffix (C4)
    cls_prefix = causal_short = None
    if not args.skip_long_context:
        n_small = max(10, min(args.steps // 2, 50))
        w3 = WORKLOADS["c3"]
        q3, k3 = (t.to(dev) for t in make_inputs(Workload(w3.name, w3.B, w3.H, w3.Sq, w3.Sk, w3.D, w3.dtype,
                                                          cls_len=w3.cls_len, seed=w3.seed + rank)))
        ms3, b2b3, _, _, kern3 = small_call_leg(fc, _cabi, w3, q3, k3, n_small, flush_buf, barrier, max_over_ranks, peaks)
        bytes3 = w3.min_bytes     # the keys once, the CLS query rows, the output
        cls_prefix = {"workload": "c3: non-causal B=32 H=16 S=577 D=64 fp16, cls_len=1, per GPU",
                      "kernel": "colsum_small_q_kernel (clusters over key ranges, bulk-copy ring) behind clear_rows_kernel",
                      "ms_per_call": ms3, "ms_per_call_back_to_back": b2b3, "kernel_ms": kern3,
                      "tflops_rows_used": w3.flop_rows_used / (ms3 * 1e-3) / 1e12,
                      "roofline": {"bound": "hbm", "achieved": bytes3 / (kern3 * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                                   "unit": "GB/s", "frac": bytes3 / (kern3 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                   "bytes_per_launch": bytes3, "traffic": load_traffic("small_q_c3"),
                                   "traffic_source": "constant from profiles/dram_traffic.json: one ncu capture of this kernel at full size",
                                   "bytes": "every key once + the CLS rows + the output; event time of the two kernels of the call",
                                   "frac_of_call": bytes3 / (ms3 * 1e-3) / 1e9 / peaks["hbm_gbs"]}}
        del q3, k3
        w4 = WORKLOADS["c4"]
        q4, k4 = (t.to(dev) for t in make_inputs(Workload(w4.name, w4.B, w4.H, w4.Sq, w4.Sk, w4.D, w4.dtype,
                                                          is_causal=True, seed=w4.seed + rank)))
        ms4, b2b4, _, _, kern4 = small_call_leg(fc, _cabi, w4, q4, k4, n_small, flush_buf, barrier, max_over_ranks, peaks)
        form4 = _cabi.short_fused_applies(w4.B, w4.H, w4.Sq, w4.Sk, True, -1, w4.D)
        # the same call through the statistics, merge and column kernels, for comparison
        _cabi.set_short_fused(_cabi.SHORT_FUSED_NEVER)
        try:
            ms4_three, _, st4, mg4, col4 = small_call_leg(fc, _cabi, w4, q4, k4, n_small, flush_buf, barrier,
                                                          max_over_ranks, peaks)
        finally:
            _cabi.set_short_fused(_cabi.SHORT_FUSED_AUTO)
        causal_short = {"workload": "c4: causal H=32 Q=128 K=4096 D=128 fp16 per GPU",
                        "kernel": ("colsum_fused_short_kernel (a cluster of %d CTAs per head, %d key blocks each: statistics, "
                                   "exchange through distributed shared memory, columns) behind clear_rows_kernel" % form4
                                   if form4 else "statistics, merge and column kernels"),
                        "ms_per_call": ms4, "ms_per_call_back_to_back": b2b4, "kernel_ms": kern4,
                        "three_kernels": {"ms_per_call": ms4_three,
                                          "pass_ms": {"statistics": st4, "merge": mg4, "columns": col4}},
                        "value": w4.flop / (ms4 * 1e-3) / 1e12, "unit": UNIT,
                        "roofline": {"bound": "tensor", "achieved": w4.flop / (ms4 * 1e-3) / 1e12, "peak": peaks["tflops"],
                                     "unit": UNIT, "frac": w4.flop / (ms4 * 1e-3) / 1e12 / peaks["tflops"],
                                     "note": ("bound by latency, not by a unit: 8.6 GFLOP would take 5 us at the tensor peak, "
                                              "the 33.5 MB of keys 5 us at the HBM rate, the 67 M exps 9 us on 128 SMs; the "
                                              "rest is the launch, the ramp of a CTA and the exchange between the phases")}}
        del q4, k4
    assert fc.device_status() == 0

    # ------------------------------------------------------------ CPU baseline (rank 0, one GPU only)
    cpu = None
    if rank == 0 and world == 1:
        cpu, _, _ = cpu_port_tflops(w, args.cpu_budget_s, 1)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": WORKLOAD_LABEL,
                       "global_batch": w.B * world,
                       "parallelism": "single GPU" if world == 1 else f"batch sharded over {world} GPUs, no collective",
                       "flop_count": "4*B*H*Sq*Sk*D (two passes)",
                       "l2": "256 MiB buffer written before every timed step (inputs are 64 MiB)",
                       "plan": plan},
            "frac_of_tensor_peak": value / world / peaks["tflops"],
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": launches_per_call * args.steps,
            "clocks": clocks,
            "causal_long_context": long_ctx,
            "short_key_axis": short_keys,
            "causal_suffix": suffix,
            "cls_prefix": cls_prefix,
            "causal_short": causal_short,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
