#!/usr/bin/env python
"""One long non-causal sample on N GPUs, split by work and split by heads.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        benchmarks/work_split.py [--heads 16] [--seq 65536] [--steps 10]

Every rank holds the same (1, H, S, 64) fp16 tensors.  Timed on the device (CUDA events,
max over ranks): `flash_colsum_work_sharded` (query rows for the statistics, keys for the
column means, two all-gathers) and, when H >= N, `flash_colsum_head_sharded` (heads over
ranks, one all-reduce); rank 0 prints one JSON line with both and the single-GPU time.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import flash_colsum_b200 as fc  # noqa: E402
from flash_colsum_b200.sharded import flash_colsum_head_sharded, flash_colsum_work_sharded, shard_range  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=65536)
    ap.add_argument("--steps", type=int, default=10)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    g = torch.Generator(device=dev).manual_seed(3)          # the same tensors on every rank
    q = torch.randn(1, args.heads, args.seq, 64, device=dev, dtype=torch.float16, generator=g)
    k = torch.randn(1, args.heads, args.seq, 64, device=dev, dtype=torch.float16, generator=g)

    def timed(fn):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out = fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), out

    single_ms, want = timed(lambda: fc.flash_colsum(q, k))
    work_ms, got = timed(lambda: flash_colsum_work_sharded(q, k))
    line = {"n_gpus": world, "heads": args.heads, "seq": args.seq, "single_gpu_ms": single_ms,
            "work_split_ms": work_ms,
            "work_split_rel_err": float(((got - want).norm() / want.norm()).item())}
    if args.heads >= world:
        lo, hi = shard_range(args.heads, world, rank)
        head_ms, got_h = timed(lambda: flash_colsum_head_sharded(q[:, lo:hi], k[:, lo:hi], args.heads))
        line["head_split_ms"] = head_ms
        line["head_split_rel_err"] = float(((got_h - want).norm() / want.norm()).item())
    assert fc.device_status() == 0
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
