"""Head-sharded causal call on two GPUs: NCCL all-reduce and the in-kernel
peer-memory reduce both reproduce the unsharded result; so does a single-head non-causal
call split by work (query rows, then keys).  Needs two devices; on a
single-GPU box the test is skipped."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import flash_colsum_b200
        from flash_colsum_b200.inputs import Workload, make_inputs
        from flash_colsum_b200.sharded import PeerAccumulator, flash_colsum_head_sharded, shard_range
        H = 6
        w = Workload("t", 1, H, 200, 3000, 128, "bf16", is_causal=True, key_outliers=True, seed=17)
        lo, hi = shard_range(H, world, rank)
        q, k = (t.to(dev) for t in make_inputs(w, heads=(lo, hi)))
        out_nccl = flash_colsum_head_sharded(q, k, H, is_causal=True)
        peer = PeerAccumulator(w.Sk, dev, dst=0)
        outs = [flash_colsum_head_sharded(q, k, H, is_causal=True, peer=peer).clone() for _ in range(3)]
        torch.cuda.synchronize()
        assert flash_colsum_b200.device_status() == 0
        # the same accumulator with calls whose kernels cannot carry the flags themselves: two decode
        # queries (the few-row kernel), and one head over two ranks (a rank with nothing to launch);
        # in between, ordinary calls again
        wf = Workload("f", 1, H, 2, 3000, 128, "bf16", is_causal=True, seed=18)
        qf, kf = (t.to(dev) for t in make_inputs(wf, heads=(lo, hi)))
        w1 = Workload("o", 1, 1, 200, 3000, 128, "bf16", is_causal=True, seed=19)
        l1, h1 = shard_range(1, world, rank)
        q1, k1 = (t.to(dev) for t in make_inputs(w1, heads=(l1, h1)))
        mixed = []
        for _ in range(2):
            mixed.append(flash_colsum_head_sharded(qf, kf, H, is_causal=True, peer=peer).clone())
            mixed.append(flash_colsum_head_sharded(q, k, H, is_causal=True, peer=peer).clone())
            mixed.append(flash_colsum_head_sharded(q1, k1, 1, is_causal=True, peer=peer).clone())
        torch.cuda.synchronize()
        assert flash_colsum_b200.device_status() == 0
        # one single-head sample split by work: query rows for the statistics, keys for the columns
        from flash_colsum_b200.sharded import flash_colsum_work_sharded
        w2 = Workload("w", 1, 1, 3000, 3000, 64, "fp16", seed=23)
        q2, k2 = (t.to(dev) for t in make_inputs(w2))
        out_work = flash_colsum_work_sharded(q2, k2)
        torch.cuda.synchronize()
        assert flash_colsum_b200.device_status() == 0
        results[rank] = (out_nccl.cpu().numpy(), [o.cpu().numpy() for o in outs], out_work.cpu().numpy(),
                         [o.cpu().numpy() for o in mixed])
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_match_unsharded():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from flash_colsum_b200.inputs import Workload, make_inputs
    from oracle import c_oracle
    from oracle.naive_colsum import parity_errors
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    w = Workload("t", 1, 6, 200, 3000, 128, "bf16", is_causal=True, key_outliers=True, seed=17)
    q, k = make_inputs(w)
    want = c_oracle.colsum_c(q, k, is_causal=True)
    for r in (0, 1):
        rel, mx = parity_errors(results[r][0], want)
        assert rel <= 1e-3 and mx <= 1e-3, ("nccl", r, rel, mx)
    for o in results[0][1]:          # the peer-memory reduce lands on rank 0
        rel, mx = parity_errors(o, want)
        assert rel <= 1e-3 and mx <= 1e-3, ("peer", rel, mx)
    wants = [c_oracle.colsum_c(*make_inputs(Workload("f", 1, 6, 2, 3000, 128, "bf16", is_causal=True, seed=18)),
                               is_causal=True),
             want,
             c_oracle.colsum_c(*make_inputs(Workload("o", 1, 1, 200, 3000, 128, "bf16", is_causal=True, seed=19)),
                               is_causal=True)]
    for i, o in enumerate(results[0][3]):   # few rows / ordinary / a rank without heads, twice over
        rel, mx = parity_errors(o, wants[i % 3])
        assert rel <= 1e-3 and mx <= 1e-3, ("mixed", i, rel, mx)
    q2, k2 = make_inputs(Workload("w", 1, 1, 3000, 3000, 64, "fp16", seed=23))
    want2 = c_oracle.colsum_c(q2, k2)
    for r in (0, 1):                 # the work split leaves the whole result on every rank
        rel, mx = parity_errors(results[r][2], want2)
        assert rel <= 1e-3 and mx <= 1e-3, ("work split", r, rel, mx)
