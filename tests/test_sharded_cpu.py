"""Head-sharded path on two CPU ranks (gloo).  The local kernel call is replaced
by the CPU checker evaluated on the rank's heads, so what is tested is the
sharding arithmetic, the global-head normalisation and the collective."""

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_local(q, k, scale, is_causal, cls_len, h_total):
    from oracle import c_oracle
    part = c_oracle.colsum_c(q, k, scale=scale, is_causal=is_causal, cls_len=cls_len)
    return torch.from_numpy(part * (q.shape[1] / h_total)).float()


def _worker(rank, world, port, H, dst, causal, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_colsum_b200.inputs import Workload, make_inputs
        from flash_colsum_b200.sharded import flash_colsum_head_sharded, shard_range
        w = Workload("t", 1 if causal else 2, H, 48, 200 if causal else 48, 64, "fp16",
                     is_causal=causal, seed=9)
        lo, hi = shard_range(H, world, rank)
        q, k = make_inputs(w, heads=(lo, hi))
        out = flash_colsum_head_sharded(q, k, H, is_causal=causal, dst=dst, local_fn=_oracle_local)
        results[rank] = out.numpy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("H,dst,causal", [(4, None, True), (3, 0, False), (1, None, True)])
def test_two_ranks_match_unsharded(H, dst, causal):
    from flash_colsum_b200.inputs import Workload, make_inputs
    from oracle import c_oracle
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), H, dst, causal, results), nprocs=world, join=True)
    w = Workload("t", 1 if causal else 2, H, 48, 200 if causal else 48, 64, "fp16",
                 is_causal=causal, seed=9)
    q, k = make_inputs(w)
    want = c_oracle.colsum_c(q, k, is_causal=causal)
    ranks = [0, 1] if dst is None else [dst]
    for r in ranks:
        np.testing.assert_allclose(results[r], want, rtol=1e-5, atol=1e-9)


def test_shard_range_covers_every_unit_once():
    from flash_colsum_b200.sharded import shard_range
    for n in (0, 1, 5, 32, 33):
        for world in (1, 2, 4, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
