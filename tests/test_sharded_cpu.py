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


# ---------------------------------------------------------------------------
# Work split (query rows for the statistics, keys for the column means) on two and three
# CPU ranks: the two kernels are replaced by float64 numpy, so what is tested is the share
# arithmetic, the padding of the gathered vectors and the two all-gathers.
# ---------------------------------------------------------------------------
def _stats_numpy(query_rows, key, scale, norm_rows, h_norm=0):
    q = query_rows.double().numpy()
    k = key.double().numpy()
    B, H, rows, _ = q.shape
    pad = -(-rows // 256) * 256
    out = np.full((B * H, pad), -np.inf)
    c = scale * np.log2(np.e)
    for b in range(B):
        for h in range(H):
            s = (q[b, h] @ k[b, h].T) * c
            m = s.max(axis=1)
            lse = m + np.log2(np.exp2(s - m[:, None]).sum(axis=1))
            out[b * H + h, :rows] = -(lse + np.log2(H * norm_rows))
    return torch.from_numpy(out).float()


def _columns_numpy(query, key_rows, neg_lse, scale):
    q = query.double().numpy()
    k = key_rows.double().numpy()
    B, H, rows, _ = q.shape
    nl = neg_lse.double().numpy()
    c = scale * np.log2(np.e)
    out = np.zeros((B, k.shape[2]))
    for b in range(B):
        for h in range(H):
            s = (q[b, h] @ k[b, h].T) * c
            out[b] += np.exp2(s + nl[b * H + h, :rows, None]).sum(axis=0)
    return torch.from_numpy(out).float()


def _work_worker(rank, world, port, S, cls, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_colsum_b200.inputs import Workload, make_inputs
        from flash_colsum_b200.sharded import flash_colsum_work_sharded
        q, k = make_inputs(Workload("w", 2, 2, S, S, 64, "fp16", cls_len=cls, seed=S))
        out = flash_colsum_work_sharded(q, k, cls_len=cls, stats_fn=_stats_numpy, columns_fn=_columns_numpy)
        results[rank] = out.numpy()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,S,cls", [(2, 300, None), (3, 700, None), (2, 520, 260), (3, 100, None)])
def test_work_split_matches_unsharded(world, S, cls):
    from flash_colsum_b200.inputs import Workload, make_inputs
    from oracle import c_oracle
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_work_worker, args=(world, _free_port(), S, cls, results), nprocs=world, join=True)
    q, k = make_inputs(Workload("w", 2, 2, S, S, 64, "fp16", cls_len=cls, seed=S))
    want = c_oracle.colsum_c(q, k, cls_len=cls)
    for r in range(world):
        assert results[r].shape == (2, S)
        np.testing.assert_allclose(results[r], want, rtol=2e-5, atol=1e-9)


def test_work_shares_cover_the_rows_in_granules():
    from flash_colsum_b200.sharded import work_shares
    for n, world, g in [(1000, 4, 256), (577, 2, 128), (100, 8, 256), (131072, 8, 256), (1, 3, 128)]:
        share, ranges = work_shares(n, world, g)
        assert share % g == 0 and len(ranges) == world
        assert ranges[0][0] == 0 and ranges[-1][1] == n
        for r, (lo, hi) in enumerate(ranges):
            assert lo == min(n, r * share) and lo <= hi <= lo + share
            if r:
                assert lo == ranges[r - 1][1]
