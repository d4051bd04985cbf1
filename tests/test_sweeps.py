"""The sweep driver (benchmarks/sweeps.py): its shapes are the reference's, its chunked
materialising baseline equals the unchunked one, and one point runs end to end on a GPU."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "benchmarks"))

import sweeps  # noqa: E402
from oracle.naive_colsum import naive_colsum_torch  # noqa: E402


def test_sweep_points_are_the_reference_benchmarks_axes():
    # benchmarks/benchmark_colsum.py:289-424 of the reference: fp16, these three axes
    assert [p["B"] for p in sweeps.SWEEPS["batched"]] == [8, 16, 32, 64, 128, 256, 512, 1024]
    assert all((p["H"], p["Sq"], p["Sk"], p["D"], p["causal"]) == (16, 1024, 1024, 64, False)
               for p in sweeps.SWEEPS["batched"])
    assert [p["Sq"] for p in sweeps.SWEEPS["single"]] == [4096 << i for i in range(7)]
    assert all(p["B"] == 1 and p["H"] == 16 and p["D"] == 64 and p["Sq"] == p["Sk"] for p in sweeps.SWEEPS["single"])
    assert [p["Sk"] for p in sweeps.SWEEPS["causal"]] == [16384 << i for i in range(5)]
    assert all((p["H"], p["Sq"], p["D"], p["causal"]) == (32, 128, 128, True) for p in sweeps.SWEEPS["causal"])
    assert len(sweeps.SWEEPS["configs"]) == 4
    assert [p["Sk"] for p in sweeps.SWEEPS["causal_short"]] == [1024, 2048, 4096, 8192]


@pytest.mark.parametrize("B,H,S,budget,chunked", [
    (6, 2, 64, 1 << 40, False),          # fits: one call
    (6, 2, 64, 2 * 2 * 64 * 64 * 4, True),   # two batch entries at a time
    (1, 2, 200, 2 * 64 * 200 * 4, True),     # one sample: 64 query rows at a time
])
def test_chunked_baseline_equals_the_whole(monkeypatch, B, H, S, budget, chunked):
    g = torch.Generator().manual_seed(S)
    q = torch.randn(B, H, S, 32, generator=g)
    k = torch.randn(B, H, S, 32, generator=g)
    monkeypatch.setattr(sweeps, "SCORE_BUDGET_BYTES", budget)
    fn, was_chunked = sweeps.naive_in_pieces(naive_colsum_torch, q, k, False, None)
    assert was_chunked == chunked
    torch.testing.assert_close(fn().float(), naive_colsum_torch(q, k).float(), rtol=1e-5, atol=1e-8)


@pytest.mark.gpu
def test_one_sweep_point_runs_with_and_without_the_reference_legs():
    pt = dict(B=2, H=4, Sq=512, Sk=512, D=64, causal=False)
    row = sweeps.run_point(pt, warmup=2, iters=5)
    assert row["device_ms"] > 0 and row["host_sync_ms"] >= row["device_ms"] * 0.5
    assert abs(row["row_sum"] - 1.0) < 1e-3 and row["peak_mem_gib"] > 0
    if os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "flash_colsum")):
        row = sweeps.run_point(pt, warmup=2, iters=5, reference=sweeps.load_reference())
        assert row["ref_naive_ms"] > 0 and row["ours_rel_l2_vs_naive"] < 1e-3
        assert row["ref_triton_ms"] is None or row["ref_triton_rel_l2"] < 1e-2
    causal = sweeps.run_point(dict(B=1, H=4, Sq=128, Sk=2048, D=128, causal=True), warmup=2, iters=5)
    assert abs(causal["row_sum"] - 1.0) < 1e-3
