"""The CPU checkers against outputs of the reference's own naive_colsum, and
against closed forms that need no reference at all."""

import numpy as np
import pytest
import torch

from flash_colsum_b200.inputs import WORKLOADS, Workload, make_inputs, digest
from oracle import c_oracle
from oracle.naive_colsum import (naive_colsum_f64, naive_colsum_torch, parity_errors)


def test_golden_inputs_regenerate_bit_exactly(golden):
    cases, _ = golden
    for w, sha in cases:
        q, k = make_inputs(w)
        assert digest(q, k) == sha, f"seeded inputs of {w.name} changed"


def test_torch_port_matches_reference_outputs(golden):
    cases, arrays = golden
    for w, _ in cases:
        q, k = make_inputs(w)
        got = naive_colsum_torch(q.float(), k.float(), is_causal=w.is_causal, cls_len=w.cls_len)
        rel, mx = parity_errors(got.numpy(), arrays[w.name])
        assert rel < 1e-6 and mx < 1e-6, (w.name, rel, mx)
        # run in the input dtype, the way the reference's tests call it
        got_native = naive_colsum_torch(q, k, is_causal=w.is_causal, cls_len=w.cls_len)
        rel, mx = parity_errors(got_native.float().numpy(), arrays[w.name + "__native"])
        assert rel < 1e-6 and mx < 1e-6, (w.name, "native", rel, mx)


def test_c_and_f64_checkers_match_reference_outputs(golden):
    cases, arrays = golden
    for w, _ in cases:
        q, k = make_inputs(w)
        want = arrays[w.name]
        for name, fn in (("c", c_oracle.colsum_c), ("f64", naive_colsum_f64)):
            got = fn(q, k, is_causal=w.is_causal, cls_len=w.cls_len)
            rel, mx = parity_errors(got, want)
            # the stored outputs are fp32 softmax results; the checkers are double
            assert rel < 5e-6 and mx < 5e-6, (w.name, name, rel, mx)


def test_head_chunked_port_equals_unchunked():
    w = Workload("t", 1, 8, 48, 300, 64, "bf16", is_causal=True, key_outliers=True, seed=3)
    q, k = make_inputs(w)
    a = naive_colsum_torch(q.float(), k.float(), is_causal=True)
    b = naive_colsum_torch(q.float(), k.float(), is_causal=True, head_chunk=3)
    rel, mx = parity_errors(b.numpy(), a.numpy())
    assert rel < 1e-6 and mx < 1e-6


@pytest.mark.parametrize("causal", [False, True])
def test_rows_sum_to_one(causal):
    q = torch.randn(2 if not causal else 1, 3, 37, 64)
    k = torch.randn(2 if not causal else 1, 3, 91 if causal else 37, 64)
    out = c_oracle.colsum_c(q, k, is_causal=causal)
    np.testing.assert_allclose(out.sum(axis=1), 1.0, rtol=0, atol=1e-12)
    assert (out >= 0).all()


def test_zero_query_closed_forms():
    """Q = 0 makes every visible key equally likely."""
    H, Sq, Sk, D = 2, 5, 12, 64
    q = torch.zeros(1, H, Sq, D)
    k = torch.randn(1, H, Sk, D)
    out = c_oracle.colsum_c(q.expand(1, H, Sq, D), k, is_causal=True)[0]
    k_past = Sk - Sq
    want = np.zeros(Sk)
    for kk in range(Sk):
        for r in range(Sq):
            if kk <= k_past + r:
                want[kk] += 1.0 / (k_past + r + 1)
    want /= Sq
    np.testing.assert_allclose(out, want, atol=1e-13)
    kq = torch.randn(1, H, Sq, D)
    flat = c_oracle.colsum_c(torch.zeros(1, H, Sq, D), kq, is_causal=False)[0]
    np.testing.assert_allclose(flat, 1.0 / Sq, atol=1e-13)


def test_dominant_key_takes_the_column():
    H, S, D = 2, 16, 64
    q = torch.ones(1, H, S, D)
    k = torch.zeros(1, H, S, D)
    k[:, :, 5, :] = 10.0           # score 80*... far above the rest
    out = c_oracle.colsum_c(q, k)[0]
    assert out[5] > 1 - 1e-9 and out.sum() == pytest.approx(1.0)


def test_cls_len_clamps_to_sequence_length():
    q = torch.randn(1, 2, 10, 64)
    k = torch.randn(1, 2, 10, 64)
    a = c_oracle.colsum_c(q, k, cls_len=64)
    b = c_oracle.colsum_c(q, k)
    np.testing.assert_allclose(a, b, atol=1e-15)


def test_headline_workload_table():
    w = WORKLOADS["c2"]
    assert (w.B, w.H, w.Sq, w.D, w.dtype) == (8, 16, 2048, 64, "fp16")
    assert w.flop == pytest.approx(1.374e11, rel=1e-3)
    assert WORKLOADS["c5"].flop == pytest.approx(1.0995e12, rel=1e-3)
    assert WORKLOADS["c3"].rows_averaged == 1


def test_f64_evaluation_takes_an_explicit_k_past():
    """The causal launcher's K_past: the inferred value reproduces the default, a smaller one
    hides keys (their column means are zero), rows still sum to one."""
    from oracle.naive_colsum import naive_colsum_f64
    g = torch.Generator().manual_seed(0)
    q = torch.randn(2, 2, 6, 8, generator=g)
    k = torch.randn(2, 2, 10, 8, generator=g)
    default = naive_colsum_f64(q, k, is_causal=True)
    np.testing.assert_array_equal(default, naive_colsum_f64(q, k, is_causal=True, k_past=4))
    fewer = naive_colsum_f64(q, k, is_causal=True, k_past=1)
    assert (fewer[:, 7:] == 0).all() and (fewer[:, :7] > 0).all()
    np.testing.assert_allclose(fewer.sum(axis=1), 1.0, rtol=1e-12)
    everything = naive_colsum_f64(q, k, is_causal=True, k_past=100)
    np.testing.assert_allclose(everything, naive_colsum_f64(q, k, is_causal=False), rtol=1e-12)


def test_topk_positions_checker():
    from oracle.naive_colsum import topk_positions
    v = np.array([[0.1, 0.5, 0.5, 0.0, 0.5, 0.2]])
    np.testing.assert_array_equal(topk_positions(v, 1), [[1]])
    np.testing.assert_array_equal(topk_positions(v, 2), [[1, 2]])
    np.testing.assert_array_equal(topk_positions(v, 4), [[1, 2, 4, 5]])
    np.testing.assert_array_equal(topk_positions(v, 6), [[0, 1, 2, 3, 4, 5]])
