"""Parity of the CUDA path with the CPU checker, through the public operator
(which calls the C ABI).  Bar: rel-L2 <= 1e-3 and max-abs <= 1e-3 of the largest
column mean, on fp32 outputs, against the checker fed the same inputs."""

import numpy as np
import pytest
import torch

from conftest import MAX_ABS_TOL, REL_L2_TOL
from flash_colsum_b200.inputs import WORKLOADS, Workload, make_inputs
from oracle import c_oracle
from oracle.naive_colsum import naive_colsum_torch, parity_errors

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fc():
    if not torch.cuda.is_available():
        pytest.fail("the gpu-marked tests need a CUDA device")
    import flash_colsum_b200
    return flash_colsum_b200


def run_gpu(fc, w: Workload, q, k, **kw):
    out = fc.flash_colsum(q.cuda(), k.cuda(), is_causal=w.is_causal, cls_len=w.cls_len, **kw)
    torch.cuda.synchronize()
    assert fc.device_status() == 0, "a device-side wait expired"
    assert out.dtype == torch.float32
    return out.cpu().numpy()


def assert_parity(got, want, what):
    rel, mx = parity_errors(got, want)
    assert np.isfinite(got).all(), what
    assert rel <= REL_L2_TOL and mx <= MAX_ABS_TOL, (what, rel, mx)


def test_golden_cases_match_reference_outputs(fc, golden):
    """Every stored output of the reference's naive_colsum (fp32 run), 16-bit cases."""
    cases, arrays = golden
    ran = 0
    for w, _ in cases:
        q, k = make_inputs(w)
        # fp32 inputs are rounded to fp16 on the way in; the stored output is of the unrounded ones
        got = run_gpu(fc, w, q, k)
        assert got.shape == arrays[w.name].shape
        assert_parity(got, arrays[w.name], w.name)
        ran += 1
    assert ran >= 23


def test_c1_shape_in_fp16_matches_checker(fc):
    """The CPU reference config (B2 H4 S256 D64) with inputs rounded to fp16."""
    w = Workload("c1_fp16", 2, 4, 256, 256, 64, "fp16", seed=0)
    q, k = make_inputs(w)
    assert_parity(run_gpu(fc, w, q, k), c_oracle.colsum_c(q, k), "c1")


SHAPES = [
    # B, H, Sq, Sk, D, dtype, causal, cls
    (4, 8, 512, 512, 64, "fp16", False, None),       # reference test_core.py:21-35
    (4, 8, 512, 512, 64, "fp16", False, 1),          # reference test_core.py:57-72
    (1, 4, 1024, 1024, 64, "fp16", False, 2),        # single-sample + cls (test_core.py:76-91, shortened)
    (1, 4, 2048, 2048, 64, "fp16", False, None),     # single-sample (test_core.py:39-53, shortened)
    (1, 8, 128, 4096, 128, "fp16", True, None),      # causal (test_core.py:95-109, shortened)
    (2, 3, 1, 1, 64, "fp16", False, None),           # one key: every mean is 1
    (1, 2, 7, 7, 128, "bf16", False, None),
    (1, 2, 129, 129, 64, "bf16", False, None),
    (3, 5, 383, 383, 128, "fp16", False, None),
    (1, 2, 1, 300, 64, "fp16", True, None),          # one decode query
    (1, 2, 257, 257, 128, "bf16", True, None),
    (1, 3, 200, 1000, 64, "fp16", True, None),
    (1, 2, 513, 3000, 128, "bf16", True, None),
    (1, 2, 300, 100, 64, "fp16", True, None),        # keys shorter than queries
    (2, 2, 640, 640, 64, "fp16", False, 130),        # cls prefix spanning two query tiles
    # one query block, sixteen or more key tiles: the column pass streams key tiles head by head
    (1, 5, 100, 2500, 64, "bf16", True, None),
    (1, 3, 256, 3000, 128, "fp16", True, None),
    (2, 4, 2100, 2100, 64, "fp16", False, 200),
    (1, 40, 70, 2200, 128, "bf16", True, None),      # a head change every few tiles
    (1, 6, 48, 2300, 128, "fp16", True, None),       # at most 64 queries: half of each tile's columns are padding
    (1, 3, 64, 2177, 64, "bf16", True, None),
    (2, 4, 2100, 2100, 64, "fp16", False, 40),
    # two query blocks, both resident in shared memory next to the ring of key tiles
    (1, 3, 400, 2500, 128, "bf16", True, None),
    (1, 5, 512, 2304, 64, "fp16", True, None),
    (2, 3, 2100, 2100, 64, "fp16", False, 300),
    (1, 20, 300, 2200, 128, "fp16", True, None),
]


@pytest.mark.parametrize("B,H,Sq,Sk,D,dtype,causal,cls", SHAPES)
def test_shapes_match_checker(fc, B, H, Sq, Sk, D, dtype, causal, cls):
    w = Workload("t", B, H, Sq, Sk, D, dtype, is_causal=causal, cls_len=cls, seed=Sq + Sk + D)
    q, k = make_inputs(w)
    got = run_gpu(fc, w, q, k)
    want = c_oracle.colsum_c(q, k, is_causal=causal, cls_len=cls)
    assert_parity(got, want, (B, H, Sq, Sk, D, dtype, causal, cls))
    np.testing.assert_allclose(got.sum(axis=1), 1.0, atol=2e-3)


def test_head_dimensions_that_are_not_64_or_128(fc):
    """Any multiple of 8 up to 128: the tensor maps zero-fill the columns up to 64 or 128, which
    add nothing to a score; the scale defaults to 1/sqrt of the real D.  Streaming passes (causal,
    long), the single-pass kernel (D < 64, short non-causal) and a CLS prefix (few rows: streaming
    passes too, the few-row kernel deals rows over D/8 lanes and takes D = 64 and 128 only)."""
    for (B, H, Sq, Sk, D, dtype, causal, cls) in [
            (2, 4, 512, 512, 32, "fp16", False, None),      # single-pass kernel, half the columns zero
            (1, 3, 300, 2200, 80, "bf16", True, None),
            (2, 2, 700, 700, 72, "fp16", False, None),
            (2, 2, 700, 700, 120, "bf16", False, 2),
            (1, 2, 128, 5000, 8, "fp16", True, None),
            (1, 4, 4, 3000, 96, "fp16", True, None),
            (1, 2, 2500, 2500, 40, "fp16", False, None)]:
        w = Workload("d", B, H, Sq, Sk, D, dtype, is_causal=causal, cls_len=cls, seed=D + Sq)
        q, k = make_inputs(w)
        got = run_gpu(fc, w, q, k)
        assert_parity(got, c_oracle.colsum_c(q, k, is_causal=causal, cls_len=cls), (B, H, Sq, Sk, D, dtype, causal, cls))
    # sliced out of a wider tensor: the row stride is not the head dimension
    wide = torch.randn(1, 2, 600, 128, device="cuda").half()
    qv, kv = wide[..., :48], wide[..., 64:112]
    got = fc.flash_colsum(qv, kv).cpu().numpy()
    assert_parity(got, c_oracle.colsum_c(qv.cpu(), kv.cpu()), "strided D=48")


def test_fp32_inputs_are_rounded_to_16_bits(fc):
    """fp32 in: rounded to fp16 (bf16 beyond fp16's range).  Exact against the checker fed the
    rounded values, and inside the bar against the checker fed the fp32 values themselves."""
    w = Workload("f", 2, 4, 600, 600, 64, "fp32", seed=41)
    q, k = make_inputs(w)
    got = fc.flash_colsum(q.cuda(), k.cuda()).cpu().numpy()
    assert_parity(got, c_oracle.colsum_c(q.half(), k.half()), "fp32 -> fp16, rounded inputs")
    assert_parity(got, c_oracle.colsum_c(q, k), "fp32 -> fp16, fp32 inputs")
    big = q * 1000.0            # |q| up to ~4000, q.k beyond fp16: still fine as fp16 operands
    got = fc.flash_colsum(big.cuda(), k.cuda(), scale=1e-4).cpu().numpy()
    assert_parity(got, c_oracle.colsum_c(big.half(), k.half(), scale=1e-4), "fp32 large")
    huge = q * 1e6              # out of fp16's range: bf16
    got = fc.flash_colsum(huge.cuda(), k.cuda(), scale=1e-7).cpu().numpy()
    assert_parity(got, c_oracle.colsum_c(huge.bfloat16(), k.bfloat16(), scale=1e-7), "fp32 -> bf16")


FEW_ROWS = [
    # B, H, R (cls_len, or query rows when causal), Sk, D, dtype, causal
    (1, 32, 1, 32768, 128, "fp16", True),     # one decode query over 32 heads: eight key ranges per head
    (1, 8, 4, 50000, 128, "bf16", True),      # ranges longer than the ring: stages are refilled
    (1, 4, 1, 200000, 64, "fp16", True),      # the longest range whose scores still fit
    (2, 3, 3, 1000, 64, "bf16", False),       # three rows (kernel built for four)
    (32, 16, 1, 577, 64, "fp16", False),      # the CLIP-style CLS call
    (1, 2, 2, 31, 128, "fp16", False),        # fewer keys than one range wants
    (3, 2, 4, 64, 64, "fp16", True),          # R = 4 queries at the end of 64 keys
    (1, 1, 4, 3, 64, "bf16", True),           # fewer keys than queries
    (25, 8, 1, 577, 64, "fp16", False),       # 200 units on 148 persistent CTAs: a unit is finished behind the next one's scores
    (10, 20, 3, 1500, 128, "bf16", False),    # the same with three rows and clusters of two
    (40, 16, 2, 300, 64, "fp16", False),      # 640 short units: four CTAs per SM, more than one unit each
    (37, 8, 4, 257, 128, "bf16", False),      # 296 short units of four rows
]


@pytest.mark.parametrize("B,H,R,Sk,D,dtype,causal", FEW_ROWS)
def test_few_query_rows_match_checker(fc, B, H, R, Sk, D, dtype, causal):
    """At most four query rows: the clustered matrix-vector kernel (key ranges over the CTAs of a
    cluster, rows staged by bulk copies, one exchange of (maximum, sum) per call)."""
    Sq = R if causal else Sk
    w = Workload("few", B, H, Sq, Sk, D, dtype, is_causal=causal, cls_len=None if causal else R, seed=R + Sk + D)
    q, k = make_inputs(w)
    if causal and B > 1:      # the operator keeps the reference's refusal of causal batches
        got = fc.flash_colsum_causal(q.cuda(), k.cuda()).cpu().numpy()
        assert fc.device_status() == 0
    else:
        got = run_gpu(fc, w, q, k)
    want = c_oracle.colsum_c(q, k, is_causal=causal, cls_len=w.cls_len)
    assert_parity(got, want, (B, H, R, Sk, D, dtype, causal))
    np.testing.assert_allclose(got.sum(axis=1), 1.0, atol=2e-3)


def test_few_query_rows_strided_keys_and_explicit_k_past(fc):
    """Key rows that are not contiguous are copied row by row; an explicit K_past below the key
    length leaves the trailing columns at zero without reading their keys."""
    from oracle.naive_colsum import naive_colsum_f64
    w = Workload("few_strided", 2, 3, 700, 700, 64, "fp16", cls_len=2, seed=77)
    q, k = make_inputs(w)
    kc = torch.empty(2, 3, 700, 80, dtype=torch.float16, device="cuda")[..., :64]   # row stride 80 elements
    kc.copy_(k)
    got = fc.flash_colsum(q.cuda(), kc, cls_len=2)
    torch.cuda.synchronize()
    assert_parity(got.cpu().numpy(), c_oracle.colsum_c(q, k, cls_len=2), "strided keys")
    w = Workload("few_k_past", 1, 4, 3, 5000, 128, "bf16", is_causal=True, seed=78)
    q, k = make_inputs(w)
    for k_past in (0, 100, 4997, 9000):
        got = fc.flash_colsum_causal(q.cuda(), k.cuda(), k_past=k_past).cpu().numpy()
        assert fc.device_status() == 0
        assert_parity(got, naive_colsum_f64(q, k, is_causal=True, k_past=k_past), f"few rows k_past {k_past}")
        if k_past + 3 < 5000:
            assert (got[:, k_past + 3:] == 0).all()


def test_key_equal_to_query_and_outlier_keys(fc):
    w = Workload("kq", 2, 4, 512, 512, 64, "fp16", key_is_query=True, seed=21)
    q, k = make_inputs(w)
    assert_parity(run_gpu(fc, w, q, k), c_oracle.colsum_c(q, k), "key=query")
    w = Workload("outl", 1, 4, 256, 4096, 128, "bf16", is_causal=True, key_outliers=True, seed=22)
    q, k = make_inputs(w)
    assert_parity(run_gpu(fc, w, q, k), c_oracle.colsum_c(q, k, is_causal=True), "outlier keys")


def test_scale_argument_and_large_scores(fc):
    w = Workload("s", 2, 2, 256, 256, 64, "fp16", seed=31)
    q, k = make_inputs(w)
    for scale in (0.5, 0.01, -0.2, 0.0):
        got = fc.flash_colsum(q.cuda(), k.cuda(), scale=scale).cpu().numpy()
        assert_parity(got, c_oracle.colsum_c(q, k, scale=scale), f"scale={scale}")
    assert fc.device_status() == 0


def test_zero_queries_give_closed_form(fc):
    H, Sq, Sk, D = 2, 70, 300, 64
    q = torch.zeros(1, H, Sq, D, dtype=torch.float16)
    k = torch.randn(1, H, Sk, D).half()
    got = fc.flash_colsum(q.cuda(), k.cuda(), is_causal=True).cpu().numpy()[0]
    k_past = Sk - Sq
    want = np.zeros(Sk)
    for r in range(Sq):
        want[: k_past + r + 1] += 1.0 / (k_past + r + 1)
    want /= Sq
    np.testing.assert_allclose(got, want, rtol=2e-5, atol=1e-9)
    flat = fc.flash_colsum(q[:, :, :, :].cuda(), torch.randn(1, H, Sq, D).half().cuda()).cpu().numpy()
    np.testing.assert_allclose(flat, 1.0 / Sq, rtol=2e-5)


def test_inputs_with_an_empty_axis(fc):
    """No batch entry, no key, no query row: what the reference's naive_colsum returns for such
    inputs (an empty result, or NaN for a mean over no rows), and nothing is launched."""
    dev = "cuda"
    h = lambda *shape: torch.empty(*shape, device=dev, dtype=torch.float16)   # noqa: E731
    out = fc.flash_colsum(h(0, 2, 4, 64), h(0, 2, 4, 64))
    assert out.shape == (0, 4) and out.dtype == torch.float32
    assert fc.flash_colsum(h(1, 2, 0, 64), h(1, 2, 0, 64)).shape == (1, 0)
    assert fc.flash_colsum(h(3, 2, 0, 64), h(3, 2, 0, 64), cls_len=1).shape == (3, 0)
    out = fc.flash_colsum(h(1, 2, 0, 64), torch.randn(1, 2, 5, 64, device=dev).half(), is_causal=True)
    assert out.shape == (1, 5) and bool(torch.isnan(out).all())
    assert fc.flash_colsum_causal(torch.randn(2, 2, 3, 64, device=dev).half(), h(2, 2, 0, 64)).shape == (2, 0)
    assert fc.flash_colsum_causal(h(0, 2, 3, 64), h(0, 2, 7, 64), out_dtype=torch.float16).dtype == torch.float16
    torch.cuda.synchronize()
    assert fc.device_status() == 0


def test_non_contiguous_views_and_out_dtype(fc):
    g = torch.Generator().manual_seed(41)
    big_q = torch.randn(2, 3, 200, 128, generator=g).half().cuda()
    big_k = torch.randn(2, 3, 200, 128, generator=g).half().cuda()
    q, k = big_q[..., :64], big_k[..., 64:]          # strided rows, offset base
    want = c_oracle.colsum_c(q.cpu(), k.cpu())
    assert_parity(fc.flash_colsum(q, k).cpu().numpy(), want, "strided views")
    qt = big_q.transpose(1, 2)[..., :64].transpose(1, 2)
    assert_parity(fc.flash_colsum(qt, k).cpu().numpy(), want, "transposed view")
    half = fc.flash_colsum(q, k, out_dtype=torch.float16)
    assert half.dtype == torch.float16
    np.testing.assert_allclose(half.float().cpu().numpy(), want, atol=1e-3, rtol=1e-3)
    assert fc.device_status() == 0


def test_repeated_calls_reuse_scratch_safely(fc):
    w = Workload("r", 2, 4, 384, 384, 64, "fp16", seed=51)
    q, k = make_inputs(w)
    qc, kc = q.cuda(), k.cuda()
    want = c_oracle.colsum_c(q, k)
    outs = [fc.flash_colsum(qc, kc) for _ in range(5)]
    for o in outs:
        assert_parity(o.cpu().numpy(), want, "repeat")
    assert fc.device_status() == 0


def test_host_entry_matches_device_entry(fc):
    w = Workload("host", 5, 4, 300, 300, 64, "fp16", seed=91)
    q, k = make_inputs(w)
    want = fc.flash_colsum(q.cuda(), k.cuda()).cpu()
    for qh, kh in ((q, k), (q.pin_memory(), k.pin_memory())):
        for chunk in (None, 1, 2, 8):      # None: chunks that shrink towards the end
            got = fc.flash_colsum_host(qh, kh, batch_chunk=chunk)
            assert got.device.type == "cpu"
            torch.testing.assert_close(got, want, rtol=2e-5, atol=1e-9)   # summation order differs with the chunking
    wc = Workload("host_causal", 1, 4, 64, 900, 128, "bf16", is_causal=True, seed=92)
    q, k = make_inputs(wc)
    torch.testing.assert_close(fc.flash_colsum_host(q, k, is_causal=True),
                               fc.flash_colsum(q.cuda(), k.cuda(), is_causal=True).cpu(), rtol=2e-5, atol=1e-9)
    with pytest.raises(ValueError, match="host tensors"):
        fc.flash_colsum_host(q.cuda(), k.cuda())
    assert fc.device_status() == 0


def test_calls_can_be_captured_in_a_cuda_graph(fc):
    """The library neither synchronises nor allocates, so a call replays from a graph."""
    w = Workload("graph", 1, 8, 128, 4096, 128, "fp16", is_causal=True, seed=81)
    q, k = (t.cuda() for t in make_inputs(w))
    fc.flash_colsum(q, k, is_causal=True)            # first call outside capture (one-time set-up)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fc.flash_colsum(q, k, is_causal=True)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fc.flash_colsum(q, k, is_causal=True)
    want = c_oracle.colsum_c(q.cpu(), k.cpu(), is_causal=True)
    for _ in range(3):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, "graph replay")
    assert fc.device_status() == 0
    # the few-row kernel (a cluster launch that is a programmatic dependent of the clearing kernel)
    for wf in (Workload("graph_cls", 8, 8, 400, 400, 64, "fp16", cls_len=1, seed=82),
               Workload("graph_decode", 1, 8, 2, 9000, 128, "bf16", is_causal=True, seed=83)):
        q, k = (t.cuda() for t in make_inputs(wf))
        call = lambda: fc.flash_colsum(q, k, is_causal=wf.is_causal, cls_len=wf.cls_len)  # noqa: E731
        call()
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            call()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = call()
        want = c_oracle.colsum_c(q.cpu(), k.cpu(), is_causal=wf.is_causal, cls_len=wf.cls_len)
        for _ in range(3):
            out.fill_(float("nan"))
            graph.replay()
            torch.cuda.synchronize()
            assert_parity(out.cpu().numpy(), want, f"graph replay {wf.name}")
    assert fc.device_status() == 0


def test_error_handling(fc):
    """The reference's error cases (tests/test_core.py:112-134), same messages."""
    dev, dt = torch.device("cuda"), torch.float16
    Q = torch.randn(2, 8, 128, 64, device=dev, dtype=dt)
    K = torch.randn(2, 8, 1024, 64, device=dev, dtype=dt)
    with pytest.raises(ValueError, match="batch size 1"):
        fc.flash_colsum(Q, K, is_causal=True)
    with pytest.raises(ValueError, match="CUDA"):
        fc.flash_colsum(torch.randn(1, 8, 128, 64), torch.randn(1, 8, 128, 64))
    K2 = torch.randn(2, 8, 256, 64, device=dev, dtype=dt)
    with pytest.raises(ValueError, match="same shape"):
        fc.flash_colsum(Q, K2)
    with pytest.raises(ValueError, match="cls_len"):
        fc.flash_colsum(Q, Q, cls_len=0)
    with pytest.raises(ValueError, match="non-causal"):
        fc.flash_colsum(Q[:1], K[:1], is_causal=True, cls_len=1)
    with pytest.raises(ValueError, match="4D"):
        fc.flash_colsum(Q[0], Q[0])
    with pytest.raises(ValueError, match="head_dim"):
        fc.flash_colsum(Q[..., :36], Q[..., :36])
    with pytest.raises(ValueError, match="head_dim"):
        fc.flash_colsum(torch.cat([Q, Q, Q], dim=-1), torch.cat([Q, Q, Q], dim=-1))
    with pytest.raises(ValueError, match="float16, bfloat16 and float32"):
        fc.flash_colsum(Q.double(), Q.double())
    with pytest.raises(ValueError, match="same dtype"):
        fc.flash_colsum(Q, Q.float())


# ------------------------------------------------------------------ full sizes
def _torch_fp32_reference(q, k, causal, cls_len, head_chunk):
    """Materialising fp32 evaluation on the GPU, a few heads at a time."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    rows = Sq if cls_len is None else min(cls_len, Sq)
    acc = torch.zeros(B, Sk, dtype=torch.float64, device=q.device)
    vis = None
    if causal:
        vis = (torch.arange(Sk, device=q.device)[None, :]
               <= (max(0, Sk - Sq) + torch.arange(Sq, device=q.device))[:, None])
    for h0 in range(0, H, head_chunk):
        s = torch.matmul(q[:, h0:h0 + head_chunk, :rows].float(),
                         k[:, h0:h0 + head_chunk].float().transpose(-1, -2)) / D ** 0.5
        if vis is not None:
            s = s.masked_fill(~vis[:rows], float("-inf"))
        acc += torch.softmax(s, dim=-1).sum(dim=(1, 2), dtype=torch.float64)
    return (acc / (H * rows)).cpu().numpy()


def test_full_size_reference_agrees_with_the_pinned_checker(fc, golden):
    """The materialising evaluation the full-size tests compare with is itself checked here: on
    stored outputs of the reference's naive_colsum and against the C checker, non-causal, causal
    and with a CLS prefix, so that the full-size comparisons hang off the pinned oracle."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        cases, arrays = golden
        ran = 0
        for w, _ in cases:
            if w.dtype == "fp32" or w.B * w.H * w.Sq * w.Sk > (1 << 24):
                continue
            if w.is_causal and w.Sk < w.Sq:
                continue     # the full-size shapes all have K_len >= Q_len
            q, k = make_inputs(w)
            got = _torch_fp32_reference(q.cuda(), k.cuda(), w.is_causal, w.cls_len, 2)
            rel, mx = parity_errors(got, arrays[w.name])
            assert rel <= 1e-5 and mx <= 1e-5, (w.name, rel, mx)
            rel, mx = parity_errors(got, c_oracle.colsum_c(q, k, is_causal=w.is_causal, cls_len=w.cls_len))
            assert rel <= 1e-5 and mx <= 1e-5, (w.name, rel, mx)
            ran += 1
        assert ran >= 8
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


@pytest.mark.parametrize("name,chunk", [("c2", 4), ("c2_kq", 4), ("c3", 16), ("c4", 32)])
def test_headline_workloads_full_size(fc, name, chunk):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        w = WORKLOADS[name]
        q, k = make_inputs(w)
        qc, kc = q.cuda(), k.cuda()
        got = run_gpu(fc, w, qc, kc)
        want = _torch_fp32_reference(qc, kc, w.is_causal, w.cls_len, chunk)
        assert_parity(got, want, name)
        np.testing.assert_allclose(got.sum(axis=1), 1.0, atol=1e-3)
        assert (got >= 0).all()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_operands_of_more_than_two_to_the_31_elements(fc):
    """Batch sizes whose operands pass 2^31 elements (4.8 GB each): every call form agrees with
    the same call on 256 batch entries at a time, and the last entries -- past the 32-bit mark
    -- with the fp32 materialising evaluation."""
    if torch.cuda.mem_get_info()[0] < (14 << 30):
        pytest.skip("needs 14 GB of free device memory")
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        B, H, S, D = 2304, 16, 1024, 64
        g = torch.Generator(device="cuda").manual_seed(5)
        q = torch.randn(B, H, S, D, generator=g, device="cuda", dtype=torch.float16)
        k = torch.randn(B, H, S, D, generator=g, device="cuda", dtype=torch.float16)
        assert q.numel() > 2 ** 31
        forms = {
            "all rows": lambda a, b: fc.flash_colsum(a, b),
            "cls prefix": lambda a, b: fc.flash_colsum(a, b, cls_len=1),
            "causal suffix": lambda a, b: fc.flash_colsum_causal(a[:, :, -128:], b),
        }
        for name, call in forms.items():
            full = call(q, k)
            parts = torch.cat([call(q[b:b + 256], k[b:b + 256]) for b in range(0, B, 256)], dim=0)
            assert fc.device_status() == 0
            rel = float((full - parts).norm() / parts.norm())
            assert rel <= 1e-4, (name, rel)
        tail = slice(B - 2, B)
        for name, causal, cls_len, rows in (("all rows", False, None, slice(None)), ("cls prefix", False, 1, slice(None)),
                                            ("causal suffix", True, None, slice(S - 128, S))):
            got = forms[name](q, k)[tail].cpu().numpy()
            want = _torch_fp32_reference(q[tail, :, rows], k[tail], causal, cls_len, 4)
            assert_parity(got, want, name)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_key_axes_of_millions_of_keys(fc):
    """Key axes of two and three million keys (ragged, one and 128 suffix queries): all heads in one
    call agree with the heads taken one by one, every column mean sums to one over the keys, and
    the last keys -- seen only by the last queries -- match a direct evaluation of those queries."""
    if torch.cuda.mem_get_info()[0] < (8 << 30):
        pytest.skip("needs 8 GB of free device memory")
    g = torch.Generator(device="cuda").manual_seed(12)
    for (H, Sq, Sk, D) in [(2, 128, 3000001, 128), (8, 1, 1 << 21, 128)]:
        q = torch.randn(1, H, Sq, D, generator=g, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(1, H, Sk, D, generator=g, device="cuda", dtype=torch.bfloat16)
        full = fc.flash_colsum(q, k, is_causal=True)
        parts = torch.stack([fc.flash_colsum(q[:, h:h + 1], k[:, h:h + 1], is_causal=True) for h in range(H)]).mean(0)
        torch.cuda.synchronize()
        assert fc.device_status() == 0
        assert float((full - parts).norm() / parts.norm()) <= 1e-5
        assert abs(float(full.sum()) - 1.0) <= 1e-4 and bool((full >= 0).all())
        # the last query alone: softmax over all keys, its weight on the last key is that key's whole column sum
        s = (q[0, :, -1:].float() @ k[0].float().transpose(-1, -2)) / D ** 0.5          # (H, 1, Sk)
        p_last = torch.softmax(s, dim=-1)[:, 0, -1].sum() / (H * Sq)
        assert abs(float(full[0, -1]) - float(p_last)) <= 1e-3 * float(p_last) + 1e-12
        del q, k, s


def test_long_inputs_take_the_interleaved_column_schedule(fc):
    """More than 300 000 query rows: the column pass deals (b, h, key tile) chunks round-robin.
    Non-causal with ragged sizes, and causal with more than one batch entry."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        w = Workload("long_rows", 2, 16, 10200, 10200, 64, "fp16", seed=21)
        q, k = make_inputs(w)
        qc, kc = q.cuda(), k.cuda()
        got = run_gpu(fc, w, qc, kc)
        assert_parity(got, _torch_fp32_reference(qc, kc, False, None, 2), w.name)
        np.testing.assert_allclose(got.sum(axis=1), 1.0, atol=1e-3)
        w = Workload("long_rows_causal", 2, 8, 20000, 20100, 128, "bf16", is_causal=True, seed=22)
        q, k = make_inputs(w)
        qc, kc = q.cuda(), k.cuda()
        got = fc.flash_colsum_causal(qc, kc).cpu().numpy()
        assert fc.device_status() == 0
        assert_parity(got, _torch_fp32_reference(qc, kc, True, None, 1), w.name)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


REFERENCE_TEST_SHAPES = [
    # the shapes of the reference's own GPU tests that are not already above at full size
    Workload("ref_non_batched", 1, 16, 8192, 8192, 64, "fp16", seed=0),                 # test_core.py:39-53
    Workload("ref_non_batched_cls2", 1, 16, 4096, 4096, 64, "fp16", cls_len=2, seed=0),  # test_core.py:76-91
    Workload("ref_causal", 1, 16, 128, 16384, 128, "fp16", is_causal=True, seed=0),      # test_core.py:95-109
]


@pytest.mark.parametrize("w", REFERENCE_TEST_SHAPES, ids=lambda w: w.name)
def test_reference_test_shapes_full_size(fc, w):
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        q, k = make_inputs(w)
        qc, kc = q.cuda(), k.cuda()
        got = run_gpu(fc, w, qc, kc)
        want = _torch_fp32_reference(qc, kc, w.is_causal, w.cls_len, 2)
        assert_parity(got, want, w.name)
        # what the reference's test asserts, on the dtype its kernels return
        half = fc.flash_colsum(qc, kc, is_causal=w.is_causal, cls_len=w.cls_len, out_dtype=torch.float16)
        assert torch.allclose(torch.from_numpy(want).half(), half.cpu(), atol=1e-3, rtol=1e-3)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_large_scores_and_peaked_rows(fc):
    """Inputs three times the usual magnitude: scores of several tens, nearly one-hot rows."""
    for w in (Workload("big_noncausal", 2, 4, 640, 640, 64, "fp16", seed=61),
              Workload("big_causal", 1, 4, 256, 2048, 128, "bf16", is_causal=True, seed=62)):
        q, k = make_inputs(w)
        q, k = (q.float() * 3).to(w.torch_dtype), (k.float() * 3).to(w.torch_dtype)
        got = run_gpu(fc, w, q, k)
        want = c_oracle.colsum_c(q, k, is_causal=w.is_causal)
        assert_parity(got, want, w.name)


def test_c5_long_context_properties_and_sampled_parity(fc):
    """131072 keys, 512 suffix queries, outlier keys, bf16: rows sum to one, the
    last key is seen by the last query only, and a 4-head slice matches the
    materialising fp32 evaluation."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        w = WORKLOADS["c5"]
        q, k = make_inputs(w)
        qc, kc = q.cuda(), k.cuda()
        got = run_gpu(fc, w, qc, kc)
        assert got.shape == (1, w.Sk)
        assert abs(got.sum() - 1.0) < 1e-3 and (got >= 0).all()
        want = _torch_fp32_reference(qc, kc, True, None, 2)
        assert_parity(got, want, "c5")
        sl = Workload("c5_slice", 1, 4, 512, 131072, 128, "bf16", is_causal=True)
        got4 = run_gpu(fc, sl, qc[:, 8:12], kc[:, 8:12])
        want4 = _torch_fp32_reference(qc[:, 8:12], kc[:, 8:12], True, None, 2)
        assert_parity(got4, want4, "c5 heads 8..11")
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


def test_batched_causal_and_explicit_k_past(fc):
    """Causal column means for B > 1, for fewer keys than queries, and with the launcher's
    K_past given explicitly -- what the reference's naive_colsum and causal launcher define
    but its operator does not offer."""
    from oracle.naive_colsum import naive_colsum_f64
    # batch of three, ragged sizes, both head dimensions
    for (B, H, Sq, Sk, D, dtype) in [(3, 2, 200, 500, 64, "bf16"), (2, 3, 128, 1024, 128, "fp16"),
                                     (3, 2, 130, 2300, 64, "fp16")]:
        w = Workload("bc", B, H, Sq, Sk, D, dtype, is_causal=True, seed=Sq + Sk)
        q, k = make_inputs(w)
        got = fc.flash_colsum_causal(q.cuda(), k.cuda()).cpu().numpy()
        assert fc.device_status() == 0
        assert got.shape == (B, Sk)
        assert_parity(got, c_oracle.colsum_c(q, k, is_causal=True), f"batched causal {B}x{H}x{Sq}x{Sk}")
    # the operator itself keeps the reference's refusal
    with pytest.raises(ValueError, match="batch size 1"):
        fc.flash_colsum(q.cuda(), k.cuda(), is_causal=True)
    # fewer keys than queries: every query sees keys up to its own index
    w = Workload("short_keys", 2, 2, 300, 120, 64, "fp16", is_causal=True, seed=4)
    q, k = make_inputs(w)
    got = fc.flash_colsum_causal(q.cuda(), k.cuda()).cpu().numpy()
    assert_parity(got, c_oracle.colsum_c(q, k, is_causal=True), "k_len < q_len")
    # explicit K_past, below / at / above the inferred value (300), and beyond the key axis
    w = Workload("k_past", 1, 4, 100, 400, 128, "fp16", is_causal=True, seed=8)
    q, k = make_inputs(w)
    for k_past in (0, 50, 300, 350, 1000):
        got = fc.flash_colsum_causal(q.cuda(), k.cuda(), k_past=k_past).cpu().numpy()
        assert fc.device_status() == 0
        assert_parity(got, naive_colsum_f64(q, k, is_causal=True, k_past=k_past), f"k_past {k_past}")
        np.testing.assert_allclose(got.sum(axis=1), 1.0, rtol=1e-4)
    # explicit K_past over a long key axis (the column pass streams key tiles head by head)
    wl = Workload("k_past_long", 1, 4, 100, 2500, 128, "fp16", is_causal=True, seed=9)
    ql, kl = make_inputs(wl)
    for k_past in (2100, 2400, 2450, 5000):
        got = fc.flash_colsum_causal(ql.cuda(), kl.cuda(), k_past=k_past).cpu().numpy()
        assert fc.device_status() == 0
        assert_parity(got, naive_colsum_f64(ql, kl, is_causal=True, k_past=k_past), f"long k_past {k_past}")
    # explicit K_past that splits the key range of the statistics pass further than the inferred
    # value would (the scratch is sized for the K_past the call passes), and one beyond the keys
    for (H, Sq, Sk, k_past) in ((1, 300, 400, 300), (1, 512, 400, 1000), (8, 1024, 1024, 1024)):
        ws = Workload("k_past_scratch", 1, H, Sq, Sk, 128, "bf16", is_causal=True, seed=10)
        qs, ks = make_inputs(ws)
        got = fc.flash_colsum_causal(qs.cuda(), ks.cuda(), k_past=k_past).cpu().numpy()
        assert fc.device_status() == 0
        assert_parity(got, naive_colsum_f64(qs, ks, is_causal=True, k_past=k_past), f"scratch k_past {H} {Sq} {Sk} {k_past}")
    default = fc.flash_colsum_causal(q.cuda(), k.cuda())
    # same kernels, same masks; only the order of the atomic adds differs between calls
    torch.testing.assert_close(default, fc.flash_colsum_causal(q.cuda(), k.cuda(), k_past=300), rtol=1e-5, atol=0)
    torch.testing.assert_close(default, fc.flash_colsum(q.cuda(), k.cuda(), is_causal=True), rtol=1e-5, atol=0)
    with pytest.raises(ValueError, match="non-negative"):
        fc.flash_colsum_causal(q.cuda(), k.cuda(), k_past=-2)


SHORT_AXES = [
    # B, H, Sq, Sk, D, dtype, causal, scale, k_past
    (1, 32, 128, 4096, 128, "fp16", True, None, None),      # the reference's causal test shape: clusters of four
    (1, 8, 128, 4096, 128, "bf16", True, None, None),       # clusters of eight
    (1, 2, 7, 7, 128, "bf16", False, None, None),           # one block, one CTA per head
    (1, 3, 100, 1000, 64, "fp16", True, None, None),
    (2, 4, 64, 300, 64, "fp16", True, None, None),          # batched causal
    (1, 5, 128, 100, 64, "fp16", True, None, None),         # fewer keys than queries
    (1, 6, 33, 2049, 128, "fp16", True, None, None),        # one key in the last block
    (1, 32, 64, 2048, 80, "fp16", True, None, None),        # head dimension padded to 128 columns
    (1, 4, 128, 3000, 64, "bf16", True, -0.2, None),        # negative scale: the MMA negates
    (1, 4, 90, 1500, 128, "fp16", True, 1e-5, None),        # scale too small for the extra columns
    (1, 4, 100, 2000, 128, "fp16", True, None, 0),          # explicit K_past: only the first keys are seen
    (1, 4, 100, 2000, 128, "fp16", True, None, 700),
    (1, 4, 100, 2000, 128, "bf16", True, None, 5000),       # beyond the key axis: no mask left
    (3, 70, 20, 600, 64, "fp16", True, None, None),         # more (batch, head) pairs than SMs: several waves
    (1, 16, 128, 40000, 128, "bf16", True, None, None),     # 20 blocks per CTA
]


@pytest.mark.parametrize("B,H,Sq,Sk,D,dtype,causal,scale,k_past", SHORT_AXES)
def test_short_query_axes_in_one_kernel(fc, B, H, Sq, Sk, D, dtype, causal, scale, k_past):
    """At most 128 query rows: the one-kernel cluster form (statistics, exchange through
    distributed shared memory, columns) against the float64 evaluation, and against the two
    streaming passes on the same inputs."""
    from flash_colsum_b200 import _cabi
    from oracle.naive_colsum import naive_colsum_f64
    w = Workload("short", B, H, Sq, Sk, D, dtype, is_causal=causal, seed=B + H + Sq + Sk)
    q, k = make_inputs(w)
    qc, kc = q.cuda(), k.cuda()

    def call():
        if causal:
            return fc.flash_colsum_causal(qc, kc, scale=scale, k_past=k_past)
        return fc.flash_colsum(qc, kc, scale=scale)
    want = naive_colsum_f64(q, k, scale=scale, is_causal=causal, k_past=k_past)
    try:
        _cabi.set_short_fused(_cabi.SHORT_FUSED_ALWAYS)
        assert _cabi.short_fused_applies(B, H, Sq, Sk, causal, -1 if k_past is None else k_past, D) is not None
        assert _cabi.call_workspace_bytes(B, H, Sq, Sk, D, causal, -1 if k_past is None else k_past) == 0
        got = call()
        torch.cuda.synchronize()
        assert fc.device_status() == 0
        again = call()                      # a second call in a row: nothing is left over from the first
        _cabi.set_short_fused(_cabi.SHORT_FUSED_NEVER)
        two_pass = call()
        torch.cuda.synchronize()
        assert fc.device_status() == 0
    finally:
        _cabi.set_short_fused(_cabi.SHORT_FUSED_AUTO)
    assert_parity(got.cpu().numpy(), want, f"one kernel {B}x{H}x{Sq}x{Sk}x{D}")
    assert_parity(two_pass.cpu().numpy(), want, f"two passes {B}x{H}x{Sq}x{Sk}x{D}")
    torch.testing.assert_close(got, again, rtol=1e-5, atol=1e-9)
    np.testing.assert_allclose(got.sum(dim=1).cpu().numpy(), 1.0, rtol=1e-4)


def test_short_query_axes_accumulate_and_graph_capture(fc):
    """The accumulate entry adds into what the buffer holds (no clearing kernel in front), and a
    call of the one-kernel form replays from a CUDA graph."""
    from flash_colsum_b200 import _cabi
    w = Workload("short_acc", 1, 8, 128, 3000, 128, "fp16", is_causal=True, seed=77)
    q, k = make_inputs(w)
    qc, kc = q.cuda(), k.cuda()
    assert _cabi.short_fused_applies(1, 4, 128, 3000) is not None
    want = c_oracle.colsum_c(q, k, is_causal=True)
    from flash_colsum_b200 import ops
    total = torch.zeros(3000, device="cuda", dtype=torch.float32)
    for h0 in (0, 4):      # two shards of four heads each, normalised by all eight
        ops._flash_colsum_causal(qc[:, h0:h0 + 4], kc[:, h0:h0 + 4], 1.0 / 128 ** 0.5, h_norm=8, accumulate_into=total)
    torch.cuda.synchronize()
    assert fc.device_status() == 0
    assert_parity(total.cpu().numpy()[None, :], want, "two head shards into one buffer")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(2):
            fc.flash_colsum(qc, kc, is_causal=True)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fc.flash_colsum(qc, kc, is_causal=True)
    for _ in range(3):
        out.fill_(-1.0)
        graph.replay()
    torch.cuda.synchronize()
    assert fc.device_status() == 0
    assert_parity(out.cpu().numpy(), want, "graph replay")


def test_random_shapes_through_every_kernel_choice(fc):
    """Sixty seeded random shapes (ragged sizes, both dtypes, head dimensions from 8 to 128, causal
    with and without an explicit K_past, CLS prefixes) against the C checker: whichever kernel the
    library picks for a shape -- few-row, single-pass, one-kernel cluster form, streaming passes --
    the result is the same function of the inputs."""
    from flash_colsum_b200 import _cabi
    from oracle.naive_colsum import naive_colsum_f64
    rng = np.random.default_rng(20240607)
    took = {"few_rows": 0, "one_kernel": 0, "single_pass": 0, "streaming": 0}
    for case in range(60):
        causal = bool(rng.integers(0, 2))
        D = int(rng.choice([8, 32, 64, 64, 80, 128, 128]))
        dtype = "fp16" if rng.integers(0, 2) else "bf16"
        B = int(rng.integers(1, 4))
        H = int(rng.integers(1, 7))
        Sk = int(rng.choice([1, 17, 128, 255, 256, 257, 600, 1000, 1537, 2200, 3100]))
        if causal:
            Sq = int(rng.choice([1, 2, 4, 5, 64, 100, 128, 129, 300, 520]))
            k_past = None if rng.integers(0, 2) else int(rng.integers(0, Sk + 50))
            cls_len = None
        else:
            Sq, k_past = Sk, None
            cls_len = None if rng.integers(0, 2) else int(rng.choice([1, 3, 4, 5, 40, 128, 129, 300]))
        w = Workload(f"fuzz{case}", B, H, Sq, Sk, D, dtype, is_causal=causal, cls_len=cls_len, seed=1000 + case)
        q, k = make_inputs(w)
        if causal:
            got = fc.flash_colsum_causal(q.cuda(), k.cuda(), k_past=k_past)
        else:
            got = fc.flash_colsum(q.cuda(), k.cuda(), cls_len=cls_len)
        torch.cuda.synchronize()
        assert fc.device_status() == 0, w
        want = naive_colsum_f64(q, k, is_causal=causal, cls_len=cls_len, k_past=k_past)
        assert_parity(got.cpu().numpy(), want, f"{w} k_past={k_past}")
        rows = Sq if cls_len is None else min(cls_len, Sq)
        if rows <= 4 and D in (64, 128):
            took["few_rows"] += 1
        elif _cabi.short_fused_applies(B, H, rows, Sk, causal, -1 if k_past is None else k_past, D) is not None:
            took["one_kernel"] += 1     # (a few of these go to the single-pass kernel: more than one wave)
        elif _cabi.single_pass_applies(B, H, Sk, D, causal, rows):
            took["single_pass"] += 1
        else:
            took["streaming"] += 1
    assert min(took.values()) >= 3, took


def test_topk_columns_matches_a_plain_sort(fc):
    """The pruning step: exact top-k positions per row, ascending, ties to the lower position."""
    from oracle.naive_colsum import topk_positions
    w = Workload("topk", 3, 4, 577, 577, 64, "fp16", seed=12)
    q, k = make_inputs(w)
    col = fc.flash_colsum(q.cuda(), k.cuda())
    for kk in (1, 7, 144, 576, 577):
        val, idx = fc.topk_columns(col, kk)
        want = topk_positions(col.cpu().numpy(), kk)
        np.testing.assert_array_equal(idx.cpu().numpy(), want)
        np.testing.assert_array_equal(val.cpu().numpy(), np.take_along_axis(col.cpu().numpy(), want, axis=1))
    # heavy ties, zeros, a long row, a padded row stride
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 5, (2, 70000), generator=g).float() * 0.25
    x[0, 100:200] = 0.0
    xp = torch.zeros(2, 70016)
    xp[:, :70000] = x
    view = xp.cuda()[:, :70000]
    for kk in (1, 1000, 35000, 70000):
        val, idx = fc.topk_columns(view, kk)
        np.testing.assert_array_equal(idx.cpu().numpy(), topk_positions(x.numpy(), kk))
    # negative values order correctly too
    y = torch.randn(4, 333, generator=g)
    val, idx = fc.topk_columns(y.cuda(), 50)
    np.testing.assert_array_equal(idx.cpu().numpy(), topk_positions(y.numpy(), 50))
    with pytest.raises(ValueError):
        fc.topk_columns(col, 0)
    with pytest.raises(ValueError):
        fc.topk_columns(col, 578)


def test_passes_run_apart_reproduce_the_call(fc):
    """The work split over devices, emulated on one: statistics per share of the query rows,
    the vectors concatenated, column means per share of the keys -- equal to the whole call."""
    from flash_colsum_b200 import ops
    from flash_colsum_b200.sharded import work_shares
    for (B, H, S, D, dtype, cls, world) in [(1, 3, 1500, 64, "fp16", None, 3), (2, 2, 700, 128, "bf16", None, 2),
                                            (1, 2, 1100, 64, "fp16", 600, 4), (1, 1, 300, 64, "fp16", None, 8),
                                            # few rows over many keys: the column shares take the short-query modes
                                            (1, 2, 4200, 64, "fp16", 400, 2), (1, 2, 4200, 128, "bf16", 100, 2)]:
        w = Workload("apart", B, H, S, S, D, dtype, cls_len=cls, seed=S + world)
        q, k = make_inputs(w)
        qc, kc = q.cuda(), k.cuda()
        rows = S if cls is None else min(cls, S)
        scale = 1.0 / D ** 0.5
        q_share, q_ranges = work_shares(rows, world, 256)
        pieces = []
        for lo, hi in q_ranges:
            piece = torch.full((B * H, q_share), float("-inf"), device="cuda")
            if hi > lo:
                part = ops.colsum_statistics(qc[:, :, lo:hi], kc, scale, rows)
                assert part.shape == (B * H, ops.statistics_rows(hi - lo))
                piece[:, :part.shape[1]] = part
            pieces.append(piece)
        neg_lse = torch.cat(pieces, dim=1)[:, :ops.statistics_rows(rows)].contiguous()
        k_share, k_ranges = work_shares(S, world, 128)
        cols = [ops.colsum_columns(qc[:, :, :rows], kc[:, :, lo:hi], neg_lse, scale) for lo, hi in k_ranges if hi > lo]
        got = torch.cat(cols, dim=1)
        assert fc.device_status() == 0
        assert got.shape == (B, S)
        assert_parity(got.cpu().numpy(), c_oracle.colsum_c(q, k, cls_len=cls), f"apart {B}x{H}x{S} world {world}")
        torch.testing.assert_close(got, fc.flash_colsum(qc, kc, cls_len=cls), rtol=2e-4, atol=1e-9)
    with pytest.raises(RuntimeError, match="norm_rows"):
        ops.colsum_statistics(qc[:, :, :256], kc, scale, 100)


def test_head_shards_accumulate_into_one_buffer(fc):
    """The accumulate entry (what head-sharded ranks call with a possibly peer-mapped buffer):
    two head shards added into one cleared buffer, normalised by the total head count, give the
    unsharded result -- on the short-query column modes, whose consumer groups combine their sums
    in shared memory before the one add per key that this entry issues."""
    from flash_colsum_b200 import ops
    for (H, Sq, Sk, D, dtype) in [(4, 33, 2300, 128, "fp16"),      # a third of a tile's columns
                                  (6, 100, 2500, 64, "bf16"),      # one query block, two key tiles per step
                                  (4, 256, 3000, 128, "fp16"),     # one query block, one key tile per step
                                  (6, 400, 2500, 128, "bf16"),     # two resident query blocks
                                  (4, 130, 2177, 64, "fp16")]:     # ragged: an odd number of key tiles
        w = Workload("acc", 1, H, Sq, Sk, D, dtype, is_causal=True, seed=H + Sq + Sk)
        q, k = make_inputs(w)
        qd, kd = q.cuda(), k.cuda()
        target = torch.zeros(Sk, device="cuda", dtype=torch.float32)
        half = H // 2
        scale = 1.0 / D ** 0.5
        for lo, hi in ((0, half), (half, H)):
            ops._flash_colsum_causal(qd[:, lo:hi], kd[:, lo:hi], scale, h_norm=H, accumulate_into=target)
        torch.cuda.synchronize()
        assert fc.device_status() == 0
        got = target.cpu().numpy()[None, :]
        assert_parity(got, c_oracle.colsum_c(q, k, is_causal=True), f"accumulate {H}x{Sq}x{Sk}x{D}")


def test_accumulate_entry_clears_the_buffer_of_the_next_call(fc):
    """A reduce target that alternates between two buffers: every call adds into one and zeroes
    the other inside its own kernels (streaming passes, and the few-row kernel), so that a run of
    calls needs no clearing kernel.  The buffer of the next call starts out dirty here."""
    from flash_colsum_b200 import ops
    for (H, Sq, Sk, D, dtype) in [(4, 100, 2500, 128, "bf16"), (4, 3, 1500, 64, "fp16")]:
        w = Workload("acc", 1, H, Sq, Sk, D, dtype, is_causal=True, seed=H + Sq + Sk)
        q, k = make_inputs(w)
        qd, kd = q.cuda(), k.cuda()
        want = c_oracle.colsum_c(q, k, is_causal=True)
        bufs = torch.full((2, Sk), 7.0, device="cuda", dtype=torch.float32)
        bufs[0].zero_()
        scale = 1.0 / D ** 0.5
        for call in range(4):
            p = call & 1
            # two head shards meet in the buffer of this call; the first one clears the other buffer
            ops._flash_colsum_causal(qd[:, :2], kd[:, :2], scale, h_norm=H, accumulate_into=bufs[p],
                                     clear_next=bufs[p ^ 1])
            ops._flash_colsum_causal(qd[:, 2:], kd[:, 2:], scale, h_norm=H, accumulate_into=bufs[p])
            torch.cuda.synchronize()
            assert fc.device_status() == 0
            assert_parity(bufs[p].cpu().numpy()[None, :], want, f"alternating target, call {call}")
            assert float(bufs[p ^ 1].abs().max().item()) == 0.0


def test_threshold_columns_matches_a_plain_filter(fc):
    """The threshold form of the pruning step: kept positions ascending, the count per row, -1 after."""
    w = Workload("thr", 3, 4, 1500, 1500, 64, "fp16", seed=13)
    q, k = make_inputs(w)
    col = fc.flash_colsum(q.cuda(), k.cuda())
    host = col.cpu().numpy()
    for thr, rel in ((1.0 / 1500, False), (0.0, False), (1.0, True), (1.5, True), (10.0, False)):
        idx, cnt = fc.threshold_columns(col, thr, relative=rel)
        idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
        for b in range(3):
            cut = np.float32(thr) * (host[b].sum(dtype=np.float32) / np.float32(1500)) if rel else np.float32(thr)
            keep = np.nonzero(host[b] >= cut)[0]
            if rel:     # the kernel's row sum is taken in another order: leave out values at the cut itself
                margin = np.abs(host[b] - cut) < 1e-6 * cut
                assert np.array_equal(idx[b, :cnt[b]][~margin[idx[b, :cnt[b]]]], keep[~margin[keep]])
            else:
                assert cnt[b] == len(keep) and np.array_equal(idx[b, :cnt[b]], keep)
            assert (idx[b, cnt[b]:] == -1).all()
    with pytest.raises(ValueError):
        fc.threshold_columns(col.half(), 0.1)


def test_a_wait_that_runs_out_reports_a_status_and_leaves_the_context_usable(fc):
    """The bounded waits of the streaming kernel: a statistics pass whose producer issues no copies
    (the flag nothing sets), with the limit lowered to 50 ms for that launch.  The waits for data
    run out, the CTA aborts through its teardown (tensor memory freed), the status word says
    which role gave up -- and the next ordinary call on the same stream is correct."""
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    q = torch.randn(128, 64, device="cuda").half()
    k = torch.randn(256, 64, device="cuda").half()
    ws = torch.empty(lib.fcs_workspace_bytes(1, 1, 128, 256, 64, 0), dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fcs_selftest_wait_expiry(q.data_ptr(), k.data_ptr(), ws.data_ptr(), ws.numel(), status.data_ptr(),
                                        0.05, stream) == 0, _cabi.last_error()
    torch.cuda.synchronize()
    assert int(status.item()) in (2, 3)       # FCS_STATUS_WAIT_MMA or FCS_STATUS_WAIT_CONSUMER
    assert lib.fcs_selftest_wait_expiry(q.data_ptr(), k.data_ptr(), ws.data_ptr(), ws.numel(), status.data_ptr(),
                                        5.0, stream) == -1     # the limit is capped
    # the library's own status word was not involved, and the kernels run as before
    w = Workload("after", 2, 3, 700, 700, 64, "fp16", seed=99)
    qq, kk = make_inputs(w)
    got = run_gpu(fc, w, qq, kk)
    assert_parity(got, c_oracle.colsum_c(qq, kk), "call after an expired wait")


def test_a_wait_that_runs_out_in_a_cluster_kernel(fc):
    """The same for a kernel on thread-block clusters (the one-kernel form for short query axes, a
    cluster of two CTAs): with nothing copied every CTA's waits run out after 50 ms, the CTAs still
    meet at their barriers and leave together, the status word is set, nothing was added to the
    output -- and the same kernel then computes a real call correctly."""
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    q = torch.randn(128, 64, device="cuda").half()
    k = torch.randn(512, 64, device="cuda").half()
    out = torch.full((512,), 7.0, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.fcs_selftest_wait_expiry_cluster(q.data_ptr(), k.data_ptr(), out.data_ptr(), status.data_ptr(),
                                                0.05, stream) == 0, _cabi.last_error()
    torch.cuda.synchronize()
    assert int(status.item()) in (2, 3)       # FCS_STATUS_WAIT_MMA or FCS_STATUS_WAIT_CONSUMER
    assert float(out.abs().max().item()) == 0.0
    w = Workload("after_cluster", 1, 6, 128, 900, 64, "fp16", is_causal=True, seed=98)
    qq, kk = make_inputs(w)
    assert _cabi.short_fused_applies(1, 6, 128, 900, True, -1, 64) is not None
    got = run_gpu(fc, w, qq, kk)
    assert_parity(got, c_oracle.colsum_c(qq, kk, is_causal=True), "call after an expired wait in a cluster")


def test_agrees_with_the_reference_kernels_where_they_are_exact(fc):
    """Against the reference's own Triton kernels (an unmodified install of the reference in
    baseline/_ref; skipped when there is none) on shapes where those kernels follow
    ``naive_colsum``: head dimension 64 and key lengths that are multiples of their tiles.
    Their result is fp16, so the bar is wider than against the checker."""
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    ref_dir = os.path.join(root, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "flash_colsum")):
        pytest.skip("no install of the reference in baseline/_ref")
    if ref_dir not in sys.path:
        sys.path.append(ref_dir)
    try:
        from flash_colsum import flash_colsum as ref_flash_colsum
    except Exception as exc:      # Triton missing or not importable here
        pytest.skip(f"the reference does not import: {exc}")
    for (B, H, Sq, Sk, causal) in [(4, 8, 1024, 1024, False), (1, 8, 2048, 2048, False), (1, 8, 128, 4096, True)]:
        w = Workload("ref", B, H, Sq, Sk, 64, "fp16", is_causal=causal, seed=B + Sk)
        q, k = make_inputs(w)
        qd, kd = q.cuda(), k.cuda()
        theirs = ref_flash_colsum(qd, kd, is_causal=causal).float()
        ours = fc.flash_colsum(qd, kd, is_causal=causal)
        torch.cuda.synchronize()
        rel = float(((ours - theirs).norm() / ours.norm()).item())
        assert theirs.shape == ours.shape and rel <= 3e-3, (B, H, Sq, Sk, causal, rel)


def test_signalled_accumulate_entry_posts_its_flags(fc):
    """The accumulate entry whose column pass carries the flags of a head-sharded call, on one GPU
    with every flag in local memory: the wait is already satisfied (nothing on this GPU waits for
    another kernel), the owner's "clear" flags and the "share is in" flag are stored, the counter
    returns to zero, the sum is right -- and a few-row call is refused so that its caller falls
    back to flags around the call."""
    from flash_colsum_b200 import _cabi, ops
    # two query blocks over many key tiles (the short-query column mode), then a longer query axis
    # (the generic column mode, which takes the flag pointers from its shared-memory copy of the call)
    for w in (Workload("sig", 1, 4, 300, 2500, 128, "bf16", is_causal=True, seed=55),
              Workload("sig_generic", 1, 4, 1100, 1500, 64, "fp16", is_causal=True, seed=56)):
        _signalled_accumulate_case(fc, w)


def _signalled_accumulate_case(fc, w):
    from flash_colsum_b200 import _cabi, ops
    q, k = make_inputs(w)
    qd, kd = q.cuda(), k.cuda()
    want = c_oracle.colsum_c(q, k, is_causal=True)
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")
    target = torch.zeros(w.Sk, device="cuda")
    nxt = torch.full((w.Sk,), 3.0, device="cuda")
    base = flags.data_ptr()
    # first two heads as "the owner" (posts two clear flags, clears the next buffer) ...
    sig = _cabi.PeerSignals()
    sig.post[0], sig.post[1] = base + 4, base + 8
    sig.post_n, sig.post_value = 2, 7
    scale = 1.0 / w.D ** 0.5
    assert ops._flash_colsum_causal(qd[:, :2], kd[:, :2], scale, h_norm=4, accumulate_into=target,
                                    clear_next=nxt, signals=sig) is not None
    # ... the other two as "another rank" (waits for a flag that is already there, reports completion)
    sig = _cabi.PeerSignals()
    flags[0] = 5
    sig.wait_flag, sig.wait_value = base, 5
    sig.counter, sig.done_flag, sig.done_value = base + 16, base + 12, 9
    assert ops._flash_colsum_causal(qd[:, 2:], kd[:, 2:], scale, h_norm=4, accumulate_into=target,
                                    signals=sig) is not None
    torch.cuda.synchronize()
    assert fc.device_status() == 0
    assert flags.tolist()[:5] == [5, 7, 7, 9, 0]
    assert float(nxt.abs().max().item()) == 0.0
    assert_parity(target.cpu().numpy()[None, :], want, "signalled accumulate")
    # two decode queries: the few-row kernel cannot carry the flags
    assert ops._flash_colsum_causal(qd[:, :, :2], kd, scale, accumulate_into=target, signals=sig) is None
