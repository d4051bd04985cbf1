"""The single-pass cluster kernel (non-causal, head dimension 64, at most 2048 keys)
against the CPU checker, and against the two-pass kernels on the same inputs.
`fcs_set_single_pass` forces one kernel or the other; the default picks by shape."""

import numpy as np
import pytest
import torch

from conftest import MAX_ABS_TOL, REL_L2_TOL
from flash_colsum_b200.inputs import Workload, make_inputs
from oracle import c_oracle
from oracle.naive_colsum import parity_errors

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def fc():
    if not torch.cuda.is_available():
        pytest.fail("the gpu-marked tests need a CUDA device")
    import flash_colsum_b200
    return flash_colsum_b200


@pytest.fixture
def kernel_choice():
    """Yields the setter; whatever a test chose, the default is back afterwards."""
    from flash_colsum_b200 import _cabi
    try:
        yield _cabi.set_single_pass
    finally:
        _cabi.set_single_pass(_cabi.SINGLE_PASS_AUTO)


def run(fc, w, q, k, **kw):
    out = fc.flash_colsum(q.cuda(), k.cuda(), cls_len=w.cls_len, **kw)
    torch.cuda.synchronize()
    assert fc.device_status() == 0, "a device-side wait expired"
    return out.cpu().numpy()


def assert_parity(got, want, what):
    rel, mx = parity_errors(got, want)
    assert np.isfinite(got).all(), what
    assert rel <= REL_L2_TOL and mx <= MAX_ABS_TOL, (what, rel, mx)


SHAPES = [
    # B, H, S, dtype, cls_len          cluster size, what it exercises
    (1, 1, 128, "fp16", None),       # 1, a single tile
    (2, 3, 256, "fp16", None),       # 1, two tiles per (batch, head), several heads per cluster
    (2, 2, 100, "fp16", None),       # 1, ragged keys and queries inside one tile
    (3, 2, 300, "bf16", None),       # 2, ragged second slice
    (2, 2, 512, "fp16", None),       # 2
    (2, 3, 577, "fp16", None),       # 3, one key in the last slice's first group
    (2, 2, 1200, "bf16", None),      # 5
    (1, 3, 1536, "fp16", None),      # 6
    (2, 2, 1700, "fp16", None),      # 7
    (2, 4, 1024, "fp16", None),      # 4
    (3, 5, 1500, "bf16", None),      # 6, ragged, more (batch, head) pairs than clusters can split evenly
    (2, 4, 2048, "fp16", None),      # 8, the longest key axis
    (3, 4, 577, "fp16", 5),          # cls_len: five query rows (more than the few-row kernel takes)
    (3, 4, 577, "fp16", 200),        # cls_len: ragged second query tile
    (40, 4, 256, "fp16", None),      # more (batch, head) pairs than resident clusters: several per cluster
    (2, 64, 512, "fp16", None),      # many heads: intermediate flushes of the tensor-memory accumulator
]


@pytest.mark.parametrize("B,H,S,dtype,cls", SHAPES)
def test_single_pass_matches_checker(fc, kernel_choice, B, H, S, dtype, cls):
    w = Workload(f"sp_{B}_{H}_{S}_{dtype}_{cls}", B, H, S, S, 64, dtype, cls_len=cls, seed=B * 1000 + S)
    q, k = make_inputs(w)
    want = c_oracle.colsum_c(q, k, cls_len=cls)
    kernel_choice(2)
    got = run(fc, w, q, k)
    assert_parity(got, want, w.name)
    np.testing.assert_allclose(got.sum(axis=1), 1.0, rtol=1e-4)
    # the two-pass kernels on the same inputs (the default may have stopped choosing them here)
    kernel_choice(1)
    assert_parity(run(fc, w, q, k), want, w.name + " two-pass")


def test_single_pass_scale_sign_and_size(fc, kernel_choice):
    w = Workload("sp_scale", 2, 2, 300, 300, 64, "fp16", seed=9)
    q, k = make_inputs(w)
    kernel_choice(2)
    for scale in (-0.2, 1.0, 1e-6, 0.0):
        got = run(fc, w, q, k, scale=scale)
        assert_parity(got, c_oracle.colsum_c(q, k, scale=scale), f"scale {scale}")


def test_single_pass_peaked_rows(fc, kernel_choice):
    """One key dominates every row by a wide margin: the other groups' weights underflow to zero."""
    w = Workload("sp_peaked", 1, 2, 512, 512, 64, "fp16", seed=3)
    q, k = make_inputs(w)
    k[:, :, 77] = 6.0 * q.float().mean(dim=2).sign().half()
    kernel_choice(2)
    got = run(fc, w, q, k, scale=1.0)
    assert_parity(got, c_oracle.colsum_c(q, k, scale=1.0), "peaked")


def test_single_pass_strided_inputs_and_repeats(fc, kernel_choice):
    """Views with padded strides; back-to-back calls on one stream reuse tensor memory and barriers."""
    w = Workload("sp_strided", 2, 3, 384, 384, 64, "fp16", seed=5)
    q, k = make_inputs(w)
    qp = torch.zeros(2, 3, 400, 72, dtype=q.dtype)
    kp = torch.zeros(2, 3, 400, 72, dtype=k.dtype)
    qp[:, :, :384, :64] = q
    kp[:, :, :384, :64] = k
    qv, kv = qp.cuda()[:, :, :384, :64], kp.cuda()[:, :, :384, :64]
    want = c_oracle.colsum_c(q, k)
    kernel_choice(2)
    outs = [fc.flash_colsum(qv, kv) for _ in range(3)]
    torch.cuda.synchronize()
    assert fc.device_status() == 0
    for o in outs:
        assert_parity(o.cpu().numpy(), want, "strided")


def test_single_pass_call_replays_from_a_cuda_graph(fc, kernel_choice):
    """The cluster launch (output clear + one kernel) neither synchronises nor allocates."""
    w = Workload("sp_graph", 2, 4, 512, 512, 64, "fp16", seed=31)
    q, k = (t.cuda() for t in make_inputs(w))
    kernel_choice(2)
    fc.flash_colsum(q, k)                      # first call outside capture (one-time set-up)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fc.flash_colsum(q, k)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = fc.flash_colsum(q, k)
    want = c_oracle.colsum_c(q.cpu(), k.cpu())
    for _ in range(3):
        out.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, "graph replay")
    assert fc.device_status() == 0


def test_default_choice_by_shape(fc, kernel_choice):
    """The default takes the single pass for well-filled short key axes; such a call runs one
    kernel, so it reports (next to) no statistics-pass time."""
    from flash_colsum_b200 import _cabi
    kernel_choice(0)
    assert _cabi.single_pass_applies(8, 16, 512) and _cabi.single_pass_applies(8, 16, 1024)
    assert not _cabi.single_pass_applies(8, 16, 2048) and _cabi.single_pass_applies(1, 16, 2048)
    _cabi.set_profiling(True)
    try:
        def pass_ms(B, H, S):
            g = torch.Generator(device="cuda").manual_seed(0)
            q = torch.randn(B, H, S, 64, device="cuda", dtype=torch.float16, generator=g)
            k = torch.randn(B, H, S, 64, device="cuda", dtype=torch.float16, generator=g)
            for _ in range(3):
                fc.flash_colsum(q, k)
            return _cabi.last_pass_ms()
        single = pass_ms(32, 16, 1024)
        double = pass_ms(32, 16, 2048)
        assert single[0] < 0.25 * single[2]     # no statistics kernel in front of the column sums
        assert double[0] > 0.5 * double[2]      # two kernels of similar length
    finally:
        _cabi.set_profiling(False)
    cl, resident = _cabi.single_pass_info(2048)
    assert cl == 8 and resident >= 1
    assert _cabi.single_pass_info(256)[0] == 1 and _cabi.single_pass_info(577)[0] == 3
