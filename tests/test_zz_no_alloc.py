"""The allocation-free entry point, called straight through the C ABI.

`fcs_colsum_batched_static_scratch` serves hosts that cannot hand the library a
workspace because they have no device allocator of their own to call (a plugin
in a server that owns all device memory, an FFI caller holding only its input
and output buffers).  Its scratch is an array built into the library, shared by
every call on the device.  The test checks that two calls in a row, on
different inputs, each reproduce what the workspace-taking entry point returns
for the same inputs, that the scratch left behind by one call does not leak
into the next, and that a problem too large for the built-in array is refused.
This file is collected last so that a failure here cannot hide another test.
"""

import numpy as np
import pytest
import torch

from conftest import MAX_ABS_TOL, REL_L2_TOL
from flash_colsum_b200.inputs import Workload, make_inputs
from oracle.naive_colsum import parity_errors

pytestmark = pytest.mark.gpu


def _call(lib, fn_name, q, k, out, status, cls_n=-1, workspace=None):
    B, H, S, D = q.shape
    args = [q.data_ptr(), k.data_ptr(), out.data_ptr(), S, B, H, S, D, 0,
            q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
            1.0 / D ** 0.5, cls_n, 0]
    if workspace is not None:
        args += [workspace.data_ptr(), workspace.numel()]
    args += [status.data_ptr(), torch.cuda.current_stream().cuda_stream]
    return getattr(lib, fn_name)(*args)


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.fail("the gpu-marked tests need a CUDA device")
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    shapes = [Workload("first", 4, 8, 512, 512, 64, "fp16", seed=71),
              Workload("second", 2, 3, 300, 300, 128, "fp16", seed=72)]
    for w in shapes:                      # two calls in a row, different sizes and data
        q, k = (t.cuda() for t in make_inputs(w))
        ws_bytes = lib.fcs_workspace_bytes(w.B, w.H, w.Sq, w.Sk, w.D, 0)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        want = torch.full((w.B, w.Sk), float("nan"), device="cuda")
        got = torch.full((w.B, w.Sk), float("nan"), device="cuda")
        assert _call(lib, "fcs_colsum_batched", q, k, want, status, workspace=ws) == 0, _cabi.last_error()
        assert _call(lib, "fcs_colsum_batched_static_scratch", q, k, got, status) == 0, _cabi.last_error()
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        rel, mx = parity_errors(got.cpu().numpy(), want.cpu().numpy())
        assert np.isfinite(got.cpu().numpy()).all()
        assert rel <= REL_L2_TOL and mx <= MAX_ABS_TOL, (w.name, rel, mx)
    # a CLS prefix longer than the few-row kernel takes goes through the same scratch
    w = shapes[0]
    q, k = (t.cuda() for t in make_inputs(w))
    ws = torch.empty(lib.fcs_workspace_bytes(w.B, w.H, 9, w.Sk, w.D, 0), dtype=torch.uint8, device="cuda")
    want = torch.empty((w.B, w.Sk), device="cuda")
    got = torch.empty((w.B, w.Sk), device="cuda")
    assert _call(lib, "fcs_colsum_batched", q, k, want, status, cls_n=9, workspace=ws) == 0
    assert _call(lib, "fcs_colsum_batched_static_scratch", q, k, got, status, cls_n=9) == 0
    torch.cuda.synchronize()
    rel, mx = parity_errors(got.cpu().numpy(), want.cpu().numpy())
    assert rel <= REL_L2_TOL and mx <= MAX_ABS_TOL, ("cls", rel, mx)


def test_static_scratch_entry_takes_calls_that_use_no_scratch_and_allocates_nothing():
    """The CLIP-style CLS call (B=32, H=16, S=577, cls_len=1) runs on the few-row kernel, which
    uses no scratch at all, so the size of the built-in array does not limit it -- although the
    two streaming passes would want 4.5 MiB for it.  Checked against the CPU checker, and the
    device's free memory and torch's allocation count do not move across the call."""
    if not torch.cuda.is_available():
        pytest.fail("the gpu-marked tests need a CUDA device")
    from flash_colsum_b200 import _cabi
    from flash_colsum_b200.inputs import WORKLOADS
    from oracle import c_oracle
    lib = _cabi.load()
    w = WORKLOADS["c3"]
    assert lib.fcs_workspace_bytes(w.B, w.H, 1, w.Sk, w.D, 0) > (4 << 20)
    assert _cabi.call_workspace_bytes(w.B, w.H, 1, w.Sk, w.D, False) == 0
    q, k = make_inputs(w)
    qc, kc = q.cuda(), k.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = torch.full((w.B, w.Sk), float("nan"), device="cuda")
    assert _call(lib, "fcs_colsum_batched_static_scratch", qc, kc, got, status, cls_n=1) == 0   # set-up call
    torch.cuda.synchronize()
    got.fill_(float("nan"))
    free_before, _ = torch.cuda.mem_get_info()
    allocated_before = torch.cuda.memory_allocated()
    segments_before = torch.cuda.memory_stats()["num_alloc_retries"], torch.cuda.memory_reserved()
    assert _call(lib, "fcs_colsum_batched_static_scratch", qc, kc, got, status, cls_n=1) == 0, _cabi.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == allocated_before
    assert (torch.cuda.memory_stats()["num_alloc_retries"], torch.cuda.memory_reserved()) == segments_before
    assert int(status.item()) == 0
    want = c_oracle.colsum_c(q, k, cls_len=1)
    rel, mx = parity_errors(got.cpu().numpy(), want)
    assert rel <= REL_L2_TOL and mx <= MAX_ABS_TOL, ("c3", rel, mx)
    # the workspace-taking entry accepts the same call with no workspace at all
    want2 = torch.empty((w.B, w.Sk), device="cuda")
    args = [qc.data_ptr(), kc.data_ptr(), want2.data_ptr(), w.Sk, w.B, w.H, w.Sk, w.D, 0,
            qc.stride(0), qc.stride(1), qc.stride(2), kc.stride(0), kc.stride(1), kc.stride(2),
            1.0 / w.D ** 0.5, 1, 0, None, 0, status.data_ptr(), torch.cuda.current_stream().cuda_stream]
    assert lib.fcs_colsum_batched(*args) == 0, _cabi.last_error()
    torch.cuda.synchronize()
    torch.testing.assert_close(want2, got, rtol=1e-5, atol=1e-9)


def test_static_scratch_entry_refuses_problems_beyond_its_limit():
    if not torch.cuda.is_available():
        pytest.fail("the gpu-marked tests need a CUDA device")
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    # head dimension 128 always takes the two streaming passes: at least 36 bytes of scratch per
    # query row.  The first batch size whose call needs more than the 4 MiB is refused.
    H, S, D = 16, 512, 128
    B = 1
    while _cabi.call_workspace_bytes(B, H, S, S, D, False) <= (4 << 20):
        B += 1
    assert 2 <= B <= 16
    q = torch.empty(1, dtype=torch.float16, device="cuda")     # never dereferenced: the call is refused first
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.fcs_colsum_batched_static_scratch(
        q.data_ptr(), q.data_ptr(), q.data_ptr(), S, B, H, S, D, 0,
        H * S * D, S * D, D, H * S * D, S * D, D, 0.125, -1, 0,
        status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert "built-in scratch" in _cabi.last_error()
