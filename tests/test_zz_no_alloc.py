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
    # the CLS-prefix form goes through the same scratch
    w = shapes[0]
    q, k = (t.cuda() for t in make_inputs(w))
    ws = torch.empty(lib.fcs_workspace_bytes(w.B, w.H, 1, w.Sk, w.D, 0), dtype=torch.uint8, device="cuda")
    want = torch.empty((w.B, w.Sk), device="cuda")
    got = torch.empty((w.B, w.Sk), device="cuda")
    assert _call(lib, "fcs_colsum_batched", q, k, want, status, cls_n=1, workspace=ws) == 0
    assert _call(lib, "fcs_colsum_batched_static_scratch", q, k, got, status, cls_n=1) == 0
    torch.cuda.synchronize()
    rel, mx = parity_errors(got.cpu().numpy(), want.cpu().numpy())
    assert rel <= REL_L2_TOL and mx <= MAX_ABS_TOL, ("cls", rel, mx)


def test_static_scratch_entry_refuses_problems_beyond_its_limit():
    if not torch.cuda.is_available():
        pytest.fail("the gpu-marked tests need a CUDA device")
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    B, H, S, D = 28, 16, 256, 64           # 28*16*256 rows * 36 bytes: just under the 4 MiB limit
    assert lib.fcs_workspace_bytes(B, H, S, S, D, 0) <= (4 << 20)
    B = 29
    assert lib.fcs_workspace_bytes(B, H, S, S, D, 0) > (4 << 20)
    q = torch.empty(1, dtype=torch.float16, device="cuda")     # never dereferenced: the call is refused first
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = lib.fcs_colsum_batched_static_scratch(
        q.data_ptr(), q.data_ptr(), q.data_ptr(), S, B, H, S, D, 0,
        H * S * D, S * D, D, H * S * D, S * D, D, 0.125, -1, 0,
        status.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -3
    assert "built-in scratch" in _cabi.last_error()
