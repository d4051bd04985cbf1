"""The C-ABI library loads and exports what the header declares; the operator's
host-side validation behaves like the reference's.  No GPU needed."""

import ctypes
import os
import re

import pytest
import torch

import flash_colsum_b200
from flash_colsum_b200 import _cabi, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_every_declared_symbol():
    lib = _cabi.load()
    header = open(os.path.join(ROOT, "include", "flash_colsum_b200.h")).read()
    declared = set(re.findall(r"\b(fcs_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_cabi.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.fcs_version() == _cabi.ABI_VERSION
    assert os.path.samefile(os.path.dirname(build.LIB_PATH), os.path.join(ROOT, "flash_colsum_b200", "_lib"))


def test_workspace_query_is_pure_host_arithmetic():
    lib = _cabi.load()
    # per query row (padded to 256): 4 bytes of -(lse) and 32 bytes of its MMA-ready form;
    # no key split for the batched headline shape
    assert lib.fcs_workspace_bytes(8, 16, 2048, 2048, 64, 0) == 8 * 16 * 2048 * (4 + 32)
    assert lib.fcs_workspace_bytes(32, 16, 1, 577, 64, 0) >= 32 * 16 * 256 * 4   # one padded query block
    assert lib.fcs_workspace_bytes(1, 32, 512, 131072, 128, 1) > 32 * 512 * 36   # key ranges split
    assert lib.fcs_workspace_bytes(1, 1, 1, 1, 100, 0) == 0
    assert lib.fcs_workspace_bytes(1, 1, 8, 8, 96, 0) > 0
    assert lib.fcs_workspace_bytes(0, 1, 1, 1, 64, 0) == 0


def test_argument_errors_come_back_as_codes_not_crashes():
    lib = _cabi.load()
    rc = lib.fcs_colsum_batched(None, None, None, 0, 1, 1, 1, 64, 0, 64, 64, 64, 64, 64, 64,
                                1.0, -1, 0, None, 0, None, None)
    assert rc < 0 and _cabi.last_error()
    rc = lib.fcs_colsum_causal(None, None, None, 1, 1, 1, 100, 0, 104, 104, 104, 104, 1.0, -1, 0,
                               None, 0, None, None)
    assert rc == -2 and "head dimension" in _cabi.last_error()


def test_argument_errors_of_the_added_entry_points():
    """Top-k selection, the passes apart and the batched causal call refuse bad arguments with a
    code and a message before anything is launched."""
    lib = _cabi.load()
    assert lib.fcs_statistics_rows(1) == 256 and lib.fcs_statistics_rows(256) == 256
    assert lib.fcs_statistics_rows(257) == 512 and lib.fcs_statistics_rows(0) == 0
    assert lib.fcs_select_topk(None, 8, 1, 8, 2, None, None, None) == -1
    assert "NULL" in _cabi.last_error()
    buf = (ctypes.c_float * 64)()
    idx = (ctypes.c_int * 64)()
    addr = ctypes.addressof
    assert lib.fcs_select_topk(addr(buf), 8, 1, 8, 9, addr(idx), None, None) == -1      # k > S
    assert "k must be" in _cabi.last_error()
    assert lib.fcs_select_topk(addr(buf), 4, 1, 8, 2, addr(idx), None, None) == -1      # row stride < S
    # statistics of a share: the normalisation cannot count fewer rows than the share has
    assert lib.fcs_colsum_statistics(addr(buf), addr(buf), addr(buf), 1, 1, 300, 300, 64, 0, 64, 64, 64, 64, 64, 64,
                                     1.0, 100, 0, None, 0, None, None) == -1
    assert "norm_rows" in _cabi.last_error()
    assert lib.fcs_colsum_columns(addr(buf), addr(buf), None, addr(buf), 300, 1, 1, 300, 300, 64, 0,
                                  64, 64, 64, 64, 64, 64, 1.0, None, 0, None, None) == -1
    assert "statistics vector" in _cabi.last_error()
    assert lib.fcs_colsum_causal_batched(None, None, None, 0, 2, 1, 1, 1, 100, 0, 104, 104, 104, 104, 104, 104,
                                         1.0, -1, 0, None, 0, None, None) < 0


def test_validation_order_and_messages_without_a_gpu():
    f = flash_colsum_b200.flash_colsum
    with pytest.raises(ValueError, match="4D"):
        f(torch.randn(2, 3, 4), torch.randn(2, 3, 4))
    with pytest.raises(ValueError, match="CUDA"):
        f(torch.randn(1, 8, 128, 64), torch.randn(1, 8, 128, 64))
    # the device check comes before the cls_len checks, as in the reference
    with pytest.raises(ValueError, match="CUDA"):
        f(torch.randn(1, 8, 128, 64), torch.randn(1, 8, 128, 64), cls_len=0)


def test_argument_errors_of_the_pruning_and_self_test_entries():
    """The threshold selection and the wait-expiry self-test refuse bad arguments before any launch;
    the product package does not import the reference install either."""
    lib = _cabi.load()
    buf = (ctypes.c_float * 64)()
    idx = (ctypes.c_int * 64)()
    addr = ctypes.addressof
    assert lib.fcs_select_threshold(None, 8, 1, 8, 0.5, 0, None, None, None) == -1
    assert lib.fcs_select_threshold(addr(buf), 4, 1, 8, 0.5, 0, addr(idx), addr(idx), None) == -1     # ld < S
    assert lib.fcs_select_threshold(addr(buf), 8, 1, 8, float("nan"), 0, addr(idx), addr(idx), None) == -1
    assert "not a number" in _cabi.last_error()
    assert lib.fcs_selftest_wait_expiry(None, None, None, 0, None, 0.05, None) == -1
    assert lib.fcs_selftest_wait_expiry(addr(buf), addr(buf), addr(buf), 0, addr(idx), 3.0, None) == -1
    assert "limit_seconds" in _cabi.last_error()
    assert lib.fcs_selftest_wait_expiry_cluster(None, None, None, None, 0.05, None) == -1
    assert lib.fcs_selftest_wait_expiry_cluster(addr(buf), addr(buf), addr(buf), addr(idx), 0.0, None) == -1
    assert lib.fcs_colsum_causal_accumulate_and_clear(None, None, None, None, 1, 1, 1, 64, 0, 64, 64, 64, 64, 1.0, -1,
                                                      0, None, 0, None, None) < 0
    # flags between GPUs: pointer counts and alignment are checked before any launch
    assert lib.fcs_peer_post(None, 1, 1, None) == -1
    ptrs = (ctypes.c_void_p * 1)(addr(idx) + 2)
    assert lib.fcs_peer_post(ptrs, 1, 1, None) == -1 and "misaligned" in _cabi.last_error()
    assert lib.fcs_peer_post(ptrs, 17, 1, None) == -1
    assert lib.fcs_peer_wait(None, 1, 1, None, None) == -1
    assert lib.fcs_peer_wait(addr(idx), 33, 1, None, None) == -1
    sig = _cabi.PeerSignals()
    sig.post_n = 16
    assert lib.fcs_colsum_causal_accumulate_signalled(None, None, None, None, 1, 1, 1, 64, 0, 64, 64, 64, 64, 1.0, -1,
                                                      0, None, 0, None, None, ctypes.byref(sig)) == -1
    assert "15" in _cabi.last_error()
    sig.post_n = 0
    sig.done_flag = addr(idx)
    assert lib.fcs_colsum_causal_accumulate_signalled(None, None, None, None, 1, 1, 1, 64, 0, 64, 64, 64, 64, 1.0, -1,
                                                      0, None, 0, None, None, ctypes.byref(sig)) == -1
    assert "counter" in _cabi.last_error()
    assert lib.fcs_colsum_causal_accumulate_signalled(None, None, None, None, 1, 1, 1, 64, 0, 64, 64, 64, 64, 1.0, -1,
                                                      0, None, 0, None, None, None) == -1
    pkg = os.path.join(ROOT, "flash_colsum_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith(".py"):
                assert "baseline/_ref" not in open(os.path.join(dirpath, fn)).read(), fn


def test_no_cpu_fallback_in_the_product_package():
    """The package never imports the CPU checkers."""
    pkg = os.path.join(ROOT, "flash_colsum_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "oracle" not in text, os.path.join(dirpath, fn)


def test_kernel_choice_rule_is_host_arithmetic():
    """Which calls take the single-pass cluster kernel: short, well-filled, non-causal, head
    dimension 64, enough (batch, head) pairs; the setter overrides in both directions."""
    from flash_colsum_b200 import _cabi
    try:
        _cabi.set_single_pass(_cabi.SINGLE_PASS_AUTO)
        assert _cabi.single_pass_applies(8, 16, 256)
        assert _cabi.single_pass_applies(8, 16, 512)
        assert _cabi.single_pass_applies(8, 16, 577)           # 75 % of three slices
        assert _cabi.single_pass_applies(8, 16, 1024)
        assert _cabi.single_pass_applies(8, 16, 1536)          # six slices
        assert not _cabi.single_pass_applies(8, 16, 300)       # 59 % of two slices
        assert not _cabi.single_pass_applies(8, 16, 1792)      # seven-CTA clusters: 15 fit, 105 SMs
        assert not _cabi.single_pass_applies(8, 16, 2048)      # eight-CTA clusters lose to two passes ...
        assert _cabi.single_pass_applies(1, 16, 2048)          # ... except on small calls
        assert not _cabi.single_pass_applies(8, 16, 4096)      # does not fit a cluster
        assert _cabi.single_pass_applies(1, 2, 512)            # small calls are cut at tile granularity
        assert not _cabi.single_pass_applies(8, 16, 512, D=128)
        assert not _cabi.single_pass_applies(8, 16, 512, is_causal=True)
        _cabi.set_single_pass(_cabi.SINGLE_PASS_ALWAYS)
        assert _cabi.single_pass_applies(1, 1, 2048) and _cabi.single_pass_applies(8, 16, 577)
        assert not _cabi.single_pass_applies(8, 16, 4096)
        _cabi.set_single_pass(_cabi.SINGLE_PASS_NEVER)
        assert not _cabi.single_pass_applies(8, 16, 512)
        with pytest.raises(ValueError):
            _cabi.set_single_pass(7)
    finally:
        _cabi.set_single_pass(_cabi.SINGLE_PASS_AUTO)
