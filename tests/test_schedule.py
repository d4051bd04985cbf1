"""The tile schedule, mask rules and planning logic of the CUDA kernels, walked
on the CPU by ``schedule_emulator.cpp`` (which includes the kernels' own
header) and compared with the CPU checker."""

import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import c_oracle
from oracle.naive_colsum import parity_errors

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "schedule_emulator.cpp")
HDR = os.path.join(os.path.dirname(HERE), "flash_colsum_b200", "csrc", "schedule.h")
LIB = os.path.join(HERE, "_schedule_emulator.so")


@pytest.fixture(scope="module")
def emu():
    if (not os.path.exists(LIB)
            or os.path.getmtime(LIB) < max(os.path.getmtime(SRC), os.path.getmtime(HDR))):
        subprocess.run(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-o", LIB, SRC], check=True)
    lib = ctypes.CDLL(LIB)
    lib.check_tile_ranges.restype = ctypes.c_int
    lib.check_tile_ranges.argtypes = [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.emulate_colsum.restype = ctypes.c_int
    lib.emulate_colsum.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_int] * 5 + [ctypes.c_float] + \
        [ctypes.c_int] * 5 + [ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p]
    lib.check_fused_short.restype = ctypes.c_int
    lib.check_fused_short.argtypes = [ctypes.c_int] * 7 + [ctypes.c_void_p, ctypes.c_int]
    lib.check_stats_digits.restype = ctypes.c_longlong
    lib.check_stats_digits.argtypes = [ctypes.c_int] * 7
    lib.scratch_need.restype = ctypes.c_longlong
    lib.scratch_need.argtypes = [ctypes.c_int] * 7 + [ctypes.c_void_p]
    return lib


INTERLEAVE_DEFAULT = 300000   # query rows from which the column pass deals its chunks round-robin


def run(emu, q, k, scale=None, causal=False, k_past=-1, cls_len=None, h_norm=0, sms=148,
        interleave_min_rows=INTERLEAVE_DEFAULT):
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    if scale is None:
        scale = 1.0 / D ** 0.5
    out = np.zeros((B, Sk), dtype=np.float32)
    nsplit = ctypes.c_int(0)
    steps = ctypes.c_longlong(0)
    qc, kc = q.contiguous(), k.contiguous()
    rc = emu.emulate_colsum(qc.data_ptr(), kc.data_ptr(), out.ctypes.data, B, H, Sq, Sk, D, scale,
                            int(causal), k_past, -1 if cls_len is None else cls_len, h_norm, sms,
                            interleave_min_rows, ctypes.addressof(nsplit), ctypes.addressof(steps))
    assert rc == 0, f"schedule walk failed with code {rc}"
    return out, nsplit.value, steps.value


CASES = [
    # B, H, Sq, Sk, D, causal, cls, sms
    (2, 3, 128, 128, 16, False, None, 148),
    (2, 2, 100, 100, 16, False, None, 148),
    (1, 2, 577, 577, 8, False, None, 148),
    (3, 2, 300, 300, 8, False, None, 7),        # few CTAs: ranges cut through key tiles
    (2, 2, 300, 300, 8, False, 1, 148),
    (1, 2, 300, 300, 8, False, 200, 5),
    (1, 2, 40, 40, 8, False, 64, 148),          # cls_len beyond the sequence
    (1, 3, 128, 1024, 8, True, None, 148),      # key ranges split (few items)
    (1, 3, 24, 200, 8, True, None, 148),
    (1, 2, 96, 96, 8, True, None, 148),
    (1, 2, 64, 40, 8, True, None, 148),         # keys shorter than queries
    (1, 2, 300, 700, 8, True, None, 148),
    (1, 2, 300, 700, 8, True, None, 3),
    (1, 1, 260, 2000, 4, True, None, 148),
    (1, 2, 129, 129, 8, True, None, 2),
    # one query block and sixteen or more key tiles: contiguous runs of the (b, h, key tile) list
    (1, 3, 128, 2300, 8, True, None, 148),
    (2, 2, 100, 2100, 8, True, None, 5),        # runs cut through heads and batch entries
    (1, 2, 2100, 2100, 4, False, 200, 7),
    (1, 3, 48, 2300, 8, True, None, 148),      # at most 64 queries: half of each tile's columns are padding
    (2, 2, 64, 2177, 8, True, None, 5),
    # two query blocks, both resident
    (1, 3, 400, 2500, 8, True, None, 148),
    (2, 2, 512, 2304, 8, True, None, 5),
    (1, 2, 2100, 2100, 4, False, 300, 7),
    (1, 2, 300, 2200, 4, True, None, 148),     # late key tiles are seen by the second block only
]


@pytest.mark.parametrize("B,H,Sq,Sk,D,causal,cls,sms", CASES)
def test_schedule_reproduces_the_checker(emu, B, H, Sq, Sk, D, causal, cls, sms):
    g = torch.Generator().manual_seed(B * 1000 + Sq + Sk)
    q = torch.randn(B, H, Sq, D, generator=g)
    k = torch.randn(B, H, Sk, D, generator=g) * 1.5
    got, nsplit, steps = run(emu, q, k, causal=causal, cls_len=cls, sms=sms)
    want = c_oracle.colsum_c(q, k, is_causal=causal, cls_len=cls)
    rel, mx = parity_errors(got, want)
    assert rel < 2e-5 and mx < 2e-5, (rel, mx, nsplit, steps)


@pytest.mark.parametrize("B,H,Sq,Sk,D,causal,cls,sms", CASES)
def test_interleaved_column_schedule_reproduces_the_checker(emu, B, H, Sq, Sk, D, causal, cls, sms):
    """The same cases with the column pass dealing (b, h, key tile) chunks round-robin, the
    distribution long inputs get."""
    g = torch.Generator().manual_seed(B * 1000 + Sq + Sk)
    q = torch.randn(B, H, Sq, D, generator=g)
    k = torch.randn(B, H, Sk, D, generator=g) * 1.5
    got, nsplit, steps = run(emu, q, k, causal=causal, cls_len=cls, sms=sms, interleave_min_rows=0)
    want = c_oracle.colsum_c(q, k, is_causal=causal, cls_len=cls)
    rel, mx = parity_errors(got, want)
    assert rel < 2e-5 and mx < 2e-5, (rel, mx, nsplit, steps)


def test_interleaved_schedule_with_many_query_blocks(emu):
    """Few (b, h, key tile) items and many query blocks: the items are cut into parts."""
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, 1, 2100, 4, generator=g)
    k = torch.randn(1, 1, 300, 4, generator=g)
    for causal in (False, True):
        got, _, _ = run(emu, q, k, causal=causal, sms=148, interleave_min_rows=0)
        want = c_oracle.colsum_c(q, k, is_causal=causal)
        assert parity_errors(got, want)[0] < 2e-5


def test_key_range_split_is_used_when_items_are_few(emu):
    q = torch.randn(1, 2, 128, 8)
    k = torch.randn(1, 2, 128 * 40, 8)
    got, nsplit, _ = run(emu, q, k, causal=True)
    assert nsplit > 1
    want = c_oracle.colsum_c(q, k, is_causal=True)
    assert parity_errors(got, want)[0] < 2e-5


def test_explicit_k_past_and_negative_scale_and_head_norm(emu):
    g = torch.Generator().manual_seed(5)
    q = torch.randn(1, 2, 50, 8, generator=g)
    k = torch.randn(1, 2, 400, 8, generator=g)
    # explicit k_past smaller than Sk - Sq: trailing keys are visible to no query
    got, _, _ = run(emu, q, k, causal=True, k_past=100)
    want = c_oracle.colsum_c(q, k[:, :, :150], is_causal=True)
    assert parity_errors(got[:, :150], want)[0] < 2e-5
    assert np.all(got[:, 150:] == 0)
    # negative scale
    got, _, _ = run(emu, q, k[:, :, :50], scale=-0.3)
    want = c_oracle.colsum_c(q, k[:, :, :50], scale=-0.3)
    assert parity_errors(got, want)[0] < 2e-5
    # normalising by a global head count halves the result of a two-head shard
    got4, _, _ = run(emu, q, k[:, :, :50], h_norm=4)
    got2, _, _ = run(emu, q, k[:, :, :50])
    np.testing.assert_allclose(got4 * 2, got2, rtol=1e-5)


@pytest.mark.parametrize("units,NQ,H,clusters,flush_units", [
    (128, 16, 16, 15, 8),      # the headline shape on eight-CTA clusters: shares cut through pairs
    (512, 8, 16, 33, 16),
    (4, 4, 2, 16, 32),         # as many clusters as tiles
    (1, 1, 1, 1, 128),
    (7, 3, 7, 5, 42),
    (2048, 2, 16, 74, 64),
    (128, 4, 64, 148, 32),     # many heads: intermediate flushes inside a batch entry
    (6, 5, 3, 30, 25),
])
def test_single_pass_work_split_covers_every_tile_once(emu, units, NQ, H, clusters, flush_units):
    assert emu.check_tile_ranges(units, NQ, H, clusters, flush_units) == 0


def test_scratch_queries_cover_every_k_past(emu):
    """Walk (B, H, Sq, Sk, k_past) on the host: the library's upper bound is never below what the
    plan of any k_past lays out, and the per-call query returns exactly that layout (shapes that
    take a kernel without scratch are asked with more than four query rows and 128 head dims, so
    that the streaming passes are what runs).  An explicit k_past shows the first query tile
    more keys than the inferred one, which can split its key range further."""
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    sms = _cabi.plan_info(1, 1, 128, 128, False)["sms"]
    need = ctypes.c_size_t(0)
    _cabi.set_short_fused(_cabi.SHORT_FUSED_NEVER)   # (at most 128 rows would take the one-kernel form)
    try:
        _walk_scratch(emu, lib, sms, need)
    finally:
        _cabi.set_short_fused(_cabi.SHORT_FUSED_AUTO)


def _walk_scratch(emu, lib, sms, need):
    walked = shortfalls = grew = 0
    for B in (1, 2, 5):
        for H in (1, 3, 8, 32):
            for Sq in (5, 100, 128, 300, 512, 1024, 1500):
                for Sk in (40, 400, 1024, 4096, 20000):
                    bound = lib.fcs_workspace_bytes(B, H, Sq, Sk, 128, 1)
                    inferred = emu.scratch_need(B, H, Sq, Sk, 1, -1, sms, None)
                    for k_past in (0, 1, 100, 255, 300, 1000, Sk - 1, Sk, Sk + 77, 3 * Sk, max(0, Sk - Sq)):
                        truth = emu.scratch_need(B, H, Sq, Sk, 1, k_past, sms, None)
                        walked += 1
                        grew += truth > inferred
                        shortfalls += truth > bound
                        assert lib.fcs_call_workspace_bytes(B, H, Sq, Sk, 128, 1, k_past, ctypes.byref(need)) == 0
                        assert need.value == truth, (B, H, Sq, Sk, k_past)
                    assert lib.fcs_call_workspace_bytes(B, H, Sq, Sk, 128, 1, -1, ctypes.byref(need)) == 0
                    assert need.value == inferred
                    # non-causal: one layout
                    assert lib.fcs_workspace_bytes(B, H, Sq, Sk, 128, 0) == emu.scratch_need(B, H, Sq, Sk, 0, 0, sms, None)
    assert shortfalls == 0, f"{shortfalls} of {walked} combinations need more scratch than the bound"
    assert grew > 0          # the walk does reach plans that an inferred k_past would have undersized
    # the combination that first showed the gap: one more key range at k_past = 300
    n_inf, n_exp = ctypes.c_int(0), ctypes.c_int(0)
    a = emu.scratch_need(1, 1, 300, 400, 1, -1, sms, ctypes.addressof(n_inf))
    b = emu.scratch_need(1, 1, 300, 400, 1, 300, sms, ctypes.addressof(n_exp))
    assert (n_inf.value, n_exp.value) == (1, 2) and b > a
    assert lib.fcs_workspace_bytes(1, 1, 300, 400, 128, 1) >= b


def test_calls_that_take_a_kernel_without_scratch_ask_for_none():
    from flash_colsum_b200 import _cabi
    lib = _cabi.load()
    need = ctypes.c_size_t(7)
    # CLS prefix of the CLIP-style shape: the few-row kernel
    assert lib.fcs_call_workspace_bytes(32, 16, 1, 577, 64, 0, 0, ctypes.byref(need)) == 0 and need.value == 0
    # four decode queries over a long key axis, causal
    assert lib.fcs_call_workspace_bytes(1, 32, 4, 8192, 128, 1, -1, ctypes.byref(need)) == 0 and need.value == 0
    # five rows over the same keys, and the causal suffix of 128 queries over 4096 keys: the one-kernel form
    assert lib.fcs_call_workspace_bytes(1, 32, 5, 8192, 128, 1, -1, ctypes.byref(need)) == 0 and need.value == 0
    assert lib.fcs_call_workspace_bytes(1, 32, 128, 4096, 128, 1, -1, ctypes.byref(need)) == 0 and need.value == 0
    assert _cabi.short_fused_applies(1, 32, 128, 4096) == (4, 4)
    # ... unless it is switched off, or the call is large: the streaming passes
    _cabi.set_short_fused(_cabi.SHORT_FUSED_NEVER)
    try:
        assert lib.fcs_call_workspace_bytes(1, 32, 128, 4096, 128, 1, -1, ctypes.byref(need)) == 0 and need.value > 0
        assert _cabi.short_fused_applies(1, 32, 128, 4096) is None
    finally:
        _cabi.set_short_fused(_cabi.SHORT_FUSED_AUTO)
    assert _cabi.short_fused_applies(1, 32, 128, 65536) == (4, 64)       # still one wave over most SMs
    assert lib.fcs_call_workspace_bytes(1, 32, 128, 131072, 128, 1, -1, ctypes.byref(need)) == 0 and need.value > 0
    assert _cabi.short_fused_applies(1, 16, 128, 65536) is None           # too few CTAs for a call this long
    assert _cabi.short_fused_applies(64, 12, 16, 197, is_causal=False, D=64) is None   # six waves of tiny CTAs
    assert lib.fcs_call_workspace_bytes(1, 32, 300, 8192, 128, 1, -1, ctypes.byref(need)) == 0 and need.value > 0
    # sizes no call accepts
    assert lib.fcs_call_workspace_bytes(1, 1, 1, 1, 100, 0, 0, ctypes.byref(need)) == -2
    assert lib.fcs_call_workspace_bytes(0, 1, 1, 1, 64, 0, 0, ctypes.byref(need)) == -1
    assert lib.fcs_call_workspace_bytes(1, 1, 1, 1, 64, 0, 0, None) == -1


# clusters of 1..8 CTAs that run at once, as a B200 answers for the one-kernel form (index = size)
B200_CLUSTERS = (ctypes.c_int * 9)(0, 148, 74, 48, 32, 28, 24, 16, 15)


@pytest.mark.parametrize("B,H,Sq,Sk,causal,k_past,expect", [
    (1, 32, 128, 4096, 1, -1, 4004),       # the reference's causal test shape: 32 clusters of four, four blocks each
    (1, 8, 128, 4096, 1, -1, 8002),
    (1, 16, 128, 4096, 1, -1, 6003),       # sixteen clusters of eight do not run at once: seven would, six are enough
    (1, 2, 7, 7, 0, 0, 1001),
    (2, 4, 64, 300, 1, -1, 2001),
    (1, 5, 128, 100, 1, -1, 1001),         # fewer keys than queries
    (1, 6, 33, 2049, 1, -1, 5002),         # nine blocks over five CTAs
    (1, 4, 100, 2000, 1, 0, 1001),         # K_past 0: the first 100 keys are all that is seen
    (1, 4, 100, 2000, 1, 700, 4001),
    (1, 4, 100, 2000, 1, 5000, 8001),
    (3, 70, 20, 600, 1, -1, 1003),         # more pairs than SMs: one CTA each
    (1, 32, 128, 65536, 1, -1, 4064),
    (1, 32, 128, 131072, 1, -1, 0),        # too long
    (1, 16, 128, 65536, 1, -1, 0),         # long and too few CTAs
    (64, 12, 16, 197, 0, 0, 0),            # six waves of one-block CTAs: the ramp is paid six times
    (1, 8, 128, 32768, 1, -1, 0),          # 64 CTAs of 16 blocks: the idle SMs cost more than the launches
    (1, 4, 128, 131072, 1, -1, 0),         # four heads of a head-sharded long context: 32 CTAs
    (1, 50, 128, 4096, 1, -1, 2008),
    (16, 16, 128, 1024, 1, -1, 1004),      # 256 pairs in two waves
    (1, 4, 129, 1000, 1, -1, 0),           # two query tiles
])
def test_one_kernel_form_plan_and_masks(emu, B, H, Sq, Sk, causal, k_past, expect):
    assert emu.check_fused_short(B, H, Sq, Sk, causal, k_past, 148, B200_CLUSTERS, 0) == expect


def test_one_kernel_form_masks_on_a_walk_of_sizes(emu):
    """Forced onto every size of a walk (ragged rows and keys, every K_past regime): both phases see
    each visible (query, key) pair exactly once."""
    walked = 0
    for Sq in (1, 5, 31, 64, 100, 127, 128):
        for Sk in (1, 40, 255, 256, 257, 600, 1024, 1500):
            for k_past in (-1, 0, 3, 200, 255, 256, 700, Sk - 1, Sk, 3 * Sk):
                rc = emu.check_fused_short(1, 3, Sq, Sk, 1, k_past, 148, B200_CLUSTERS, 1)
                assert rc > 0, (Sq, Sk, k_past, rc)
                walked += 1
            assert emu.check_fused_short(2, 2, Sq, Sk, 0, 0, 148, B200_CLUSTERS, 1) > 0
    assert walked == 7 * 8 * 10


@pytest.mark.parametrize("B,H,Sq,Sk,causal,k_past,sms", [
    (8, 16, 2048, 2048, 0, 0, 148),        # the headline shape: 2048 items, no key split
    (1, 32, 512, 131072, 1, -1, 148),      # long context: key ranges split
    (3, 5, 383, 383, 0, 0, 148),
    (1, 2, 700, 5000, 1, 100, 148),
    (2, 7, 130, 900, 1, -1, 7),            # a grid that is no multiple of anything
    (5, 3, 1000, 1000, 0, 0, 100),
    (1, 1, 1, 1, 0, 0, 148),
])
def test_statistics_items_advance_by_digits(emu, B, H, Sq, Sk, causal, k_past, sms):
    """Going from one item of a CTA to its next by adding the grid's digits gives the same items as
    decoding every index afresh, for every CTA, and covers every item once."""
    assert emu.check_stats_digits(B, H, Sq, Sk, causal, k_past, sms) > 0
