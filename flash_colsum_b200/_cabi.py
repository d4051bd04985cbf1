"""ctypes binding of the C ABI declared in ``include/flash_colsum_b200.h``."""

from __future__ import annotations

import ctypes
import os
import warnings
from typing import Optional

from . import build as _build

# every symbol the header declares
EXPORTED_SYMBOLS = (
    "fcs_version", "fcs_last_error", "fcs_workspace_bytes", "fcs_call_workspace_bytes",
    "fcs_colsum_batched", "fcs_colsum_non_batched", "fcs_colsum_causal",
    "fcs_set_profiling", "fcs_last_pass_ms", "fcs_plan_info",
    "fcs_colsum_batched_static_scratch", "fcs_colsum_causal_accumulate", "fcs_colsum_causal_accumulate_and_clear",
    "fcs_set_single_pass", "fcs_single_pass_info", "fcs_single_pass_applies",
    "fcs_set_short_fused", "fcs_short_fused_applies",
    "fcs_colsum_causal_batched", "fcs_select_topk", "fcs_select_threshold",
    "fcs_statistics_rows", "fcs_colsum_statistics", "fcs_colsum_columns", "fcs_selftest_wait_expiry",
    "fcs_selftest_wait_expiry_cluster",
    "fcs_peer_post", "fcs_peer_wait", "fcs_colsum_causal_accumulate_signalled",
)

ABI_VERSION = 202   # fcs_version() of the library these argument lists were written for
FCS_OK = 0
FCS_ERR_UNSUPPORTED = -2
FCS_DTYPE_FP16 = 0
FCS_DTYPE_BF16 = 1

_lib: Optional[ctypes.CDLL] = None

_i, _i64, _f, _p, _sz = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t


class PeerSignals(ctypes.Structure):
    """`FcsPeerSignals` of the header."""
    _fields_ = [("wait_flag", _p), ("wait_value", _i), ("post", _p * 15), ("post_n", _i), ("post_value", _i),
                ("counter", _p), ("done_flag", _p), ("done_value", _i)]


class LibraryMissing(RuntimeError):
    """The CUDA library is not built; there is no other implementation to fall back to."""


def load() -> ctypes.CDLL:
    """Load the library, building it when sources are newer and nvcc is present.

    Fails loudly if the library can neither be found nor built.
    """
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("FLASH_COLSUM_B200_LIB")   # an explicit build to load instead
    if path:
        if not os.path.exists(path):
            raise LibraryMissing(f"FLASH_COLSUM_B200_LIB={path} does not exist")
    elif not _build.is_stale():
        path = _build.LIB_PATH
    else:
        path = _build.LIB_PATH
        try:
            path = _build.build()
        except Exception as exc:  # no nvcc on this machine
            if not os.path.exists(path):
                raise LibraryMissing(
                    f"{path} is missing and could not be built ({exc}); "
                    "run `python -m flash_colsum_b200.build` where nvcc is available") from exc
            # an older build is all there is: it is used only if it speaks this binding's ABI (below)
            warnings.warn(f"flash_colsum_b200: {path} is older than its sources and could not be rebuilt ({exc})")
    lib = ctypes.CDLL(path)
    lib.fcs_version.restype = _i
    lib.fcs_version.argtypes = []
    if lib.fcs_version() != ABI_VERSION:
        raise LibraryMissing(f"{path} reports version {lib.fcs_version()}, this binding needs {ABI_VERSION}; "
                             "rebuild it with `python -m flash_colsum_b200.build --force`")
    lib.fcs_last_error.restype = ctypes.c_char_p
    lib.fcs_last_error.argtypes = []
    lib.fcs_workspace_bytes.restype = _sz
    lib.fcs_workspace_bytes.argtypes = [_i] * 6
    lib.fcs_call_workspace_bytes.restype = _i
    lib.fcs_call_workspace_bytes.argtypes = [_i] * 7 + [ctypes.POINTER(_sz)]
    lib.fcs_colsum_batched.restype = _i
    lib.fcs_colsum_batched.argtypes = [_p, _p, _p, _i64, _i, _i, _i, _i, _i] + [_i64] * 6 + \
        [_f, _i, _i, _p, _sz, _p, _p]
    lib.fcs_colsum_non_batched.restype = _i
    lib.fcs_colsum_non_batched.argtypes = [_p, _p, _p, _i, _i, _i, _i] + [_i64] * 4 + \
        [_f, _i, _i, _p, _sz, _p, _p]
    lib.fcs_colsum_causal.restype = _i
    lib.fcs_colsum_causal.argtypes = [_p, _p, _p, _i, _i, _i, _i, _i] + [_i64] * 4 + \
        [_f, _i, _i, _p, _sz, _p, _p]
    lib.fcs_colsum_causal_batched.restype = _i
    lib.fcs_colsum_causal_batched.argtypes = [_p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64,
                                              _i64, _f, _i, _i, _p, _sz, _p, _p]
    lib.fcs_statistics_rows.restype = _sz
    lib.fcs_statistics_rows.argtypes = [_i]
    lib.fcs_colsum_statistics.restype = _i
    lib.fcs_colsum_statistics.argtypes = [_p, _p, _p, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64, _i64,
                                          _f, _i64, _i, _p, _sz, _p, _p]
    lib.fcs_colsum_columns.restype = _i
    lib.fcs_colsum_columns.argtypes = [_p, _p, _p, _p, _i64, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _i64, _i64,
                                       _i64, _f, _p, _sz, _p, _p]
    lib.fcs_select_topk.restype = _i
    lib.fcs_select_topk.argtypes = [_p, _i64, _i, _i, _i, _p, _p, _p]
    lib.fcs_colsum_causal_accumulate_signalled.restype = _i
    lib.fcs_colsum_causal_accumulate_signalled.argtypes = [_p, _p, _p, _p, _i, _i, _i, _i, _i] + [_i64] * 4 + \
        [_f, _i, _i, _p, _sz, _p, _p, ctypes.POINTER(PeerSignals)]
    lib.fcs_peer_post.restype = _i
    lib.fcs_peer_post.argtypes = [ctypes.POINTER(_p), _i, _i, _p]
    lib.fcs_peer_wait.restype = _i
    lib.fcs_peer_wait.argtypes = [_p, _i, _i, _p, _p]
    lib.fcs_selftest_wait_expiry.restype = _i
    lib.fcs_selftest_wait_expiry.argtypes = [_p, _p, _p, _sz, _p, ctypes.c_double, _p]
    lib.fcs_selftest_wait_expiry_cluster.restype = _i
    lib.fcs_selftest_wait_expiry_cluster.argtypes = [_p, _p, _p, _p, ctypes.c_double, _p]
    lib.fcs_select_threshold.restype = _i
    lib.fcs_select_threshold.argtypes = [_p, _i64, _i, _i, _f, _i, _p, _p, _p]
    lib.fcs_colsum_causal_accumulate.restype = _i
    lib.fcs_colsum_causal_accumulate.argtypes = lib.fcs_colsum_causal.argtypes
    lib.fcs_colsum_causal_accumulate_and_clear.restype = _i
    lib.fcs_colsum_causal_accumulate_and_clear.argtypes = [_p, _p, _p, _p, _i, _i, _i, _i, _i] + [_i64] * 4 + \
        [_f, _i, _i, _p, _sz, _p, _p]
    lib.fcs_colsum_batched_static_scratch.restype = _i
    lib.fcs_colsum_batched_static_scratch.argtypes = [_p, _p, _p, _i64, _i, _i, _i, _i, _i] + [_i64] * 6 + \
        [_f, _i, _i, _p, _p]
    lib.fcs_set_profiling.restype = _i
    lib.fcs_set_profiling.argtypes = [_i]
    lib.fcs_set_single_pass.restype = _i
    lib.fcs_set_single_pass.argtypes = [_i]
    lib.fcs_single_pass_applies.restype = _i
    lib.fcs_single_pass_applies.argtypes = [_i, _i, _i, _i, _i, _i]
    lib.fcs_single_pass_info.restype = _i
    lib.fcs_single_pass_info.argtypes = [_i, ctypes.POINTER(_i), ctypes.POINTER(_i)]
    lib.fcs_set_short_fused.restype = _i
    lib.fcs_set_short_fused.argtypes = [_i]
    lib.fcs_short_fused_applies.restype = _i
    lib.fcs_short_fused_applies.argtypes = [_i, _i, _i, _i, _i, _i, _i, ctypes.POINTER(_i), ctypes.POINTER(_i)]
    lib.fcs_last_pass_ms.restype = _i
    lib.fcs_last_pass_ms.argtypes = [_p, _p, _p]
    lib.fcs_plan_info.restype = _i
    lib.fcs_plan_info.argtypes = [_i] * 5 + [_p] * 4
    _lib = lib
    return lib


def last_error() -> str:
    return load().fcs_last_error().decode("utf-8", "replace")


def set_profiling(enabled: bool) -> None:
    load().fcs_set_profiling(int(bool(enabled)))


def single_pass_applies(B: int, H: int, sk: int, D: int = 64, is_causal: bool = False,
                        sq_rows: Optional[int] = None) -> bool:
    """Whether a call with these sizes takes the single-pass kernel under the current mode
    (``sq_rows``: query rows that enter the mean, default ``sk``)."""
    return bool(load().fcs_single_pass_applies(B, H, sk if sq_rows is None else sq_rows, sk, D, int(is_causal)))


def single_pass_info(sk: int):
    """(CTAs per cluster, clusters resident at once) of the single-pass kernel for `sk` keys."""
    cl, n = _i(0), _i(0)
    if load().fcs_single_pass_info(int(sk), ctypes.byref(cl), ctypes.byref(n)) != FCS_OK:
        raise ValueError(f"the single-pass kernel does not cover {sk} keys")
    return cl.value, n.value


SINGLE_PASS_AUTO, SINGLE_PASS_NEVER, SINGLE_PASS_ALWAYS = 0, 1, 2


def set_single_pass(mode: int) -> None:
    """Kernel choice for short non-causal calls (`fcs_set_single_pass`)."""
    if load().fcs_set_single_pass(int(mode)) != FCS_OK:
        raise ValueError(f"single-pass mode must be 0, 1 or 2, got {mode}")
    _call_workspace.clear()   # the scratch a call uses follows the kernel it takes


SHORT_FUSED_AUTO, SHORT_FUSED_NEVER, SHORT_FUSED_ALWAYS = 0, 1, 2


def set_short_fused(mode: int) -> None:
    """Kernel choice for short query axes over short key axes (`fcs_set_short_fused`)."""
    if load().fcs_set_short_fused(int(mode)) != FCS_OK:
        raise ValueError(f"short-fused mode must be 0, 1 or 2, got {mode}")
    _call_workspace.clear()   # the scratch a call uses follows the kernel it takes


def short_fused_applies(B: int, H: int, sq_rows: int, sk: int, is_causal: bool = True, k_past: int = -1,
                        D: int = 128):
    """(cluster size, key blocks per CTA) when a call with these sizes takes the one-kernel form for
    short query axes under the current mode, else None.  Calls with at most four query rows are decided
    before this; so are calls that the single-pass kernel takes, unless this form runs them in one wave."""
    cl, bpc = _i(0), _i(0)
    if not load().fcs_short_fused_applies(B, H, sq_rows, sk, D, int(is_causal), int(k_past), ctypes.byref(cl),
                                          ctypes.byref(bpc)):
        return None
    return cl.value, bpc.value


_call_workspace: dict = {}   # (sizes, k_past) -> fcs_call_workspace_bytes; host arithmetic, cached per shape


def call_workspace_bytes(B: int, H: int, sq_rows: int, Sk: int, D: int, is_causal: bool, k_past: int = -1) -> int:
    """Scratch bytes the call with exactly these arguments uses (0: none, pass no workspace)."""
    key = (B, H, sq_rows, Sk, D, bool(is_causal), k_past)
    n = _call_workspace.get(key)
    if n is None:
        out = _sz(0)
        if load().fcs_call_workspace_bytes(B, H, sq_rows, Sk, D, int(is_causal), int(k_past),
                                           ctypes.byref(out)) != FCS_OK:
            raise RuntimeError(f"flash_colsum_b200: {last_error()}")
        n = int(out.value)
        if len(_call_workspace) < 4096:
            _call_workspace[key] = n
    return n


def last_pass_ms():
    """(statistics, merge, column) pass durations in ms of the last profiled call."""
    vals = [ctypes.c_float(0.0) for _ in range(3)]
    rc = load().fcs_last_pass_ms(*[ctypes.addressof(v) for v in vals])
    if rc != FCS_OK:
        raise RuntimeError(last_error())
    return tuple(float(v.value) for v in vals)


def plan_info(B: int, H: int, sq_rows: int, Sk: int, is_causal: bool) -> dict:
    nsplit, sms = ctypes.c_int(0), ctypes.c_int(0)
    items, steps = ctypes.c_longlong(0), ctypes.c_longlong(0)
    rc = load().fcs_plan_info(B, H, sq_rows, Sk, int(is_causal), ctypes.addressof(nsplit),
                              ctypes.addressof(items), ctypes.addressof(steps), ctypes.addressof(sms))
    if rc != FCS_OK:
        raise RuntimeError("fcs_plan_info rejected the sizes")
    return {"nsplit": nsplit.value, "stats_items": items.value, "colsum_steps": steps.value,
            "sms": sms.value}
