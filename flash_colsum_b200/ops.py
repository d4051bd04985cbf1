"""The operator: column means of softmax attention without forming the matrix.

Same call as the reference's ``flash_colsum`` (flash_colsum/ops.py:13-105): same
arguments, same validation order and messages, same three-way dispatch (causal /
single-sample / batched) -- each branch calls one C-ABI entry point of the CUDA
library instead of a Triton launcher.  There is no CPU path and no fallback: if
the library is missing the call raises.
"""

from __future__ import annotations

import contextlib
import ctypes
from typing import Dict, Optional, Tuple

import torch

from . import _cabi

_DTYPE_CODE = {torch.float16: _cabi.FCS_DTYPE_FP16, torch.bfloat16: _cabi.FCS_DTYPE_BF16}

# one sticky device-status word per device, zeroed once
_status: Dict[int, torch.Tensor] = {}


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


def device_status(device=None) -> int:
    """Synchronise and return the device status word (0 = no kernel gave up a wait)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_status_word(dev).item())


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """Unit inner stride, outer strides multiples of 16 bytes, 16-byte aligned base."""
    s0, s1, s2, s3 = t.stride()
    if s3 == 1 and s0 > 0 and s1 > 0 and s2 > 0 and (s0 | s1 | s2) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous()


# The wrappers below run for every call, and calls of a dozen microseconds of GPU work are
# bound by them: the device guard is skipped when the tensors' device is the current one, and
# the stream handle comes from the raw getter instead of a Stream object.
_NO_GUARD = contextlib.nullcontext()
_raw_stream_getter = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _on_device(device: torch.device):
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)


def _raw_stream(device: torch.device) -> int:
    """cudaStream_t of torch's current stream on `device`, as an integer."""
    if _raw_stream_getter is not None:
        idx = device.index
        return _raw_stream_getter(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


def _rows(cls_n: int, S: int) -> int:
    return S if cls_n == -1 else min(cls_n, S)


def _check(rc: int) -> None:
    if rc != _cabi.FCS_OK:
        raise RuntimeError(f"flash_colsum_b200: {_cabi.last_error()} (code {rc})")


def _round_fp32(query: torch.Tensor, key: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 inputs are rounded to 16 bits before the tensor cores see them: to fp16, whose ten
    mantissa bits are those of the TF32 format the reference's ``tl.dot`` gives fp32 operands
    (kernel_noncausal_batched.py:37,54), or to bf16 when a value lies outside fp16's range.
    The range check reads one number back from the device (the call synchronises)."""
    limit = 60000.0
    big = max(float(query.abs().max()), float(key.abs().max())) if query.numel() and key.numel() else 0.0
    dt = torch.float16 if big < limit else torch.bfloat16
    return query.to(dt), key.to(dt)


def _prepare(query: torch.Tensor, key: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
    if key.dtype != query.dtype:
        raise ValueError(f"query and key must have the same dtype, got {query.dtype} and {key.dtype}")
    if key.device != query.device:
        raise ValueError(f"query and key must be on the same device, got {query.device} and {key.device}")
    if query.dtype == torch.float32:
        query, key = _round_fp32(query, key)
    if query.dtype not in _DTYPE_CODE:
        raise ValueError(f"flash_colsum supports float16, bfloat16 and float32 inputs, got {query.dtype}")
    if query.shape[3] % 8 or not 8 <= query.shape[3] <= 128:
        raise ValueError(f"head_dim must be a multiple of 8 from 8 to 128, got {query.shape[3]}")
    return _tma_ready(query), _tma_ready(key), _DTYPE_CODE[query.dtype]


class _NoWorkspace:
    """Stands in for the scratch tensor of a call that uses none."""

    @staticmethod
    def data_ptr() -> int:
        return 0

    @staticmethod
    def numel() -> int:
        return 0


_NO_WORKSPACE = _NoWorkspace()


def _workspace(lib, device, B, H, rows, Sk, D, causal, k_past: int = -1):
    """Scratch for exactly this call: nothing is allocated when the call takes the few-row or
    the single-pass kernel, and a causal call is sized for the ``k_past`` it passes."""
    n = _cabi.call_workspace_bytes(B, H, rows, Sk, D, causal, k_past)
    if n == 0:
        return _NO_WORKSPACE
    return torch.empty(n, dtype=torch.uint8, device=device)


def _workspace_two_pass(lib, device, B, H, rows, Sk, D) -> torch.Tensor:
    """Scratch for an entry point that always runs a streaming pass (the passes run apart)."""
    n = lib.fcs_workspace_bytes(B, H, rows, Sk, D, 0)
    if n == 0:
        raise RuntimeError("flash_colsum_b200: fcs_workspace_bytes rejected the sizes")
    return torch.empty(n, dtype=torch.uint8, device=device)


def _flash_colsum_batched(Q: torch.Tensor, K: torch.Tensor, scale: float, CLS_N: int = -1,
                          h_norm: int = 0) -> torch.Tensor:
    """(B, S) fp32.  Counterpart of kernel_noncausal_batched.py:102."""
    lib = _cabi.load()
    Q, K, code = _prepare(Q, K)
    B, H, S, D = Q.shape
    with _on_device(Q.device):
        out = torch.empty((B, S), device=Q.device, dtype=torch.float32)
        ws = _workspace(lib, Q.device, B, H, _rows(CLS_N, S), S, D, False)
        _check(lib.fcs_colsum_batched(
            Q.data_ptr(), K.data_ptr(), out.data_ptr(), S, B, H, S, D, code,
            Q.stride(0), Q.stride(1), Q.stride(2), K.stride(0), K.stride(1), K.stride(2),
            float(scale), int(CLS_N), int(h_norm), ws.data_ptr(), ws.numel(),
            _status_word(Q.device).data_ptr(), _raw_stream(Q.device)))
    return out


def _flash_colsum_non_batched(Q: torch.Tensor, K: torch.Tensor, scale: float, CLS_N: int = -1,
                              h_norm: int = 0) -> torch.Tensor:
    """(1, S) fp32.  Counterpart of kernel_noncausal.py:95."""
    lib = _cabi.load()
    Q, K, code = _prepare(Q, K)
    _, H, S, D = Q.shape
    with _on_device(Q.device):
        out = torch.empty((1, S), device=Q.device, dtype=torch.float32)
        ws = _workspace(lib, Q.device, 1, H, _rows(CLS_N, S), S, D, False)
        _check(lib.fcs_colsum_non_batched(
            Q.data_ptr(), K.data_ptr(), out.data_ptr(), H, S, D, code,
            Q.stride(1), Q.stride(2), K.stride(1), K.stride(2),
            float(scale), int(CLS_N), int(h_norm), ws.data_ptr(), ws.numel(),
            _status_word(Q.device).data_ptr(), _raw_stream(Q.device)))
    return out


def _flash_colsum_causal(Q: torch.Tensor, K: torch.Tensor, scale: float, K_past: Optional[int] = None,
                         h_norm: int = 0, accumulate_into: Optional[torch.Tensor] = None,
                         clear_next: Optional[torch.Tensor] = None, signals=None) -> Optional[torch.Tensor]:
    """(1, K_len) fp32.  Counterpart of kernel_causal.py:94.

    With ``accumulate_into`` (fp32, contiguous, K_len elements, already cleared by
    the caller; may be a peer-mapped tensor of another GPU) the result is added
    into that tensor instead of a fresh one; ``clear_next`` (same form, local memory)
    is zeroed by the same kernels, for a target that alternates between two buffers;
    ``signals`` (a ``_cabi.PeerSignals``) makes the column pass order itself against the
    other GPUs -- the call then returns None, having launched nothing, when its shape takes
    a kernel that cannot do so (at most four query rows).
    """
    lib = _cabi.load()
    Q, K, code = _prepare(Q, K)
    _, H, Q_len, D = Q.shape
    K_len = K.shape[2]
    with _on_device(Q.device):
        head, tail = (), ()
        if accumulate_into is None:
            out = torch.empty((1, K_len), device=Q.device, dtype=torch.float32)
            entry = lib.fcs_colsum_causal
        else:
            out = accumulate_into
            for t in (out,) if clear_next is None else (out, clear_next):
                if t.dtype != torch.float32 or t.numel() != K_len or not t.is_contiguous():
                    raise ValueError("accumulate_into / clear_next must be contiguous fp32 tensors with K_len elements")
            entry = lib.fcs_colsum_causal_accumulate
            if signals is not None:
                entry = lib.fcs_colsum_causal_accumulate_signalled
                head = (0 if clear_next is None else clear_next.data_ptr(),)
                tail = (ctypes.byref(signals),)
            elif clear_next is not None:
                entry = lib.fcs_colsum_causal_accumulate_and_clear
                head = (clear_next.data_ptr(),)
        ws = _workspace(lib, Q.device, 1, H, Q_len, K_len, D, True, -1 if K_past is None else int(K_past))
        rc = entry(
            Q.data_ptr(), K.data_ptr(), out.data_ptr(), *head, H, Q_len, K_len, D, code,
            Q.stride(1), Q.stride(2), K.stride(1), K.stride(2),
            float(scale), -1 if K_past is None else int(K_past), int(h_norm),
            ws.data_ptr(), ws.numel(),
            _status_word(Q.device).data_ptr(), _raw_stream(Q.device), *tail)
        if signals is not None and rc == _cabi.FCS_ERR_UNSUPPORTED:
            return None
        _check(rc)
    return out


def _without_work(query: torch.Tensor, key: torch.Tensor) -> Optional[torch.Tensor]:
    """The result for inputs with an empty axis, which launch nothing: what ``naive_colsum`` of the
    reference returns for them (baselines.py:35-78) -- an empty (B, S_k) tensor when there is no
    batch entry or no key, and NaN (a mean over no rows) when there are keys but no query rows or heads."""
    B, H, S_q, _ = query.shape
    S_k = key.shape[2]
    if B == 0 or S_k == 0:
        return torch.empty((B, S_k), device=query.device, dtype=torch.float32)
    if S_q == 0 or H == 0:
        return torch.full((B, S_k), float("nan"), device=query.device, dtype=torch.float32)
    return None


def flash_colsum(
    query: torch.Tensor,
    key: torch.Tensor,
    scale: Optional[float] = None,
    is_causal: bool = False,
    cls_len: Optional[int] = None,
    *,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Column means of the attention matrix.

    Args:
        query: (B, H, S, D) for non-causal or (1, H, Q_len, D) for causal; fp16 or bf16
            (fp32 is accepted and rounded to fp16, or to bf16 when out of fp16's range);
            D a multiple of 8 up to 128.
        key: same shape as query (non-causal) or (1, H, K_len, D) (causal).
        scale: score scale, default 1/sqrt(D).
        is_causal: queries are aligned to the end of the keys and key j is visible
            to query i iff j <= max(0, K_len - Q_len) + i.
        cls_len: non-causal only; average over the first ``min(cls_len, S)`` query
            rows instead of all of them.
        out_dtype: dtype of the result.  Default fp32, the precision the kernels
            accumulate in (column means of long sequences are fp16 subnormals);
            pass ``torch.float16`` for the dtype the reference's kernels return.

    Returns:
        (B, S) for non-causal, (1, K_len) for causal.

    Raises:
        ValueError: invalid shapes/arguments, with the reference's messages
        (flash_colsum/ops.py:59-97).
    """
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError(f"Expected 4D tensors, got query.ndim={query.ndim}, key.ndim={key.ndim}")

    if query.device.type != 'cuda':
        raise ValueError(f"Flash attention only supports CUDA tensors, got {query.device}")

    if cls_len is not None and is_causal:
        raise ValueError("cls_len is only supported for non-causal attention")
    if cls_len is not None and cls_len <= 0:
        raise ValueError(f"cls_len must be positive, got {cls_len}")

    B_q, H_q, S_q, D_q = query.shape
    B_k, H_k, S_k, D_k = key.shape

    if scale is None:
        scale = 1.0 / (D_q ** 0.5)

    if is_causal:
        if B_q != 1 or B_k != 1:
            raise ValueError(
                f"Causal attention currently only supports batch size 1, got B_q={B_q}, B_k={B_k}")
        if H_q != H_k or D_q != D_k:
            raise ValueError(
                f"Query and key must have same heads and head_dim, got "
                f"H_q={H_q}, H_k={H_k}, D_q={D_q}, D_k={D_k}")
        out = _without_work(query, key)
        if out is None:
            out = _flash_colsum_causal(query, key, scale)
    else:
        if B_q != B_k or H_q != H_k or S_q != S_k or D_q != D_k:
            raise ValueError(
                f"For non-causal attention, query and key must have same shape, got "
                f"query: {query.shape}, key: {key.shape}")
        cls_n = -1 if cls_len is None else int(cls_len)
        out = _without_work(query, key)
        if out is not None:
            pass
        elif B_q == 1:
            out = _flash_colsum_non_batched(query, key, scale, CLS_N=cls_n)
        else:
            out = _flash_colsum_batched(query, key, scale, CLS_N=cls_n)

    if out_dtype is not None and out_dtype != out.dtype:
        out = out.to(out_dtype)
    return out


def flash_colsum_causal(
    query: torch.Tensor,
    key: torch.Tensor,
    scale: Optional[float] = None,
    *,
    k_past: Optional[int] = None,
    out_dtype: Optional[torch.dtype] = None,
) -> torch.Tensor:
    """Causal column means for any batch size, with the launcher's ``K_past`` exposed.

    What the reference defines but does not offer through ``flash_colsum``: its
    operator refuses ``B > 1`` (flash_colsum/ops.py:79-82) and never passes
    ``K_past`` (ops.py:89; kernel_causal.py:94-113), while ``naive_colsum`` computes
    batched causal column means (baselines.py:45-63) including ``K_len < Q_len``
    (baselines.py:58-62).

    Args:
        query: (B, H, Q_len, D), key: (B, H, K_len, D); fp16 or bf16, CUDA.
        k_past: keys every query sees before its own position -- key j is visible to
            query i iff ``j <= k_past + i``; default ``max(0, K_len - Q_len)``.
    Returns:
        (B, K_len), fp32 unless ``out_dtype`` says otherwise.
    """
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError(f"Expected 4D tensors, got query.ndim={query.ndim}, key.ndim={key.ndim}")
    if query.device.type != 'cuda':
        raise ValueError(f"Flash attention only supports CUDA tensors, got {query.device}")
    B, H, Q_len, D = query.shape
    if key.shape[0] != B or key.shape[1] != H or key.shape[3] != D:
        raise ValueError(
            f"Query and key must have same batch, heads and head_dim, got query: {query.shape}, key: {key.shape}")
    if k_past is not None and k_past < 0:
        raise ValueError(f"k_past must be non-negative, got {k_past}")
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    out = _without_work(query, key)
    if out is not None:
        return out if out_dtype is None else out.to(out_dtype)
    lib = _cabi.load()
    Q, K, code = _prepare(query, key)
    K_len = K.shape[2]
    with _on_device(Q.device):
        out = torch.empty((B, K_len), device=Q.device, dtype=torch.float32)
        ws = _workspace(lib, Q.device, B, H, Q_len, K_len, D, True, -1 if k_past is None else int(k_past))
        _check(lib.fcs_colsum_causal_batched(
            Q.data_ptr(), K.data_ptr(), out.data_ptr(), K_len, B, H, Q_len, K_len, D, code,
            Q.stride(0), Q.stride(1), Q.stride(2), K.stride(0), K.stride(1), K.stride(2),
            float(scale), -1 if k_past is None else int(k_past), 0, ws.data_ptr(), ws.numel(),
            _status_word(Q.device).data_ptr(), _raw_stream(Q.device)))
    if out_dtype is not None and out_dtype != out.dtype:
        out = out.to(out_dtype)
    return out


def statistics_rows(q_rows: int) -> int:
    """Rows per (batch, head) of the vector :func:`colsum_statistics` returns (``q_rows``
    rounded up to 256)."""
    return int(_cabi.load().fcs_statistics_rows(int(q_rows)))


def colsum_statistics(query_rows: torch.Tensor, key: torch.Tensor, scale: float, norm_rows: int,
                      h_norm: int = 0) -> torch.Tensor:
    """First pass alone (`fcs_colsum_statistics`): for the given query rows (any row range of a
    call, as a view) against all keys, minus (log2-sum-exp + log2(heads * norm_rows)).

    Returns fp32 ``(B * H, statistics_rows(rows))``; entries past the given rows are -inf.
    Non-causal.  With :func:`colsum_columns` this splits the work of one call over devices
    that all hold the inputs.
    """
    lib = _cabi.load()
    Q, K, code = _prepare(query_rows, key)
    B, H, rows, D = Q.shape
    Sk = K.shape[2]
    with _on_device(Q.device):
        lse = torch.full((B * H, statistics_rows(rows)), float("-inf"), dtype=torch.float32, device=Q.device)
        ws = _workspace_two_pass(lib, Q.device, B, H, rows, Sk, D)
        _check(lib.fcs_colsum_statistics(
            Q.data_ptr(), K.data_ptr(), lse.data_ptr(), B, H, rows, Sk, D, code,
            Q.stride(0), Q.stride(1), Q.stride(2), K.stride(0), K.stride(1), K.stride(2),
            float(scale), int(norm_rows), int(h_norm), ws.data_ptr(), ws.numel(),
            _status_word(Q.device).data_ptr(), _raw_stream(Q.device)))
    return lse


def colsum_columns(query: torch.Tensor, key_rows: torch.Tensor, neg_lse: torch.Tensor,
                   scale: float) -> torch.Tensor:
    """Second pass alone (`fcs_colsum_columns`): column means of the given keys (any row range
    of the key tensor, as a view) over all query rows of ``query``, from the statistics of all
    those rows (``neg_lse``: fp32, contiguous, ``(B * H, statistics_rows(query rows))``).
    Returns fp32 ``(B, key rows)``; nothing is left to reduce."""
    lib = _cabi.load()
    Q, K, code = _prepare(query, key_rows)
    B, H, rows, D = Q.shape
    k_rows = K.shape[2]
    if (neg_lse.dtype != torch.float32 or not neg_lse.is_contiguous()
            or tuple(neg_lse.shape) != (B * H, statistics_rows(rows))):
        raise ValueError(f"neg_lse must be contiguous fp32 of shape {(B * H, statistics_rows(rows))}")
    with _on_device(Q.device):
        out = torch.empty((B, k_rows), device=Q.device, dtype=torch.float32)
        ws = _workspace_two_pass(lib, Q.device, B, H, rows, k_rows, D)
        _check(lib.fcs_colsum_columns(
            Q.data_ptr(), K.data_ptr(), neg_lse.data_ptr(), out.data_ptr(), k_rows, B, H, rows, k_rows, D, code,
            Q.stride(0), Q.stride(1), Q.stride(2), K.stride(0), K.stride(1), K.stride(2),
            float(scale), ws.data_ptr(), ws.numel(),
            _status_word(Q.device).data_ptr(), _raw_stream(Q.device)))
    return out


def topk_columns(colsum: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The ``k`` most-attended key positions of every row of a column-mean tensor.

    ``colsum``: (B, S) fp32 CUDA tensor (what :func:`flash_colsum` returns).  Returns
    ``(values, indices)``, both (B, k), positions ascending (the kept tokens stay in
    order; ties go to the lower position), ``indices`` int32.  Runs on the current
    stream without synchronising -- the pruning step of the reference's use case,
    which the reference leaves to the caller.
    """
    if colsum.ndim != 2 or colsum.dtype != torch.float32 or colsum.device.type != "cuda":
        raise ValueError("topk_columns takes a 2-D fp32 CUDA tensor")
    B, S = colsum.shape
    if not 1 <= k <= S:
        raise ValueError(f"k must be in 1..{S}, got {k}")
    if colsum.stride(1) != 1:
        colsum = colsum.contiguous()
    lib = _cabi.load()
    with _on_device(colsum.device):
        idx = torch.empty((B, k), dtype=torch.int32, device=colsum.device)
        val = torch.empty((B, k), dtype=torch.float32, device=colsum.device)
        _check(lib.fcs_select_topk(colsum.data_ptr(), colsum.stride(0), B, S, int(k), idx.data_ptr(),
                                   val.data_ptr(), _raw_stream(colsum.device)))
    return val, idx


def threshold_columns(colsum: torch.Tensor, threshold: float, relative: bool = False
                      ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The key positions of every row whose column mean reaches a threshold.

    ``colsum``: (B, S) fp32 CUDA tensor.  A position is kept when its value is at least
    ``threshold``, or -- with ``relative`` -- at least ``threshold`` times the row's average
    value (1.0: more than a uniform share of the attention).  Returns ``(indices, counts)``:
    ``indices`` (B, S) int32 holds the kept positions of row b, ascending, in its first
    ``counts[b]`` entries and -1 after them; ``counts`` is (B,) int32.  Runs on the current
    stream without synchronising (the number kept stays on the device).
    """
    if colsum.ndim != 2 or colsum.dtype != torch.float32 or colsum.device.type != "cuda":
        raise ValueError("threshold_columns takes a 2-D fp32 CUDA tensor")
    if threshold != threshold:
        raise ValueError("threshold is not a number")
    B, S = colsum.shape
    if colsum.stride(1) != 1:
        colsum = colsum.contiguous()
    lib = _cabi.load()
    with _on_device(colsum.device):
        idx = torch.empty((B, S), dtype=torch.int32, device=colsum.device)
        cnt = torch.empty((B,), dtype=torch.int32, device=colsum.device)
        _check(lib.fcs_select_threshold(colsum.data_ptr(), colsum.stride(0), B, S, float(threshold), int(relative),
                                        idx.data_ptr(), cnt.data_ptr(), _raw_stream(colsum.device)))
    return idx, cnt


_copy_streams: Dict[int, torch.cuda.Stream] = {}


def _host_chunks(B: int, batch_chunk: Optional[int]):
    """(first entry, entries) of the chunks a host-memory call is copied and computed in."""
    if batch_chunk is not None:
        if batch_chunk <= 0:
            raise ValueError(f"batch_chunk must be positive, got {batch_chunk}")
        return [(b0, min(batch_chunk, B - b0)) for b0 in range(0, B, batch_chunk)]
    out, b0 = [], 0
    while b0 < B:
        left = B - b0
        n = left - max(1, left // 4) if left > 2 else 1
        out.append((b0, n))
        b0 += n
    return out


def flash_colsum_host(
    query: torch.Tensor,
    key: torch.Tensor,
    scale: Optional[float] = None,
    is_causal: bool = False,
    cls_len: Optional[int] = None,
    *,
    device: Optional[torch.device] = None,
    batch_chunk: Optional[int] = None,
) -> torch.Tensor:
    """``flash_colsum`` for inputs that live in host memory; returns a host tensor.

    Same arguments as :func:`flash_colsum`, but ``query`` and ``key`` are CPU
    tensors (pinned memory makes the copies asynchronous).  A batched call is cut
    along the batch into chunks whose host-to-device copies run on a second stream
    while the chunk before is being computed, so the call costs about the copy time
    of the inputs plus the compute of the last chunk.  By default the chunks shrink
    towards the end (three quarters of what is left, then single entries): few large
    copies, and only one entry's compute behind the last copy; ``batch_chunk`` asks
    for uniform chunks of that many entries instead.
    Causal and single-sample calls are copied in one piece.
    """
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError(f"Expected 4D tensors, got query.ndim={query.ndim}, key.ndim={key.ndim}")
    if query.device.type != "cpu" or key.device.type != "cpu":
        raise ValueError("flash_colsum_host takes host tensors; use flash_colsum for CUDA tensors")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B = query.shape[0]
    if is_causal or B == 1 or key.shape[0] != B:
        out = flash_colsum(query.to(dev, non_blocking=True), key.to(dev, non_blocking=True), scale,
                           is_causal, cls_len)
        return out.cpu()
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        copy_stream = _copy_streams.get(idx)
        if copy_stream is None:
            copy_stream = _copy_streams[idx] = torch.cuda.Stream(device=dev)
        main = torch.cuda.current_stream(dev)
        out = torch.empty((B, key.shape[2]), dtype=torch.float32, device=dev)
        copy_stream.wait_stream(main)
        staged = []
        for b0, n in _host_chunks(B, batch_chunk):
            with torch.cuda.stream(copy_stream):
                qd = query[b0:b0 + n].to(dev, non_blocking=True)
                kd = key[b0:b0 + n].to(dev, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy_stream)
            staged.append((b0, qd, kd, ready))
        for b0, qd, kd, ready in staged:
            main.wait_event(ready)
            # a one-entry chunk takes the single-sample entry point, a longer one the batched one
            out[b0:b0 + qd.shape[0]] = flash_colsum(qd, kd, scale, False, cls_len)
            qd.record_stream(main)
            kd.record_stream(main)
        return out.cpu()


__all__ = ["flash_colsum", "flash_colsum_causal", "flash_colsum_host", "topk_columns", "threshold_columns",
           "device_status"]
