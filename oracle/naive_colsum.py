"""CPU restatement of the reference's materialising column-mean of attention.

TEST INFRASTRUCTURE ONLY.  Nothing on the product path imports this module: it is
the checker used by the tests, by the smoke test and by the CPU-baseline leg of
the benchmark.  The product path is the CUDA library and fails loudly without it.

What it restates (reference flash_colsum/baselines.py:13-78, ``naive_colsum``):

* scores = (Q @ K^T) * scale, scale defaulting to 1/sqrt(D)   (baselines.py:38-42)
* causal mask, suffix-aligned: with S_k >= S_q the first K_past = S_k - S_q keys
  are visible to every query and the last S_q keys are lower-triangular
  (baselines.py:49-57); with S_k < S_q the plain ``k <= q`` mask
  (baselines.py:58-62).  Both are ``k <= max(0, S_k - S_q) + q``.
* softmax over keys in fp32, cast back to the input dtype      (baselines.py:66)
* mean over heads and over either all query rows or the first
  ``min(cls_len, S_q)`` rows (non-causal only)                  (baselines.py:68-76)

Parity pin: ``tests/golden/naive_colsum_golden.npz`` holds outputs of the
reference function itself (imported from a checkout of the reference by
``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this file and
the C restatement against every one of them.
"""

from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch


def causal_k_past(s_q: int, s_k: int) -> int:
    """Number of prefix keys every query sees (kernel_causal.py:113)."""
    return max(0, s_k - s_q)


def naive_colsum_torch(query: torch.Tensor, key: torch.Tensor,
                       scale: Optional[float] = None, is_causal: bool = False,
                       cls_len: Optional[int] = None,
                       head_chunk: Optional[int] = None) -> torch.Tensor:
    """Torch-on-CPU port, same operator sequence as the reference.

    With ``head_chunk`` the heads are processed that many at a time and the
    per-chunk sums added in fp32, so that long key lengths fit in host memory;
    the result is then fp32 whatever the input dtype.
    """
    B, H, S_q, D = query.shape
    S_k = key.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if not is_causal and cls_len is not None:
        if cls_len <= 0:
            raise ValueError(f"cls_len must be positive, got {cls_len}")
        rows = min(int(cls_len), S_q)
    else:
        rows = S_q

    visible = None
    if is_causal:
        q_idx = torch.arange(S_q).unsqueeze(1)
        k_idx = torch.arange(S_k).unsqueeze(0)
        visible = k_idx <= (causal_k_past(S_q, S_k) + q_idx)

    def one(qc: torch.Tensor, kc: torch.Tensor) -> torch.Tensor:
        s = torch.matmul(qc, kc.transpose(-2, -1)) * scale
        if visible is not None:
            s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1, dtype=torch.float32).to(qc.dtype)
        return p[:, :, :rows, :]

    if head_chunk is None:
        return one(query, key).mean(dim=(1, 2))
    acc = torch.zeros(B, S_k, dtype=torch.float32)
    for h0 in range(0, H, head_chunk):
        p = one(query[:, h0:h0 + head_chunk], key[:, h0:h0 + head_chunk])
        acc += p.to(torch.float32).sum(dim=(1, 2))
    return acc / float(H * rows)


def naive_colsum_f64(query, key, scale: Optional[float] = None,
                     is_causal: bool = False, cls_len: Optional[int] = None,
                     k_past: Optional[int] = None) -> np.ndarray:
    """numpy float64 evaluation of the same definition, (b, h) at a time.

    ``k_past`` replaces the inferred ``max(0, S_k - S_q)`` of the causal rule, as the
    reference's causal launcher allows (flash_colsum/kernel_causal.py:94-113)."""
    q = np.asarray(query.detach().to(torch.float64).numpy() if isinstance(query, torch.Tensor) else query,
                   dtype=np.float64)
    k = np.asarray(key.detach().to(torch.float64).numpy() if isinstance(key, torch.Tensor) else key,
                   dtype=np.float64)
    B, H, S_q, D = q.shape
    S_k = k.shape[2]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    rows = min(int(cls_len), S_q) if (cls_len is not None and not is_causal) else S_q
    out = np.zeros((B, S_k), dtype=np.float64)
    limit = None
    if is_causal:
        limit = (causal_k_past(S_q, S_k) if k_past is None else int(k_past)) + np.arange(S_q)[:, None]
    kk = np.arange(S_k)[None, :]
    for b in range(B):
        for h in range(H):
            s = (q[b, h] @ k[b, h].T) * scale
            if limit is not None:
                s = np.where(kk <= limit, s, -np.inf)
            s = s - s.max(axis=1, keepdims=True)
            e = np.exp(s)
            p = e / e.sum(axis=1, keepdims=True)
            out[b] += p[:rows].sum(axis=0)
    return out / float(H * rows)


def topk_positions(colsum, k: int) -> np.ndarray:
    """Per row, the k positions with the largest value, ascending; ties go to the lower
    position.  The checker for the pruning step (plain sort)."""
    v = np.asarray(colsum)
    out = np.empty((v.shape[0], k), dtype=np.int64)
    for b in range(v.shape[0]):
        order = np.lexsort((np.arange(v.shape[1]), -v[b].astype(np.float64)))
        out[b] = np.sort(order[:k])
    return out


def parity_errors(got, want):
    """(rel-L2, max-abs / max column mean) of fp32/fp64 arrays."""
    g = np.asarray(got, dtype=np.float64)
    w = np.asarray(want, dtype=np.float64)
    rel_l2 = float(np.linalg.norm(g - w) / max(np.linalg.norm(w), 1e-300))
    max_abs = float(np.abs(g - w).max() / max(np.abs(w).max(), 1e-300))
    return rel_l2, max_abs
