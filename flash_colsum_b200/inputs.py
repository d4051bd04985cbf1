"""Seeded synthetic inputs for the attention column-mean workloads.

The reference benchmarks on ``torch.randn`` tensors only
(benchmarks/benchmark_colsum.py:302-303, 348-349, 394-395), so seeded normal
tensors of the benchmark shapes are the benchmark.  Everything is drawn on the
CPU from one ``torch.Generator`` in fp32 -- query first, then key, then (for the
outlier workload) one U(0.5, 2) factor per key position -- and only then cast,
so a CPU checker fed the cast-then-upcast values sees exactly the numbers the
GPU kernels see.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


@dataclass(frozen=True)
class Workload:
    """One named shape of the operator call."""

    name: str
    B: int
    H: int
    Sq: int
    Sk: int
    D: int
    dtype: str = "fp16"
    is_causal: bool = False
    cls_len: Optional[int] = None
    key_outliers: bool = False   # scale key rows by per-position U(0.5, 2)
    key_is_query: bool = False   # K = Q.clone() (strong diagonal)
    seed: int = 0

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype]

    @property
    def rows_averaged(self) -> int:
        """Query rows per head that enter the mean."""
        if self.cls_len is not None and not self.is_causal:
            return min(int(self.cls_len), self.Sq)
        return self.Sq

    @property
    def flop(self) -> float:
        """Nominal work, two passes of 2*B*H*Sq*Sk*D, masks not discounted."""
        return 4.0 * self.B * self.H * self.Sq * self.Sk * self.D

    @property
    def flop_rows_used(self) -> float:
        """Same count restricted to the query rows the result depends on."""
        return 4.0 * self.B * self.H * self.rows_averaged * self.Sk * self.D

    @property
    def min_bytes(self) -> float:
        """Least HBM traffic: the used query rows and all keys once, plus the output."""
        el = 4 if self.dtype == "fp32" else 2
        return (self.B * self.H * (self.rows_averaged + self.Sk) * self.D * el
                + self.B * self.Sk * 4)


# The five shapes the headline numbers are quoted on.
WORKLOADS = {
    "c1": Workload("c1", 2, 4, 256, 256, 64, "fp32"),
    "c2": Workload("c2", 8, 16, 2048, 2048, 64, "fp16"),
    "c2_kq": Workload("c2_kq", 8, 16, 2048, 2048, 64, "fp16", key_is_query=True),
    "c3": Workload("c3", 32, 16, 577, 577, 64, "fp16", cls_len=1),
    "c4": Workload("c4", 1, 32, 128, 4096, 128, "fp16", is_causal=True),
    "c5": Workload("c5", 1, 32, 512, 131072, 128, "bf16", is_causal=True,
                   key_outliers=True),
}


def make_inputs(w: Workload, heads: Optional[Tuple[int, int]] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """CPU tensors (query, key) for ``w`` in its dtype.

    ``heads=(lo, hi)`` returns only that head range; the full tensors are still
    drawn so every shard of a head-sharded run sees the same numbers as the
    unsharded run.
    """
    g = torch.Generator().manual_seed(w.seed)
    q = torch.randn(w.B, w.H, w.Sq, w.D, generator=g, dtype=torch.float32)
    if w.key_is_query:
        k = q.clone()
    else:
        k = torch.randn(w.B, w.H, w.Sk, w.D, generator=g, dtype=torch.float32)
    if w.key_outliers:
        f = torch.rand(w.Sk, generator=g, dtype=torch.float32) * 1.5 + 0.5
        k = k * f[None, None, :, None]
    if heads is not None:
        lo, hi = heads
        q = q[:, lo:hi]
        k = k[:, lo:hi]
    return q.to(w.torch_dtype).contiguous(), k.to(w.torch_dtype).contiguous()


def digest(*tensors: torch.Tensor) -> str:
    """sha256 over the raw bytes of the tensors; pins regenerated inputs."""
    h = hashlib.sha256()
    for t in tensors:
        t = t.detach().cpu().contiguous()
        h.update(t.view(torch.uint8).numpy().tobytes())
    return h.hexdigest()
