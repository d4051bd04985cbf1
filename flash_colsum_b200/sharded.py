"""Head-sharded column means across the GPUs of one node.

Each (batch, head) unit contributes additively to its batch row of the result,
so the heads are split over the ranks, every rank runs the local kernels with
the mean taken over the GLOBAL head count, and the small fp32 per-key partial
vectors are summed with one collective.  One process per GPU
(``torch.distributed``, NCCL over NVLink); no exchange happens inside the
kernels.  The reference has no multi-GPU path; its single-GPU launchers are
flash_colsum/kernel_causal.py:94 and kernel_noncausal_batched.py:102.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def shard_range(n: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous balanced split of ``n`` units: ranks < n % world get one more."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(n, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def _local_partial(query: torch.Tensor, key: torch.Tensor, scale: float, is_causal: bool,
                   cls_len: Optional[int], h_total: int) -> torch.Tensor:
    """This rank's heads, normalised by the global head count: fp32 (B, S_k)."""
    if is_causal:
        return ops._flash_colsum_causal(query, key, scale, h_norm=h_total)
    cls_n = -1 if cls_len is None else int(cls_len)
    if query.shape[0] == 1:
        return ops._flash_colsum_non_batched(query, key, scale, CLS_N=cls_n, h_norm=h_total)
    return ops._flash_colsum_batched(query, key, scale, CLS_N=cls_n, h_norm=h_total)


def flash_colsum_head_sharded(
    query_shard: torch.Tensor,
    key_shard: torch.Tensor,
    h_total: int,
    scale: Optional[float] = None,
    is_causal: bool = False,
    cls_len: Optional[int] = None,
    group: Optional[dist.ProcessGroup] = None,
    dst: Optional[int] = None,
    local_fn: Callable = _local_partial,
) -> torch.Tensor:
    """Column means when each rank holds ``(B, H_local, S, D)`` of the heads.

    ``h_total`` is the number of heads over all ranks.  With ``dst=None`` every
    rank returns the full result (all-reduce); otherwise only rank ``dst`` does
    (reduce) and the others return their partial.  A rank may hold zero heads
    (``H_local == 0``): it contributes zeros.
    """
    if query_shard.ndim != 4 or key_shard.ndim != 4:
        raise ValueError("Expected 4D tensors")
    if h_total <= 0:
        raise ValueError(f"h_total must be positive, got {h_total}")
    if cls_len is not None and is_causal:
        raise ValueError("cls_len is only supported for non-causal attention")
    B, h_local, _, D = query_shard.shape
    if h_local > h_total:
        raise ValueError(f"shard has {h_local} heads but h_total is {h_total}")
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    if h_local == 0:
        partial = torch.zeros(B, key_shard.shape[2], dtype=torch.float32, device=query_shard.device)
    else:
        partial = local_fn(query_shard, key_shard, scale, is_causal, cls_len, h_total)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        if dst is None:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
        else:
            dist.reduce(partial, dst=dst, op=dist.ReduceOp.SUM, group=group)
    return partial


__all__ = ["shard_range", "flash_colsum_head_sharded"]
