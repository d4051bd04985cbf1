"""Column means across the GPUs of one node: heads split over the ranks (below), or the work
of one call split by query rows and keys (`flash_colsum_work_sharded`, at the end).

Head-sharded:

Each (batch, head) unit contributes additively to its batch row of the result,
so the heads are split over the ranks, every rank runs the local kernels with
the mean taken over the GLOBAL head count, and the small fp32 per-key partial
vectors are summed with one collective.  One process per GPU
(``torch.distributed``, NCCL over NVLink); no exchange happens inside the
kernels.  The reference has no multi-GPU path; its single-GPU launchers are
flash_colsum/kernel_causal.py:94 and kernel_noncausal_batched.py:102.
"""

from __future__ import annotations

import os
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


class PeerAccumulator:
    """Two fp32 ``(1, S_k)`` buffers and a few flags per rank in symmetric (peer-mapped) memory.

    Used to fold the reduce of the head-sharded causal call into the kernels: every
    rank's column pass adds its per-key sums straight into a buffer of rank ``dst``
    over NVLink (plain system-scope atomic adds to a peer address, no multicast); the last
    CTA of that pass then stores a flag on rank ``dst`` (release, system scope), and rank
    ``dst`` waits for the flags of all ranks -- a bounded wait in a one-warp kernel -- and has
    the sum.  No collective and no all-to-all barrier: only rank ``dst`` waits for the others.
    Calls alternate between the two buffers: while call n adds into one, rank ``dst`` zeroes
    the other inside its statistics pass and its column pass then tells every rank so (a second
    flag); a rank's column pass of call n + 1 adds nothing before it has seen that flag of
    call n.  One process per GPU; the constructor is a collective over ``group``.
    """

    DONE, CLEARED = 0, 32     # int32 slots of the flag array

    def __init__(self, k_len: int, device: torch.device, group=None, dst: int = 0):
        # peer mappings only: keep NVLink multicast objects out of it
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        from . import _cabi
        group = group if group is not None else dist.group.WORLD
        self.k_len = int(k_len)
        self.dst = int(dst)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 16:
            raise ValueError("the peer-memory reduce is built for the GPUs of one node (at most 16 ranks)")
        self.local = symm_mem.empty((2, self.k_len), dtype=torch.float32, device=device)
        self.handle = symm_mem.rendezvous(self.local, group)
        both = self.handle.get_buffer(self.dst, (2, self.k_len), torch.float32)
        self.targets = (both[0], both[1])
        self.local.zero_()
        self.flags = symm_mem.empty((64,), dtype=torch.int32, device=device)
        self.flag_handle = symm_mem.rendezvous(self.flags, group)
        self.flags.zero_()
        # the CTA counter of the column pass is local and hot: ordinary device memory (atomics on the
        # peer-mapped allocation cost ~0.45 us each, one per CTA)
        self._counter = torch.zeros(1, dtype=torch.int32, device=device)
        self._lib = _cabi.load()
        self._cabi = _cabi
        self._device = device
        self._others = [r for r in range(self.world) if r != self.dst]
        flags_on_dst = self.flag_handle.get_buffer(self.dst, (64,), torch.int32)
        self._keep = [flags_on_dst]
        if self.rank == self.dst:
            peers = [self.flag_handle.get_buffer(r, (64,), torch.int32) for r in self._others]
            self._keep += peers
            self._cleared_ptrs = [t.data_ptr() + 4 * self.CLEARED for t in peers]
            self._post = (ctypes.c_void_p * max(1, len(peers)))(*self._cleared_ptrs)
        else:
            self._done_ptr = flags_on_dst.data_ptr() + 4 * (self.DONE + self.rank)
            self._post = (ctypes.c_void_p * 1)(self._done_ptr)
        self.calls = 0
        self.parity = 0
        torch.cuda.synchronize(device)
        self.handle.barrier(channel=0)     # every rank's buffers and flags are clear before the first add
        torch.cuda.synchronize(device)

    def _signals(self, n: int):
        sig = self._cabi.PeerSignals()
        if self.rank == self.dst:
            for i, ptr in enumerate(self._cleared_ptrs):
                sig.post[i] = ptr
            sig.post_n, sig.post_value = len(self._cleared_ptrs), n
        else:
            sig.wait_flag = self.flags.data_ptr() + 4 * self.CLEARED
            sig.wait_value = n - 1
            sig.counter = self._counter.data_ptr()
            sig.done_flag, sig.done_value = self._done_ptr, n
        return sig

    def reduce(self, launch: Callable) -> torch.Tensor:
        """Run ``launch(target, clear_next, signals)`` on every rank; rank ``dst`` gets the summed
        result (a view of its local buffer, valid until the call after the next one), the others a
        stale buffer.  ``clear_next`` is the buffer of the next call on rank ``dst`` (to be zeroed
        by the launched kernels) and None elsewhere.  ``launch`` returns False when its kernels
        cannot take the signals (it then ran them without, between the same flags issued by
        one-warp kernels)."""
        from . import ops
        self.calls += 1
        n, p = self.calls, self.parity
        lib, dev = self._lib, self._device
        is_dst = self.rank == self.dst
        with ops._on_device(dev):
            stream = ops._raw_stream(dev)
            status = ops._status_word(dev).data_ptr()
            in_kernel = launch(self.targets[p], self.local[p ^ 1] if is_dst else None, self._signals(n))
            if not in_kernel:
                # the same protocol by separate one-warp kernels around the launch
                if not is_dst:
                    ops._check(lib.fcs_peer_wait(self.flags.data_ptr() + 4 * self.CLEARED, 1, n - 1, status, stream))
                launch(self.targets[p], self.local[p ^ 1] if is_dst else None, None)
                if self._others or not is_dst:
                    if is_dst and self._others:
                        ops._check(lib.fcs_peer_post(self._post, len(self._others), n, stream))
                    elif not is_dst:
                        ops._check(lib.fcs_peer_post(self._post, 1, n, stream))
            if is_dst and self._others:
                lo, hi = min(self._others), max(self._others)
                base = self.flags.data_ptr() + 4 * self.DONE
                # (rank dst's own slot is never posted: wait on the slots before and after it)
                if lo < self.dst:
                    ops._check(lib.fcs_peer_wait(base + 4 * lo, self.dst - lo, n, status, stream))
                if hi > self.dst:
                    ops._check(lib.fcs_peer_wait(base + 4 * (self.dst + 1), hi - self.dst, n, status, stream))
        self.parity = p ^ 1
        return self.local[p:p + 1]


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
    peer: Optional[PeerAccumulator] = None,
) -> torch.Tensor:
    """Column means when each rank holds ``(B, H_local, S, D)`` of the heads.

    ``h_total`` is the number of heads over all ranks.  With ``dst=None`` every
    rank returns the full result (all-reduce); otherwise only rank ``dst`` does
    (reduce) and the others return their partial.  A rank may hold zero heads
    (``H_local == 0``): it contributes zeros.

    With ``peer`` (causal only) there is no collective at all: every rank's
    kernels add into the buffer of rank ``peer.dst`` through peer memory, and only
    that rank's return value is the result.
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
    if peer is not None:
        if not is_causal:
            raise ValueError("the peer-memory reduce is implemented for the causal call")
        if peer.k_len != key_shard.shape[2]:
            raise ValueError(f"peer buffer holds {peer.k_len} keys, the call has {key_shard.shape[2]}")

        def launch(target: torch.Tensor, clear_next: Optional[torch.Tensor], signals) -> bool:
            if h_local > 0:
                out = ops._flash_colsum_causal(query_shard, key_shard, scale, h_norm=h_total, accumulate_into=target,
                                               clear_next=clear_next, signals=signals)
                return out is not None
            if signals is not None:
                return False          # no kernels of this rank to carry the flags
            if clear_next is not None:
                clear_next.zero_()
            return True

        return peer.reduce(launch)
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


__all__ = ["shard_range", "flash_colsum_head_sharded", "PeerAccumulator"]


def work_shares(n: int, world_size: int, granule: int):
    """Contiguous shares of ``n`` rows over ``world_size`` ranks, each a multiple of ``granule``
    rows long (the last one takes what is left, later ones may be empty).  Returns the share
    length and the list of ``(lo, hi)``."""
    per = -(-n // world_size)
    share = -(-per // granule) * granule
    return share, [(min(n, r * share), min(n, (r + 1) * share)) for r in range(world_size)]


def flash_colsum_work_sharded(
    query: torch.Tensor,
    key: torch.Tensor,
    scale: Optional[float] = None,
    cls_len: Optional[int] = None,
    group=None,
    stats_fn: Optional[Callable] = None,
    columns_fn: Optional[Callable] = None,
) -> torch.Tensor:
    """One non-causal call split over the ranks of ``group`` by WORK, not by heads: every rank
    holds the whole ``query`` and ``key`` (B, H, S, D); rank r runs the statistics pass for its
    share of the query rows, the ranks all-gather the per-row statistics (4 bytes per row and
    head), rank r runs the column pass for its share of the keys, and the finished column
    blocks are all-gathered into the (B, S) result on every rank.  For calls with fewer heads
    than GPUs (a long single sample).  ``stats_fn`` / ``columns_fn`` replace the two kernels
    (CPU tests)."""
    if query.ndim != 4 or key.shape != query.shape:
        raise ValueError(f"query and key must be 4-D tensors of the same shape, got {query.shape}, {key.shape}")
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, H, S, D = query.shape
    if scale is None:
        scale = 1.0 / (D ** 0.5)
    rows = S if cls_len is None else min(int(cls_len), S)
    stats_fn = stats_fn or ops.colsum_statistics
    columns_fn = columns_fn or ops.colsum_columns
    dev = query.device

    # pass 1 on a share of the query rows (multiples of 256 so that the vectors concatenate)
    q_share, q_ranges = work_shares(rows, world, 256)
    lo, hi = q_ranges[rank]
    mine = torch.full((B * H, q_share), float("-inf"), dtype=torch.float32, device=dev)
    if hi > lo:
        part = stats_fn(query[:, :, lo:hi], key, scale, rows)
        mine[:, :part.shape[1]] = part[:, :q_share]
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    total_rows = -(-rows // 256) * 256
    neg_lse = torch.cat(gathered, dim=1)[:, :total_rows].contiguous()

    # pass 2 on a share of the keys: its output columns are final
    k_share, k_ranges = work_shares(S, world, 128)
    lo, hi = k_ranges[rank]
    block = torch.zeros((B, k_share), dtype=torch.float32, device=dev)
    if hi > lo:
        block[:, :hi - lo] = columns_fn(query[:, :, :rows], key[:, :, lo:hi], neg_lse, scale)
    blocks = [torch.empty_like(block) for _ in range(world)]
    dist.all_gather(blocks, block, group=group)
    return torch.cat(blocks, dim=1)[:, :S].contiguous()
