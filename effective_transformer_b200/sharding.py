"""Sequence-sharded replicas: the bookkeeping around a batch that is split over
several GPUs, one process per GPU.

Sequences are independent (attention never crosses them and every other stage
is per token), so the forward pass of a shard needs no exchange step.  The only
traffic between GPUs is the optional gather of the shard outputs behind the
pass, which this module implements: every rank sends its padded [b_r, S, H]
output to the destination rank, which receives all of them into one local
buffer and puts the sequences back into the order of the original batch.
Receives land in the destination's own memory; no kernel is handed a peer's
memory.  The reference has no multi-GPU mode; `workloads.balanced_shards`
decides which sequences a rank owns.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


def shard_row_offsets(shards: Sequence[np.ndarray]) -> np.ndarray:
    """First row of every rank's block in the gathered (rank-major) buffer, plus the total."""
    off = np.zeros(len(shards) + 1, dtype=np.int64)
    off[1:] = np.cumsum([len(s) for s in shards])
    return off


def inverse_order(shards: Sequence[np.ndarray]) -> np.ndarray:
    """inv such that gathered[inv[i]] is sequence i of the original batch, when `gathered` holds the
    ranks' blocks one after another, each in the order `shards[r]` lists its sequences."""
    order = np.concatenate([np.asarray(s, dtype=np.int64) for s in shards])
    inv = np.empty_like(order)
    inv[order] = np.arange(len(order), dtype=np.int64)
    return inv


class OutputGather:
    """Gathers the ranks' padded outputs on `dst` and restores the batch order.

    Buffers are allocated once (the destination's [B, S, H] receive buffer and the re-ordered
    result), so a call only moves data: one send per rank, `world - 1` receives and one local copy
    on the destination, then a row gather by the inverse permutation."""

    def __init__(self, shards: Sequence[np.ndarray], seq_len: int, hidden: int, dtype: torch.dtype,
                 device: torch.device, dst: int = 0, group: Optional[dist.ProcessGroup] = None):
        self.shards = [np.asarray(s, dtype=np.int64) for s in shards]
        self.group, self.dst = group, dst
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if len(self.shards) != self.world:
            raise ValueError("one shard per rank is required")
        self.offsets = shard_row_offsets(self.shards)
        self.batch = int(self.offsets[-1])
        self.row_shape = (seq_len, hidden)
        self.bytes_received = 0
        if self.rank == dst:
            self.recv = torch.empty((self.batch, seq_len, hidden), dtype=dtype, device=device)
            self.result = torch.empty_like(self.recv)
            self.inv = torch.from_numpy(inverse_order(self.shards)).to(device)
            elem = self.recv.element_size() * seq_len * hidden
            self.bytes_received = int(sum(len(s) for r, s in enumerate(self.shards) if r != dst)) * elem
        else:
            self.recv = self.result = self.inv = None

    def __call__(self, local_out: torch.Tensor) -> Optional[torch.Tensor]:
        """local_out: this rank's [b_r, S, H] output.  Returns the [B, S, H] tensor in the original
        batch order on the destination rank, None elsewhere."""
        mine = len(self.shards[self.rank])
        if tuple(local_out.shape) != (mine,) + self.row_shape:
            raise ValueError("local_out must be [len(shards[rank]), S, H]")
        ops: List[dist.P2POp] = []
        if self.rank == self.dst:
            for r in range(self.world):
                lo, hi = int(self.offsets[r]), int(self.offsets[r + 1])
                if hi == lo:
                    continue
                if r == self.dst:
                    self.recv[lo:hi].copy_(local_out)
                else:
                    ops.append(dist.P2POp(dist.irecv, self.recv[lo:hi], r, self.group))
        elif mine > 0:
            ops.append(dist.P2POp(dist.isend, local_out.contiguous(), self.dst, self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        if self.rank != self.dst:
            return None
        torch.index_select(self.recv, 0, self.inv, out=self.result)
        return self.result
