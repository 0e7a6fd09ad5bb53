"""Multi-GPU partitioning of the quantized GEMMs: one process per GPU, ``torch.distributed`` for plumbing.

* Batched W8A8 (MoE-expert shape): the batch dimension shards across ranks; the batches are independent,
  so the data path has no collective.  An all-gather of the outputs exists only for callers that want
  the full tensor on every rank.
* W4A16 with a large output dimension: weight columns (rows of ``B_packed[N, K/2]`` and columns of
  ``scales[K/g, N]``) shard across ranks, activations are replicated, and the ``[M, N/g]`` output blocks
  are reassembled with one all-gather (NCCL over NVLink on GPUs, gloo in the CPU tests).

No kernel reads another GPU's memory: operands are resident on their rank, only outputs move.
The reference has no counterpart (its only multi-device code is one-sided SHMEM demos).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int, multiple: int = 1) -> Tuple[int, int]:
    """Contiguous [begin, end) owned by ``rank`` when ``total`` units are split over ``world`` ranks.

    Units are dealt in blocks of ``multiple`` (e.g. 128 weight rows); earlier ranks get the extra blocks."""
    if total % multiple != 0:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    blocks = total // multiple
    base, extra = divmod(blocks, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * multiple, end * multiple


def shard_batches(tensors, world: int, rank: int):
    """Slice dim 0 (the batch) of every tensor to this rank's range."""
    b0, b1 = shard_range(tensors[0].shape[0], world, rank)
    return [t[b0:b1].contiguous() for t in tensors]


class ColumnShardedW4A16:
    """W4A16 linear layer whose output features are split over the ranks of a process group.

    Holds this rank's rows of ``B_packed`` and columns of ``scales`` (made contiguous once, at load).
    ``forward(A)`` runs the local GEMM and, unless ``gather=False``, all-gathers the column blocks into the
    full ``[M, N]`` output on every rank."""

    def __init__(self, B_packed: torch.Tensor, scales: Optional[torch.Tensor], zero: int = 8, group_size: int = 128,
                 group: Optional[dist.ProcessGroup] = None, gemm: Optional[Callable] = None, multiple: int = 128):
        self.pg = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N = B_packed.shape[0]
        if self.N % (multiple * self.world) != 0:
            raise ValueError(f"N={self.N} must split into equal blocks of {multiple} over {self.world} ranks")
        self.n0, self.n1 = shard_range(self.N, self.world, self.rank, multiple)
        self.B_local = B_packed[self.n0:self.n1].contiguous()
        self.s_local = None if scales is None else scales[:, self.n0:self.n1].contiguous()
        self.zero, self.group_size = zero, group_size
        if gemm is None:
            from .ops import w4a16_gemm as gemm
        self._gemm = gemm

    def to(self, device):
        self.B_local = self.B_local.to(device)
        if self.s_local is not None:
            self.s_local = self.s_local.to(device)
        return self

    def forward(self, A: torch.Tensor, gather: bool = True) -> torch.Tensor:
        C_local = self._gemm(A, self.B_local, self.s_local, self.zero, self.group_size)
        if not gather or self.world == 1:
            return C_local
        M, nl = C_local.shape
        parts = torch.empty((self.world * M, nl), dtype=C_local.dtype, device=C_local.device)
        dist.all_gather_into_tensor(parts, C_local, group=self.pg)  # rank r's block lands in rows [r*M, (r+1)*M)
        return parts.view(self.world, M, nl).permute(1, 0, 2).reshape(M, self.world * nl)

    __call__ = forward
