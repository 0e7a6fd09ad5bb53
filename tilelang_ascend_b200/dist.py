"""Multi-GPU partitioning of the quantized GEMMs: one process per GPU, ``torch.distributed`` for plumbing.

* Batched W8A8 (MoE-expert shape): the batch dimension shards across ranks; the batches are independent,
  so the data path has no collective.  An all-gather of the outputs exists only for callers that want
  the full tensor on every rank.
* W4A16 with a large output dimension: weight columns (rows of ``B_packed[N, K/2]`` and columns of
  ``scales[K/g, N]``) shard across ranks, activations are replicated, and the ``[M, N/g]`` output blocks
  are reassembled on every rank: on the GPUs of one node by the GEMM kernel itself, which stores its block into
  every rank's output buffer over NVLink (peer stores from the epilogue, no collective on the data), else with
  one all-gather (NCCL, or gloo in the CPU tests).

* Grouped (ragged) W8A8: whole groups (experts) shard across ranks; each rank holds its experts' weights and
  scales and receives only its groups' rows, so again no collective on the data path.

No kernel reads another GPU's memory or waits for another GPU: operands are resident on their rank, only
outputs move, as plain stores.  The reference's multi-device code is its one-sided SHMEM demos
(examples/shmem/shmem_mm_test_put_nbi.py:69-74: a GEMM followed by a put of its result), which is the
pattern the peer-store form fuses into the GEMM's epilogue.
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
    ``forward(A)`` runs the local GEMM and, unless ``gather=False``, leaves the full ``[M, N]`` output on every rank.

    Two ways of assembling it:

    * peer stores (CUDA ranks of one node, the default there): every rank owns a full ``[M, N]`` buffer, the
      buffers are mapped into all processes once per token count, and the GEMM kernel's epilogue writes this
      rank's column block into every rank's buffer itself.  The output crosses NVLink while the GEMM still runs,
      nothing is re-arranged afterwards.  What tells a rank that all blocks have landed is a flag per peer in a
      small mapped array, set and awaited by one tiny kernel behind the GEMM (``landed="flags"``, the default), or
      a one-element all-reduce (``landed="allreduce"``).  Two buffers alternate, so a rank may still read one
      result while its peers already write the next: a returned tensor stays valid until the forward after next
      of the same token count (copy it in stream order to keep it longer).
    * collective (``peer_stores=False``, CPU / gloo, or when mapping fails): one all-gather of the ``[M, N/g]``
      blocks and a copy into column order (no copy for a single token, whose blocks are already in order)."""

    def __init__(self, B_packed: torch.Tensor, scales: Optional[torch.Tensor], zero: int = 8, group_size: int = 128,
                 group: Optional[dist.ProcessGroup] = None, gemm: Optional[Callable] = None, multiple: int = 128,
                 peer_stores="auto", share_buffers_with: Optional["ColumnShardedW4A16"] = None, landed: str = "flags"):
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
        self._custom_gemm = gemm is not None
        if gemm is None:
            from .ops import w4a16_gemm as gemm
        self._gemm = gemm
        self.peer_stores = peer_stores
        self._peers = {}    # (M, dtype) -> [generation 0, generation 1], each (own buffer, [address per rank])
        self._gen = {}
        self._opened = []   # (base address, device) of every mapping of a peer's allocation
        if landed not in ("flags", "allreduce"):
            raise ValueError("landed must be 'flags' or 'allreduce'")
        self.landed = landed
        self._token = None  # one element, all-reduced as the "all blocks have landed" barrier (landed="allreduce")
        self._flags = None  # (own int32 flag array, [address of this rank's slot in every rank's array])
        self._owner = self  # the layer whose output buffers this one writes (several layers of one shape, say the
        if share_buffers_with is not None:  # same projection of different blocks, can share them)
            if share_buffers_with.N != self.N or share_buffers_with.world != self.world:
                raise ValueError("layers that share output buffers must have the same N and process group")
            self._owner = share_buffers_with._owner

    def to(self, device):
        self.B_local = self.B_local.to(device)
        if self.s_local is not None:
            self.s_local = self.s_local.to(device)
        return self

    # ---------------------------------------------------------------- peer-store plumbing
    def _use_peers(self, A) -> bool:
        if self.peer_stores is False or self._custom_gemm or self.world == 1 or self.world > 8 or not A.is_cuda:
            return False
        return (self.n1 - self.n0) % 64 == 0 and self.N % 8 == 0

    def _peer_buffers(self, M, dtype, device):
        if self._owner is not self:
            return self._owner._peer_buffers(M, dtype, device)
        key = (M, dtype)
        if key not in self._peers:
            from .ops import ipc_export, ipc_open
            gens = []
            for _ in range(2):
                buf = torch.empty((M, self.N), dtype=dtype, device=device)
                infos = [None] * self.world
                dist.all_gather_object(infos, ipc_export(buf), group=self.pg)
                ptrs = []
                for r, (handle, off) in enumerate(infos):
                    if r == self.rank:
                        ptrs.append(buf.data_ptr())
                    else:
                        base = ipc_open(handle, device)
                        self._opened.append((base, device))
                        ptrs.append(base + off)
                gens.append((buf, ptrs))
            self._peers[key] = gens
            self._gen[key] = 0
            if self._token is None:
                self._token = torch.zeros(1, dtype=torch.float32, device=device)
            if self._flags is None and self.landed == "flags":
                flags = torch.zeros(64, dtype=torch.int32, device=device)  # a slot per rank; the rest pads the line
                infos = [None] * self.world
                dist.all_gather_object(infos, ipc_export(flags), group=self.pg)
                slots = []
                for r, (handle, off) in enumerate(infos):
                    if r == self.rank:
                        slots.append(flags.data_ptr() + 4 * self.rank)
                    else:
                        base = ipc_open(handle, device)
                        self._opened.append((base, device))
                        slots.append(base + off + 4 * self.rank)
                self._flags = (flags, slots)
                torch.cuda.synchronize(device)  # the flags are zero before any peer can signal
            dist.barrier(group=self.pg)  # every rank has mapped every buffer before anyone writes
        return key

    def close(self):
        """Unmap the peers' buffers (collective: every rank calls it, none may still be writing)."""
        if self._opened:
            from .ops import ipc_close
            torch.cuda.synchronize()
            dist.barrier(group=self.pg)
            for base, device in self._opened:
                ipc_close(base, device)
            self._opened = []
            self._peers = {}
            self._flags = None

    # ---------------------------------------------------------------- forward
    def forward(self, A: torch.Tensor, gather: bool = True) -> torch.Tensor:
        if gather and self.world > 1 and self._use_peers(A):
            try:
                key = self._peer_buffers(A.shape[0], A.dtype, A.device)
            except Exception as exc:  # mapping is not possible here (no peer access, another allocator): use the collective
                if self.peer_stores is True:
                    raise
                import warnings
                warnings.warn(f"peer stores are not available ({exc}); gathering with a collective instead")
                self.peer_stores = False
            else:
                from .ops import w4a16_gemm_gather
                own = self._owner
                g = own._gen[key]
                own._gen[key] = g ^ 1
                buf, ptrs = own._peers[key][g]
                w4a16_gemm_gather(A, self.B_local, self.s_local, self.zero, self.group_size, ptrs, self.N, self.n0)
                # in stream order behind the kernel: all ranks' blocks have landed in this rank's buffer
                if own._flags is not None:
                    from .ops import peer_signal_wait
                    # the epoch is counted on the device (slot 32 of the flag array), so graph replays keep counting
                    peer_signal_wait(own._flags[1], own._flags[0], epoch_counter=own._flags[0][32:33])
                else:
                    dist.all_reduce(own._token, group=self.pg)
                return buf
        C_local = self._gemm(A, self.B_local, self.s_local, self.zero, self.group_size)
        if not gather or self.world == 1:
            return C_local
        M, nl = C_local.shape
        parts = torch.empty((self.world * M, nl), dtype=C_local.dtype, device=C_local.device)
        dist.all_gather_into_tensor(parts, C_local, group=self.pg)  # rank r's block lands in rows [r*M, (r+1)*M)
        if M == 1:
            return parts.view(1, self.world * nl)  # one token: the blocks are already in column order
        return parts.view(self.world, M, nl).permute(1, 0, 2).reshape(M, self.world * nl)

    __call__ = forward


def shard_groups(batch_sizes_list, world: int, rank: int):
    """Expert-parallel split of a grouped (ragged) problem: contiguous groups per rank.

    Returns ``(g0, g1, row0, row1)``: this rank owns groups [g0, g1) and therefore rows [row0, row1) of the
    stacked ``A`` / ``C``.  Groups are dealt as ``shard_range`` deals batches; sizes may differ, so the row counts
    per rank differ too (ragged groups are balanced by the caller's routing, not here)."""
    sizes = [int(x) for x in batch_sizes_list]
    g0, g1 = shard_range(len(sizes), world, rank)
    row0 = sum(sizes[:g0])
    return g0, g1, row0, row0 + sum(sizes[g0:g1])


class GroupShardedW8A8:
    """Grouped W8A8 layer whose groups (experts) are split over the ranks of a process group.

    Holds this rank's ``B[g0:g1]`` and ``scale[g0:g1]``.  ``forward(A_local, scale_a_local)`` takes this rank's rows
    of the stacked activations (rows ``row0:row1`` of the global stack) and returns the matching rows of the
    output; ``gather=True`` all-gathers the (ragged) row blocks into the full ``[total_M, N]`` on every rank."""

    def __init__(self, batch_sizes_list, B: torch.Tensor, scale: torch.Tensor, out_dtype=torch.bfloat16,
                 group: Optional[dist.ProcessGroup] = None, gemm: Optional[Callable] = None,
                 metadata: Optional[Callable] = None):
        self.pg = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.sizes = [int(x) for x in batch_sizes_list]
        self.g0, self.g1, self.row0, self.row1 = shard_groups(self.sizes, self.world, self.rank)
        self.B_local = B[self.g0:self.g1].contiguous()
        self.scale_local = scale[self.g0:self.g1].contiguous() if scale.dim() == 2 else scale
        self.out_dtype = out_dtype
        if gemm is None:
            from .ops import grouped_quant_matmul as gemm
        if metadata is None:
            from .ops import build_block_metadata as metadata
        self._gemm, self._meta_fn, self._meta = gemm, metadata, None

    def to(self, device):
        self.B_local = self.B_local.to(device)
        self.scale_local = self.scale_local.to(device)
        self._meta = None
        return self

    def forward(self, A_local: torch.Tensor, scale_a_local: Optional[torch.Tensor] = None, gather: bool = False):
        if A_local.shape[0] != self.row1 - self.row0:
            raise ValueError(f"rank {self.rank} owns {self.row1 - self.row0} rows, got {A_local.shape[0]}")
        if self._meta is None or self._meta.device != A_local.device:
            self._meta = self._meta_fn(self.sizes[self.g0:self.g1], 128, A_local.device)
        C_local = self._gemm(A_local, self.B_local, self._meta, self.scale_local, scale_a_local, out_dtype=self.out_dtype)
        if not gather or self.world == 1:
            return C_local
        # ragged row blocks: pad each rank's block to the largest one, gather once, cut the padding off
        counts = [r1 - r0 for _, _, r0, r1 in (shard_groups(self.sizes, self.world, r) for r in range(self.world))]
        most, n = max(counts), C_local.shape[1]
        padded = C_local
        if C_local.shape[0] < most:
            padded = torch.zeros((most, n), dtype=C_local.dtype, device=C_local.device)
            padded[:C_local.shape[0]] = C_local
        parts = torch.empty((self.world * most, n), dtype=C_local.dtype, device=C_local.device)
        dist.all_gather_into_tensor(parts, padded, group=self.pg)
        return torch.cat([parts[r * most:r * most + c] for r, c in enumerate(counts)], dim=0)

    __call__ = forward
