"""KV-head sharding across GPUs (one process per GPU).

The reference is single-device; its attention is independent per KV head (it loops over them,
src/ollm/backends/mlx_ops.py:81-87, and concatenates on the head axis, :152), so rank r keeps KV heads
[r * Hkv / N, (r + 1) * Hkv / N) with their query heads and pages, and the only exchange is an all-gather
of the attention outputs.  K/V never cross GPUs; page tables and lengths are identical on every rank
because every rank issues the same cache calls.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    n_q_heads: int
    n_kv_heads: int

    def __post_init__(self):
        if self.world <= 0 or not 0 <= self.rank < self.world:
            raise ValueError("rank must lie in [0, world)")
        if self.n_kv_heads <= 0 or self.n_q_heads % self.n_kv_heads:
            raise ValueError("query heads must be divisible by key/value heads")
        if self.n_kv_heads % self.world:
            raise ValueError(f"KV-head sharding needs num_kv_heads ({self.n_kv_heads}) divisible by the world size ({self.world})")

    @property
    def local_kv_heads(self) -> int:
        return self.n_kv_heads // self.world

    @property
    def local_q_heads(self) -> int:
        return self.n_q_heads // self.world

    @property
    def kv_slice(self) -> slice:
        return slice(self.rank * self.local_kv_heads, (self.rank + 1) * self.local_kv_heads)

    @property
    def q_slice(self) -> slice:
        return slice(self.rank * self.local_q_heads, (self.rank + 1) * self.local_q_heads)

    def take_q(self, x: torch.Tensor, head_dim: int = 1) -> torch.Tensor:
        """This rank's query heads of a tensor whose `head_dim` axis holds all query heads."""
        return x.narrow(head_dim, self.q_slice.start, self.local_q_heads)

    def take_kv(self, x: torch.Tensor, head_dim: int = 1) -> torch.Tensor:
        return x.narrow(head_dim, self.kv_slice.start, self.local_kv_heads)


def gather_head_outputs(out_local: torch.Tensor, shard: HeadShard, group: Optional[dist.ProcessGroup] = None,
                        buffer: Optional[torch.Tensor] = None, head_dim: int = 1) -> torch.Tensor:
    """All-gather per-rank outputs (`head_dim` axis = local query heads) into the full head axis.

    Query head h lives on rank h // local_q_heads, so concatenating the ranks' slices along the head axis in
    rank order restores the reference's head order (mlx_ops.py:152).  `buffer` ([world, *out_local.shape])
    avoids an allocation per step.
    """
    if shard.world == 1:
        return out_local
    out_local = out_local.contiguous()
    if buffer is None:
        buffer = torch.empty((shard.world,) + tuple(out_local.shape), dtype=out_local.dtype, device=out_local.device)
    # dim-0 concatenation of the ranks' tensors: the one output form every backend (NCCL, gloo) accepts
    dist.all_gather_into_tensor(buffer.view((-1,) + tuple(out_local.shape[1:])), out_local, group=group)
    # [world, ..., local_heads, ...] -> [..., world * local_heads, ...]
    moved = buffer.movedim(0, head_dim)                       # [..., world, local_heads, ...]
    shape = list(out_local.shape)
    shape[head_dim] = shard.world * shape[head_dim]
    return moved.reshape(shape)


class PeerGather:
    """Buffers for the output gather that is fused into the decode merge kernel.

    Every rank holds two gathered buffers ``[world, n_seqs, local_q_heads, head_dim]`` (used alternately) and
    a flag array ``[world]``; all of them are peer-mapped (torch symmetric memory over NVLink), so a rank's
    merge kernel can store its rows straight into every rank's buffer and raise its flag there.  With
    ``world == 1`` plain device tensors are used, which exercises the same kernel path on one GPU.
    K/V never cross GPUs; only the outputs do.
    """

    def __init__(self, shard: HeadShard, n_seqs: int, head_dim: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None):
        self.shard = shard
        self.shape = (shard.world, n_seqs, shard.local_q_heads, head_dim)
        self.epoch = 0
        esize = torch.empty((), dtype=dtype).element_size()
        self.slab_bytes = int(torch.Size(self.shape).numel()) * esize
        if shard.world == 1:
            self.buf = torch.zeros((2,) + self.shape, dtype=dtype, device=device)
            self.flags = torch.zeros((1,), dtype=torch.int32, device=device)
            self.buf_ptrs = [self.buf.data_ptr()]
            self.flag_ptrs = [self.flags.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm
            group = group or dist.group.WORLD
            self.buf = symm.empty((2,) + self.shape, dtype=dtype, device=device)
            self.flags = symm.empty((shard.world,), dtype=torch.int32, device=device)
            self.buf.zero_()
            self.flags.zero_()
            hb = symm.rendezvous(self.buf, group.group_name)
            hf = symm.rendezvous(self.flags, group.group_name)
            self.buf_ptrs = [int(p) for p in hb.buffer_ptrs]
            self.flag_ptrs = [int(p) for p in hf.buffer_ptrs]
            self._handles = (hb, hf)
            torch.cuda.synchronize(device)
            dist.barrier(group=group)

    def _descriptors(self):
        # the two argument blocks (one per buffer parity) are built once: a decode step must not pay for
        # marshalling 2 x world pointers every time
        import ctypes as C
        from . import _lib
        if not hasattr(self, "_desc"):
            world = self.shard.world
            self._keep, self._desc = [], []
            flag_arr = (C.c_void_p * world)(*self.flag_ptrs)
            for parity in (0, 1):
                out_arr = (C.c_void_p * world)(*[p + parity * self.slab_bytes for p in self.buf_ptrs])
                d = _lib.SkvPeerGather(rank=self.shard.rank, world=world, epoch=0,
                                       out_ptrs=C.cast(out_arr, C.POINTER(C.c_void_p)),
                                       flag_ptrs=C.cast(flag_arr, C.POINTER(C.c_void_p)), wait_flags=self.flags.data_ptr())
                self._keep.append((out_arr, flag_arr))
                self._desc.append(d)
            self._views = [self.buf[0], self.buf[1]]
        return self._desc

    def begin(self, wait: bool = True):
        """Advance to the next epoch; returns (argument block for the library call, local gathered view)."""
        desc = self._descriptors()
        self.epoch += 1
        parity = self.epoch & 1
        d = desc[parity]
        d.epoch = self.epoch
        d.wait_flags = self.flags.data_ptr() if wait else None
        return d, self._views[parity]


@dataclass(frozen=True)
class SequenceShard:
    """Contiguous, page-aligned split of every sequence's tokens over the ranks: rank r holds tokens
    ``[r * span, (r + 1) * span)`` of each sequence, ``span`` a multiple of the page size.  Attention is
    associative along the key axis through the reference's (max, sum, weighted-V) merge
    (src/ollm/backends/mlx_ops.py:125-144), so every rank attends its own keys and the un-normalised partials
    are merged after one all-gather."""

    rank: int
    world: int
    span: int            # tokens per rank per sequence
    page_size: int = 16

    def __post_init__(self):
        if self.world <= 0 or not 0 <= self.rank < self.world:
            raise ValueError("rank must lie in [0, world)")
        if self.span <= 0 or self.span % self.page_size:
            raise ValueError("span must be a positive multiple of the page size")

    def owner(self, position: int) -> int:
        """Rank that stores the token at a global position (the last rank also takes everything beyond)."""
        return min(position // self.span, self.world - 1)

    def local_range(self, length: int):
        """(first global position, number of tokens) this rank holds of a sequence of ``length`` tokens."""
        start = self.rank * self.span
        end = length if self.rank == self.world - 1 else min(length, start + self.span)
        return start, max(0, end - start)

    def local_position(self, position: int) -> int:
        """A global query position in this rank's own token numbering (negative: none of its keys are allowed)."""
        return position - self.rank * self.span


def sequence_sharded_decode(pool, layer: int, q: torch.Tensor, q_pos_global, seq_shard: SequenceShard, *,
                            group: Optional[dist.ProcessGroup] = None, eps: float = 1e-12) -> torch.Tensor:
    """Decode attention when each rank's pool holds a token range of every sequence: local partial, all-gather
    of the float32 partials (``[n_seqs, q_heads, head_dim + 2]`` per rank), merge on every rank."""
    from .pool import merge_partials
    local = pool.decode_partial(layer, q, q_pos=[seq_shard.local_position(int(p)) for p in q_pos_global])
    if seq_shard.world == 1:
        parts = local.unsqueeze(0)
    else:
        parts = torch.empty((seq_shard.world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(parts.view((-1,) + tuple(local.shape[1:])), local, group=group)
    return merge_partials(parts, eps=eps, dtype=q.dtype)
