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


class PeerExchange:
    """Receive buffers and result buffers of the exchange that the decode merge kernel runs between GPUs.

    Every rank holds one receive buffer (two halves used alternately, by epoch parity) that all ranks can store
    into: torch symmetric memory over NVLink, peer-mapped at construction (a collective: every rank of ``group``
    must build the same object at the same point).  Rows cross as 16-byte stores whose 8-byte halves carry the
    call's epoch, so the receiving kernel validates each word by itself.  The result lands in a plain local tensor
    (``n_results`` of them in rotation, two by default, so that one can still be read while the next steps fill the
    others).  With
    ``world == 1`` ordinary device memory is used, which runs the same kernel code on one GPU.  K/V never cross
    GPUs; only output rows (or partial rows) do.
    """

    def __init__(self, mode: int, rank: int, world: int, n_seqs: int, n_q_heads: int, head_dim: int, dtype: torch.dtype,
                 device: torch.device, group: Optional[dist.ProcessGroup] = None, n_results: int = 2):
        import ctypes as C
        from . import _lib
        if n_results < 2:
            raise ValueError("an exchange needs at least two result buffers")
        self.n_results = n_results
        self.mode, self.rank, self.world = mode, rank, world
        self.n_seqs, self.n_q_heads, self.head_dim = n_seqs, n_q_heads, head_dim
        self.epoch = 0
        code = _lib.BF16 if dtype == torch.bfloat16 else _lib.F32
        nbytes = int(_lib.lib.skv_exchange_bytes(mode, world, n_seqs, n_q_heads, head_dim, code))
        if nbytes == 0:
            raise ValueError("exchange: unsupported mode, world size (1..8) or shape")
        self.out_shape = ((world, n_seqs, n_q_heads, head_dim) if mode == _lib.XCHG_HEAD_GATHER
                          else (n_seqs, n_q_heads, head_dim))
        self._outs = [torch.zeros(self.out_shape, dtype=dtype, device=device) for _ in range(n_results)]
        if world == 1:
            self.recv = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            self.recv_ptrs = [self.recv.data_ptr()]
        else:
            import os
            # plain peer mappings are all this needs: no NVLink multicast object is bound to the buffers
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm
            group = group or dist.group.WORLD
            self.recv = symm.empty(nbytes, dtype=torch.uint8, device=device)
            self.recv.zero_()
            handle = symm.rendezvous(self.recv, group.group_name)
            self.recv_ptrs = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
            torch.cuda.synchronize(device)
            dist.barrier(group=group)          # every rank's buffer is zero before anybody stores into it
        self._group = group
        # the argument block is built once: a decode step must not pay for marshalling `world` pointers
        self._ptr_arr = (C.c_void_p * world)(*self.recv_ptrs)
        self._desc = _lib.SkvExchange(mode=mode, rank=rank, world=world, epoch=0,
                                      recv_ptrs=C.cast(self._ptr_arr, C.POINTER(C.c_void_p)), out=0)
        self._out_ptrs = [t.data_ptr() for t in self._outs]

    def check(self, n_seqs: int, n_q_heads: int, head_dim: int):
        if (n_seqs, n_q_heads, head_dim) != (self.n_seqs, self.n_q_heads, self.head_dim):
            raise ValueError("exchange buffers do not match q")

    def begin(self):
        """Advance to the next epoch; returns (argument block for the library call, local result view)."""
        self.epoch += 1
        which = self.epoch % self.n_results          # the receive halves alternate by epoch parity inside the kernel
        d = self._desc
        d.epoch = self.epoch
        d.out = self._out_ptrs[which]
        return d, self._outs[which]

    def advance(self):
        """``begin`` for a caller that already holds a pointer to the argument block: returns the result view only."""
        self.epoch = e = self.epoch + 1
        which = e % self.n_results
        d = self._desc
        d.epoch = e
        d.out = self._out_ptrs[which]
        return self._outs[which]

    def close(self):
        """Collective: all ranks stop using the buffers before any rank lets go of its own."""
        if self.world > 1 and self.recv is not None:
            torch.cuda.synchronize(self.recv.device)
            dist.barrier(group=self._group)
        self.recv = None
        self._handle = None


class PeerGather(PeerExchange):
    """Output all-gather of KV-head sharding, fused into the merge kernel: result ``[world, n_seqs, local_q_heads,
    head_dim]``; slot r holds rank r's query heads (concatenating the slots along the head axis restores the
    reference's head order, src/ollm/backends/mlx_ops.py:152)."""

    def __init__(self, shard: HeadShard, n_seqs: int, head_dim: int, dtype: torch.dtype, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, n_results: int = 2):
        from . import _lib
        super().__init__(_lib.XCHG_HEAD_GATHER, shard.rank, shard.world, n_seqs, shard.local_q_heads, head_dim, dtype, device, group,
                         n_results)
        self.shard = shard
        self.shape = self.out_shape


class PeerSeqMerge(PeerExchange):
    """Cross-rank merge of sequence sharding, fused into the merge kernel: each rank's un-normalised partial row goes
    to the row's owner, the owner applies the reference's chunk-merge rule (mlx_ops.py:125-146) and sends the
    finished row to everyone; result ``[n_seqs, q_heads, head_dim]``, identical on all ranks."""

    def __init__(self, rank: int, world: int, n_seqs: int, n_q_heads: int, head_dim: int, dtype: torch.dtype,
                 device: torch.device, group: Optional[dist.ProcessGroup] = None, n_results: int = 2):
        from . import _lib
        super().__init__(_lib.XCHG_SEQ_MERGE, rank, world, n_seqs, n_q_heads, head_dim, dtype, device, group, n_results)


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


@dataclass(frozen=True)
class InterleavedShard:
    """Round-robin split of every sequence's tokens over the ranks in blocks of ``block`` tokens (a multiple of the
    page size): block j of a sequence lives on rank ``j % world``.  Unlike the contiguous split it balances ragged
    batches (a short sequence is spread over all ranks too).  A rank keeps its tokens in their global order, so the
    keys a query at position p may see are the first ``local_count(p + 1)`` tokens of the rank."""

    rank: int
    world: int
    block: int = 16
    page_size: int = 16

    def __post_init__(self):
        if self.world <= 0 or not 0 <= self.rank < self.world:
            raise ValueError("rank must lie in [0, world)")
        if self.block <= 0 or self.block % self.page_size:
            raise ValueError("block must be a positive multiple of the page size")

    def owner(self, position: int) -> int:
        return (position // self.block) % self.world

    def local_count(self, length: int, rank: Optional[int] = None) -> int:
        """Tokens among global positions [0, length) that live on ``rank`` (default: this rank)."""
        r = self.rank if rank is None else rank
        cycle = self.block * self.world
        full, rest = divmod(length, cycle)
        return full * self.block + min(max(rest - r * self.block, 0), self.block)

    def local_range(self, length: int):
        return None, self.local_count(length)

    def local_position(self, position: int) -> int:
        """A global query position as the index of the last local key it may see (-1: none)."""
        return self.local_count(position + 1) - 1

    def global_positions(self, length: int):
        """Global positions of this rank's tokens of a sequence of ``length`` tokens, in local order."""
        out = []
        cycle = self.block * self.world
        start = self.rank * self.block
        while start < length:
            out.extend(range(start, min(start + self.block, length)))
            start += cycle
        return out


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
