"""Chunked grouped-query attention with the reference's call signature.

Mirrors ``online_chunked_grouped_attention_mx`` and its unmasked twin
(src/ollm/backends/mlx_ops.py:32-178): same arguments, same shape rules and error messages, same
conventions (absolute query positions, bottom-right alignment by default, a row with no allowed
key returns 0).  ``k`` / ``v`` are dense CUDA tensors ``[B, Hkv, Lk, D]`` or the paged views that
``PagedKVCache.update`` returns.  ``q_block_size`` / ``k_block_size`` are validated and otherwise
ignored: the kernels choose their own tiling and the result does not depend on it beyond rounding.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import lib, raise_for_status


class PagedView:
    """Handle on one layer's K or V history held in pages (what ``PagedKVCache.update`` returns
    in place of the reference's dense concatenated tensors, src/ollm/mlx_kvcache.py:125)."""

    def __init__(self, cache, layer: int, which: str):
        self.cache, self.layer, self.which = cache, layer, which

    @property
    def shape(self):
        c = self.cache
        return (c.batch_size, c.pool.cfg.num_kv_heads, c.get_seq_length(self.layer), c.pool.cfg.head_dim)

    @property
    def ndim(self):
        return 4

    @property
    def dtype(self):
        return self.cache.pool.cfg.dtype

    @property
    def itemsize(self) -> int:
        return 2 if self.dtype == torch.bfloat16 else 4

    @property
    def nbytes(self) -> int:
        """Bytes of the history this view denotes (what a dense tensor of the same shape would hold)."""
        n = self.itemsize
        for d in self.shape:
            n *= int(d)
        return n

    def materialize(self) -> torch.Tensor:
        k, v = self.cache.materialize(self.layer)
        return k if self.which == "key" else v

    def __getitem__(self, idx):
        return self.materialize()[idx]

    def __array__(self, dtype=None, copy=None):
        t = self.materialize()
        a = (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()
        return a.astype(dtype) if dtype is not None else a


def _normalize_query_positions(query_positions, batch_size: int, query_length: int):
    """``[Lq]`` / ``[1, Lq]`` -> ``[B, Lq]`` int32 (mlx_ops.py:17-29).  Host values stay on the host."""
    if isinstance(query_positions, torch.Tensor):
        pos = query_positions.to(torch.int32)
    else:
        pos = torch.as_tensor(np.asarray(query_positions).astype(np.int32))
    if pos.dim() == 1:
        pos = pos.unsqueeze(0)
    if tuple(pos.shape) == (1, query_length) and batch_size > 1:
        pos = pos.expand(batch_size, query_length)
    if tuple(pos.shape) != (batch_size, query_length):
        raise ValueError(
            "query_positions must have shape [query_length] or "
            f"[batch, query_length], got {tuple(pos.shape)}"
        )
    return pos


def chunked_grouped_attention(
    q: torch.Tensor,
    k,
    v,
    query_positions: Optional[object] = None,
    causal: bool = True,
    q_block_size: int = 32768,
    k_block_size: int = 1024,
    eps: float = 1e-12,
) -> torch.Tensor:
    if q_block_size <= 0 or k_block_size <= 0:
        raise ValueError("attention block sizes must be positive")
    if not isinstance(q, torch.Tensor) or not q.is_cuda:
        raise RuntimeError("chunked_grouped_attention needs CUDA tensors; there is no CPU path")
    if q.dim() != 4:
        raise ValueError("q must have shape [batch, heads, length, head_dim]")
    B, Hq, Lq, D = q.shape
    _, Hkv, Lk, Dk = k.shape
    if D != Dk:
        raise ValueError("q and k must share last-dim size")
    if k.shape[0] != B or v.shape[0] != B:
        raise ValueError("q, k, and v must share batch size")
    if v.shape[1] != Hkv or v.shape[2] != Lk:
        raise ValueError("k and v must share head and sequence dimensions")
    if v.shape[3] != D:
        raise ValueError("q, k, and v must share last-dim size")
    if Hkv <= 0 or Hq % Hkv != 0:
        raise ValueError("query heads must be divisible by key/value heads")
    if causal and Lk < Lq:
        raise ValueError("causal attention requires key length >= query length")
    if q.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("q must be float32 or bfloat16")

    positions = None
    if causal and query_positions is not None:
        positions = _normalize_query_positions(query_positions, B, Lq)
        if not positions.is_cuda and Lk >= Lq:
            # Host positions that equal the default arange(Lk - Lq, Lk) (what the decoder passes for every cached
            # call, llama_mlx.py:777) need no device copy at all: the kernels compute that default themselves.  A
            # pageable host-to-device copy here would also stall the host until the stream drains, once per layer.
            default = torch.arange(Lk - Lq, Lk, dtype=torch.int32)
            if bool((positions == default.unsqueeze(0)).all()):
                positions = None

    paged = isinstance(k, PagedView)
    if paged != isinstance(v, PagedView):
        raise ValueError("k and v must both be dense tensors or both be paged views")
    if paged:
        if k.cache is not v.cache or k.layer != v.layer:
            raise ValueError("k and v views must come from the same cache layer")
        cache = k.cache
        if q.dtype != cache.pool.cfg.dtype:
            raise ValueError("q must have the cache's dtype")
        if Lq == 1 and causal:
            q_pos = None if positions is None else [int(x) for x in positions.reshape(-1).tolist()]
            out = cache.pool.decode_attention(k.layer, q.reshape(B, Hq, D).contiguous(), seq_ids=cache.seq_ids,
                                              q_pos=q_pos, eps=eps)
            return out.reshape(B, Hq, 1, D)
        if Lq >= 32 and D == 128 and q.dtype == torch.bfloat16 and cache.pool.cfg.page_size % 16 != 0:
            # Long query blocks go to the tensor-core kernel.  With pages of a multiple of 16 tokens it reads the
            # pages themselves through the pool's tensor maps (the call below); other page sizes are gathered into
            # dense K/V first: O(Lk) bytes, small next to the O(Lq * Lk) attention work the tensor cores take over.
            k_dense, v_dense = cache.materialize(k.layer)
            return chunked_grouped_attention(q, k_dense, v_dense, query_positions=positions, causal=causal,
                                             q_block_size=q_block_size, k_block_size=k_block_size, eps=eps)
        return cache.pool.prefill_attention(k.layer, q, seq_ids=cache.seq_ids, positions=positions, causal=causal, eps=eps)

    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k and v must share a dtype")
    qc, kc, vc = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty_like(qc)
    pos_ptr = None
    if positions is not None:
        positions = positions.to(device=q.device, dtype=torch.int32).contiguous()
        pos_ptr = positions.data_ptr()
    st = lib.skv_attn_dense(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr(), pos_ptr, B, Hq, Hkv, Lq, Lk, D,
                            _lib.BF16 if q.dtype == torch.bfloat16 else _lib.F32, 1 if causal else 0, float(eps),
                            _dense_status_word(q.device).data_ptr(), torch.cuda.current_stream(q.device).cuda_stream)
    raise_for_status(st)
    return out


_DENSE_STATUS = {}


def _dense_status_word(device: torch.device) -> torch.Tensor:
    """One int32 per device that the dense tensor-core kernel ORs bit 8 into when a bounded wait ran out."""
    key = torch.device(device).index or 0
    word = _DENSE_STATUS.get(key)
    if word is None:
        word = _DENSE_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return word


def check_dense_attention_status(device=None) -> int:
    """Read and clear the status word of the dense attention calls made on ``device`` (synchronises it).  Raises
    DeviceFlagError when a kernel gave up on a bounded wait: the outputs of the calls since the last check are
    then not to be trusted.  The paged calls report through ``PagedPool.check_device_status`` instead."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _DENSE_STATUS.get(device.index or 0)
    if word is None:
        return 0
    flag = int(word.item())
    if flag:
        word.zero_()
        raise _lib.DeviceFlagError(f"dense attention status word 0x{flag:x} (8: a bounded wait ran out)")
    return 0


def chunked_grouped_attention_no_mask(
    q, k, v, position_ids: Optional[object] = None, q_block_size: int = 32768, k_block_size: int = 1024,
    eps: float = 1e-12,
):
    """Unmasked compatibility entry point; ``position_ids`` is accepted and ignored (mlx_ops.py:155-178)."""
    del position_ids
    return chunked_grouped_attention(q, k, v, causal=False, q_block_size=q_block_size, k_block_size=k_block_size, eps=eps)
