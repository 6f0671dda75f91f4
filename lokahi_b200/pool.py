"""PagedPool: Python handle on one skv_pool (page allocator, page tables, lengths, device pages).

Thin by design: argument marshalling and status -> exception mapping only.  All bookkeeping lives in
the C++ pool, all arithmetic in the CUDA kernels.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib
from ._lib import lib, raise_for_status, i32_array


@dataclass(frozen=True)
class PagedKVConfig:
    """Frozen, validated pool geometry (mirrors the reference's frozen policy dataclasses,
    e.g. src/ollm/core/ssd_offload.py:19-52)."""

    num_layers: int
    num_kv_heads: int
    head_dim: int
    num_pages: int
    max_seqs: int
    max_pages_per_seq: int
    page_size: int = 16
    dtype: torch.dtype = torch.bfloat16
    device: int = 0            # CUDA ordinal, or -1 for a bookkeeping-only pool (no device memory)
    host_pages: int = 0
    rope_theta: Optional[float] = None
    rope_scaling_factor: float = 1.0

    def __post_init__(self):
        for name in ("num_layers", "num_kv_heads", "head_dim", "num_pages", "max_seqs", "max_pages_per_seq", "page_size"):
            if not isinstance(getattr(self, name), int) or getattr(self, name) <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if self.host_pages < 0:
            raise ValueError("host_pages must be non-negative")
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("dtype must be torch.float32 or torch.bfloat16")
        if self.head_dim % 2:
            raise ValueError("head_dim must be even")
        if not self.rope_scaling_factor > 0:
            raise ValueError("rope_scaling_factor must be positive")


def rope_inv_freq(dim: int, base: float) -> np.ndarray:
    """float32 ``1 / base ** (arange(0, dim, 2) / dim)`` as MLXRotaryEmbedding builds it
    (src/ollm/llama_mlx.py:111-114)."""
    exponent = np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)
    return (np.float32(1.0) / np.power(np.float32(base), exponent, dtype=np.float32)).astype(np.float32)


def _stream_ptr(device_index: int) -> int:
    return torch.cuda.current_stream(device_index).cuda_stream


class PagedPool:
    def __init__(self, cfg: PagedKVConfig):
        self.cfg = cfg
        self._h = C.c_void_p()
        self.esize = 2 if cfg.dtype == torch.bfloat16 else 4
        c = _lib.SkvConfig(
            device=cfg.device, dtype=_lib.BF16 if cfg.dtype == torch.bfloat16 else _lib.F32,
            num_layers=cfg.num_layers, num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
            page_size=cfg.page_size, num_pages=cfg.num_pages, max_seqs=cfg.max_seqs,
            max_pages_per_seq=cfg.max_pages_per_seq, host_pages=cfg.host_pages)
        if cfg.device >= 0 and not torch.cuda.is_available():
            raise RuntimeError("PagedPool needs a CUDA device; there is no CPU path (device=-1 is bookkeeping only)")
        st = lib.skv_create(C.byref(c), C.byref(self._h))
        if st != _lib.OK:
            h, self._h = self._h, C.c_void_p()
            try:
                raise_for_status(st, h)
            finally:
                if h:
                    lib.skv_destroy(h)
        self._workspaces = {}
        self._inv_freq_dev = None
        if cfg.rope_theta is not None:
            self.set_rope(rope_inv_freq(cfg.head_dim, cfg.rope_theta), cfg.rope_scaling_factor)

    # -- life cycle -------------------------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            lib.skv_destroy(self._h)
            self._h = C.c_void_p()
            self._workspaces = {}

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, st):
        raise_for_status(st, self._h)

    @property
    def stream(self) -> int:
        return 0 if self.cfg.device < 0 else _stream_ptr(self.cfg.device)

    @property
    def torch_device(self) -> torch.device:
        return torch.device("cuda", self.cfg.device)

    # -- sequences ----------------------------------------------------------------------------
    def alloc_sequence(self) -> int:
        out = C.c_int32()
        self._check(lib.skv_alloc_sequence(self._h, C.byref(out)))
        return out.value

    # The next three publish their change to the device copy of the tables on the current stream of the pool's
    # device, like every compute call, so a pool driven from a side stream stays ordered.
    def free_sequence(self, seq: int):
        self._check(lib.skv_free_sequence(self._h, seq, self.stream))

    def reserve(self, seq: int, total_tokens: int):
        self._check(lib.skv_reserve(self._h, seq, total_tokens, self.stream))

    def set_page_table(self, seq: int, pages: Sequence[int], length: int):
        arr = i32_array(pages)
        self._check(lib.skv_set_page_table(self._h, seq, arr, len(arr), length, self.stream))

    def truncate(self, layer: int, new_length: int, seq_ids=None, n_seqs: Optional[int] = None):
        """Shorten a layer's history of the given sequences to ``new_length`` tokens (pages are kept)."""
        ids = i32_array(seq_ids)
        n = len(ids) if ids is not None else n_seqs
        self._check(lib.skv_truncate(self._h, layer, ids, n, new_length, self.stream))

    def length(self, layer: int, seq: int) -> int:
        out = C.c_int32()
        self._check(lib.skv_length(self._h, layer, seq, C.byref(out)))
        return out.value

    def lengths(self, layer: int, n: Optional[int] = None) -> np.ndarray:
        n = self.cfg.max_seqs if n is None else n
        out = (C.c_int32 * n)()
        self._check(lib.skv_lengths(self._h, layer, out, n))
        return np.frombuffer(out, dtype=np.int32).copy()

    def page_table(self, seq: int) -> np.ndarray:
        out = (C.c_int32 * self.cfg.max_pages_per_seq)()
        n = C.c_int32()
        self._check(lib.skv_page_table(self._h, seq, out, self.cfg.max_pages_per_seq, C.byref(n)))
        return np.frombuffer(out, dtype=np.int32)[: n.value].copy()

    def counters(self) -> dict:
        out = (C.c_int64 * 8)()
        self._check(lib.skv_pool_counters(self._h, out))
        names = ("free_pages", "used_pages", "free_host_slots", "pages_evicted", "pages_prefetched",
                 "bytes_d2h", "bytes_h2d", "live_sequences")
        return dict(zip(names, [int(x) for x in out]))

    # -- raw views ------------------------------------------------------------------------------
    def layer_views(self, layer: int):
        """(K, V) torch views ``[num_pages, kv_heads, page_size, head_dim]`` aliasing the device pools."""
        k, v = C.c_void_p(), C.c_void_p()
        self._check(lib.skv_pool_pointers(self._h, layer, C.byref(k), C.byref(v)))
        c = self.cfg
        shape = (c.num_pages, c.num_kv_heads, c.page_size, c.head_dim)
        return _alias(k.value, shape, c.dtype, c.device), _alias(v.value, shape, c.dtype, c.device)

    # -- RoPE -------------------------------------------------------------------------------------
    def set_rope(self, inv_freq: np.ndarray, scaling_factor: float = 1.0):
        inv = np.ascontiguousarray(inv_freq, dtype=np.float32)
        self._check(lib.skv_set_rope(self._h, inv.ctypes.data_as(C.POINTER(C.c_float)), inv.size, float(scaling_factor)))
        self.inv_freq = inv
        self.rope_scaling = float(scaling_factor)
        if self.cfg.device >= 0:
            self._inv_freq_dev = torch.from_numpy(inv).to(self.torch_device)

    # -- K1 -----------------------------------------------------------------------------------------
    def append(self, layer: int, k: Optional[torch.Tensor], v: Optional[torch.Tensor], *, n_new: Optional[int] = None,
               seq_ids=None, start_pos=None, rope_k: bool = False, q: Optional[torch.Tensor] = None,
               layout: str = "bhld"):
        """Append tokens of ``k``/``v`` to a layer.

        ``layout`` "bhld": ``[n_seqs, kv_heads, n_new, head_dim]`` (the reference's update layout);
        "bhd": ``[n_seqs, kv_heads, head_dim]`` (one token per sequence).  ``q`` (same layout, query
        heads) is rotated in place when given.  Any strides are accepted as long as head_dim is contiguous.
        """
        a = _lib.SkvAppendArgs()
        a.layer = layer
        if k is None:   # bookkeeping-only pools
            if n_new is None or (seq_ids is None and start_pos is None):
                raise ValueError("n_new and seq_ids or start_pos are needed without tensors")
            n_seqs = len(seq_ids) if seq_ids is not None else len(start_pos)
        else:
            self._check_tensor(k, "k")
            self._check_tensor(v, "v")
            if k.shape != v.shape:
                raise ValueError("key and value states must have identical shapes")
            n_seqs = k.shape[0]
            if layout == "bhld":
                if k.dim() != 4:
                    raise ValueError("key and value states must have rank 4")
                n_new = k.shape[2]
                a.kv_stride_seq, a.kv_stride_head, a.kv_stride_tok = k.stride(0), k.stride(1), k.stride(2)
                vs = (v.stride(0), v.stride(1), v.stride(2))
            elif layout == "bhd":
                if k.dim() != 3:
                    raise ValueError("layout 'bhd' needs rank-3 tensors")
                n_new = 1
                a.kv_stride_seq, a.kv_stride_head, a.kv_stride_tok = k.stride(0), k.stride(1), 0
                vs = (v.stride(0), v.stride(1), 0)
            else:
                raise ValueError(f"unknown layout {layout!r}")
            if vs != (a.kv_stride_seq, a.kv_stride_head, a.kv_stride_tok):
                v = v.contiguous()
                k = k.contiguous()
                a.kv_stride_seq, a.kv_stride_head = k.stride(0), k.stride(1)
                a.kv_stride_tok = k.stride(2) if layout == "bhld" else 0
            if k.shape[1] != self.cfg.num_kv_heads or k.shape[-1] != self.cfg.head_dim:
                raise ValueError("new key states must match cached batch, head, and feature dimensions")
            a.k, a.v = k.data_ptr(), v.data_ptr()
        a.n_seqs, a.n_new = n_seqs, n_new
        ids = i32_array(seq_ids)
        starts = i32_array(start_pos)
        a.seq_ids = ids if ids is not None else None
        a.start_pos = starts if starts is not None else None
        a.rope_k = 1 if rope_k else 0
        if q is not None:
            self._check_tensor(q, "q")
            if q.shape[0] != n_seqs or q.shape[-1] != self.cfg.head_dim:
                raise ValueError("q must match the batch and head_dim of k")
            a.q_in = a.q_out = q.data_ptr()
            a.n_q_heads = q.shape[1]
            a.q_stride_seq, a.q_stride_head = q.stride(0), q.stride(1)
            a.q_stride_tok = q.stride(2) if layout == "bhld" else 0
        self._check(lib.skv_append(self._h, C.byref(a), self.stream))

    def _check_tensor(self, t: torch.Tensor, name: str):
        if not t.is_cuda or t.device.index != self.cfg.device:
            raise ValueError(f"{name} must live on cuda:{self.cfg.device}")
        if t.dtype != self.cfg.dtype:
            raise ValueError(f"{name} has dtype {t.dtype}, pool stores {self.cfg.dtype}")
        if t.stride(-1) != 1:
            raise ValueError(f"{name} must be contiguous along head_dim")

    # -- K2 -------------------------------------------------------------------------------------------
    def gather(self, layer: int, seq_ids=None, n_seqs: Optional[int] = None, max_len: Optional[int] = None):
        """Dense ``[n_seqs, kv_heads, max_len, head_dim]`` K and V of a layer."""
        ids = i32_array(seq_ids)
        n_seqs = len(ids) if ids is not None else n_seqs
        if n_seqs is None:
            raise ValueError("seq_ids or n_seqs is needed")
        if max_len is None:
            lens = self.lengths(layer)
            max_len = int(max(lens[s] for s in (seq_ids if seq_ids is not None else range(n_seqs))))
        c = self.cfg
        k = torch.empty((n_seqs, c.num_kv_heads, max_len, c.head_dim), dtype=c.dtype, device=self.torch_device)
        v = torch.empty_like(k)
        self._check(lib.skv_gather(self._h, layer, ids, n_seqs, k.data_ptr(), v.data_ptr(), max_len, self.stream))
        return k, v

    # -- K3 -------------------------------------------------------------------------------------------
    def workspace(self, n_seqs: int, n_q_heads: int) -> torch.Tensor:
        key = (n_seqs, n_q_heads)
        ws = self._workspaces.get(key)
        if ws is None:
            nbytes = lib.skv_decode_workspace_bytes(self._h, n_seqs, n_q_heads)
            ws = torch.empty(nbytes, dtype=torch.uint8, device=self.torch_device)
            self._workspaces[key] = ws
        return ws

    def decode_attention(self, layer: int, q: torch.Tensor, *, seq_ids=None, q_pos=None, eps: float = 1e-12,
                         out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``q`` ``[n_seqs, q_heads, head_dim]`` -> output of the same shape."""
        self._check_tensor(q, "q")
        if q.dim() != 3 or not q.is_contiguous():
            raise ValueError("q must be a contiguous [n_seqs, q_heads, head_dim] tensor")
        n_seqs, hq, _ = q.shape
        if out is None:
            out = torch.empty_like(q)
        ws = self.workspace(n_seqs, hq)
        self._check(lib.skv_decode_attn(self._h, layer, i32_array(seq_ids), n_seqs, q.data_ptr(), out.data_ptr(),
                                        i32_array(q_pos), hq, float(eps), ws.data_ptr(), ws.numel(), self.stream))
        return out

    def decode_attention_xchg(self, layer: int, q: torch.Tensor, exchange, *, seq_ids=None, q_pos=None,
                              eps: float = 1e-12) -> torch.Tensor:
        """``decode_attention`` with the exchange between GPUs fused into the merge kernel (``exchange`` is a
        ``sharding.PeerGather`` under KV-head sharding or a ``sharding.PeerSeqMerge`` under sequence sharding).
        Returns the exchange's local result view, complete for anything enqueued after the call."""
        self._check_tensor(q, "q")
        if q.dim() != 3 or not q.is_contiguous():
            raise ValueError("q must be a contiguous [n_seqs, q_heads, head_dim] tensor")
        n_seqs, hq, _ = q.shape
        exchange.check(n_seqs, hq, self.cfg.head_dim)
        desc, view = exchange.begin()
        ws = self.workspace(n_seqs, hq)
        self._check(lib.skv_decode_attn_xchg(self._h, layer, i32_array(seq_ids), n_seqs, q.data_ptr(), i32_array(q_pos), hq,
                                             float(eps), ws.data_ptr(), ws.numel(), C.byref(desc), self.stream))
        return view

    decode_attention_gather = decode_attention_xchg

    def decode_partial(self, layer: int, q: torch.Tensor, *, seq_ids=None, q_pos=None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Attention of ``q`` ``[n_seqs, q_heads, head_dim]`` over the keys this pool holds, as un-normalised
        float32 rows ``[n_seqs, q_heads, head_dim + 2]`` = (weighted V sum, max, sum): the unit that
        ``merge_partials`` combines across key ranges (sequence sharding)."""
        self._check_tensor(q, "q")
        if q.dim() != 3 or not q.is_contiguous():
            raise ValueError("q must be a contiguous [n_seqs, q_heads, head_dim] tensor")
        n_seqs, hq, d = q.shape
        if out is None:
            out = torch.empty((n_seqs, hq, d + 2), dtype=torch.float32, device=q.device)
        ws = self.workspace(n_seqs, hq)
        self._check(lib.skv_decode_partial(self._h, layer, i32_array(seq_ids), n_seqs, q.data_ptr(), i32_array(q_pos), hq,
                                           ws.data_ptr(), ws.numel(), out.data_ptr(), self.stream))
        return out

    def _step_args(self, q, k, v, out, seq_ids, eps, exchange, positions, store, consecutive):
        """Checked argument block of ``skv_decode_step_ex``; returns (block, objects that must outlive the call)."""
        for name, t in (("q", q), ("k", k), ("v", v)) + ((("out", out),) if out is not None else ()):
            self._check_tensor(t, name)
            if t.dim() != 3 or t.stride(2) != 1 or t.stride(1) != t.shape[2]:
                raise ValueError(f"{name} must be [n_seqs, heads, head_dim] with the heads of a row packed")
        n_seqs, hq, _ = q.shape
        if k.shape != (n_seqs, self.cfg.num_kv_heads, self.cfg.head_dim) or v.shape != k.shape:
            raise ValueError("new key states must match cached batch, head, and feature dimensions")
        if out is not None and out.shape != q.shape:
            raise ValueError("out must have q's shape")
        a = _lib.SkvStepArgs()
        keep = []
        a.n_seqs, a.n_q_heads, a.eps = n_seqs, hq, float(eps)
        a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
        a.q_row_stride, a.k_row_stride, a.v_row_stride = q.stride(0), k.stride(0), v.stride(0)
        if out is not None:
            a.out, a.out_row_stride = out.data_ptr(), out.stride(0)
        if seq_ids is not None:
            ids = i32_array(seq_ids)
            if len(ids) != n_seqs:
                raise ValueError("seq_ids must have one entry per row of q")
            a.seq_ids = ids
            keep.append(ids)
        if (positions is None) != (store is None):
            raise ValueError("positions and store are given together or not at all")
        if positions is not None:
            pos = i32_array(positions)
            st = (C.c_uint8 * n_seqs)(*[1 if x else 0 for x in store])
            if len(pos) != n_seqs:
                raise ValueError("positions must have one entry per row of q")
            a.positions, a.store = pos, st
            keep += [pos, st]
        ws = self.workspace(n_seqs, hq)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        a.flags = _lib.STEP_CONSECUTIVE if consecutive else 0
        if exchange is not None:
            exchange.check(n_seqs, hq, self.cfg.head_dim)
        return a, keep

    def decode_step(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, eps: float = 1e-12,
                    out: Optional[torch.Tensor] = None, seq_ids=None, exchange=None, positions=None, store=None,
                    consecutive: bool = False, partial: bool = False) -> torch.Tensor:
        """RoPE-on-write append of one token per sequence plus decode attention in one library call.
        ``q`` ``[n_seqs, q_heads, head_dim]`` is rotated in place; ``k``, ``v`` ``[n_seqs, kv_heads, head_dim]``; rows
        may be strided slices of one fused projection output as long as the heads of a row are packed.  The
        sequences are ``seq_ids`` (distinct; default 0..n_seqs-1) and the token goes to each one's current length.
        ``exchange`` (``sharding.PeerGather`` / ``PeerSeqMerge``) fuses the exchange between GPUs into the merge
        kernel and the call returns its local result view.  ``positions`` / ``store``: sequence sharding (the
        token's absolute position per row, and whether this pool keeps it).  ``consecutive=True`` states that
        nothing was enqueued on the stream since this pool's previous step and that q, k, v were complete before
        it: the step then overlaps the previous step's merge kernel (see ``skv_step_args`` in the header).
        ``partial=True`` returns un-normalised float32 rows ``[n_seqs, q_heads, head_dim + 2]`` (what ``decode_partial``
        writes) instead of the output, for a merge done elsewhere."""
        if partial:
            if exchange is not None:
                raise ValueError("partial and exchange exclude each other")
            part = torch.empty((q.shape[0], q.shape[1], q.shape[2] + 2), dtype=torch.float32, device=q.device)
        elif out is None and exchange is None:
            out = torch.empty_like(q)
        a, keep = self._step_args(q, k, v, None if (exchange is not None or partial) else out, seq_ids, eps, exchange,
                                  positions, store, consecutive)
        a.layer = layer
        view = out
        if partial:
            a.partial_out = part.data_ptr()
            view = part
        if exchange is not None:
            desc, view = exchange.begin()
            a.xchg = C.pointer(desc)
        self._check(lib.skv_decode_step_ex(self._h, C.byref(a), self.stream))
        del keep
        return view

    def decode_step_binder(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None, *,
                           seq_ids=None, eps: float = 1e-12, exchange=None, positions=None, store=None,
                           consecutive: bool = False):
        """``decode_step`` for buffers that stay put (the static tensors of a CUDA graph, the buffers of a decode
        loop): the tensors are checked once, here, and the returned ``call(layer, stream)`` only makes the
        library call (with an exchange it returns the step's result view).  The caller keeps the tensors alive and
        unchanged in shape for as long as it uses the callable."""
        if out is None and exchange is None:
            raise ValueError("out or exchange is needed")
        a, keep = self._step_args(q, k, v, None if exchange is not None else out, seq_ids, eps, exchange, positions, store,
                                  consecutive)
        h, fn, ref = self._h, lib.skv_decode_step_ex, C.byref(a)
        if exchange is None:
            def call(layer: int, stream: int):
                a.layer = layer
                st = fn(h, ref, stream)
                if st:
                    raise_for_status(st, h)
                return out
        else:
            advance = exchange.advance
            a.xchg = C.pointer(exchange._desc)          # the one argument block of the exchange, updated in place per call

            def call(layer: int, stream: int):
                a.layer = layer
                view = advance()
                st = fn(h, ref, stream)
                if st:
                    raise_for_status(st, h)
                return view
        call._keep = (a, keep, q, k, v, out)
        return call

    def decode_step_gather(self, layer: int, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, gather, *,
                           eps: float = 1e-12, seq_ids=None, consecutive: bool = False) -> torch.Tensor:
        """``decode_step`` under KV-head sharding: append, attend and the output gather in one library call.
        Returns this rank's gathered view ``[world, n_seqs, local_q_heads, head_dim]``."""
        return self.decode_step(layer, q, k, v, eps=eps, seq_ids=seq_ids, exchange=gather, consecutive=consecutive)

    def decode_attention_static(self, layer: int, q: torch.Tensor, *, seq_ids=None, q_pos=None, eps: float = 1e-12,
                                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``decode_attention`` for callers that may not allocate device memory: the split-K partials
        go to a 16 MiB array built into the library instead of a workspace tensor, so this wrapper
        creates nothing but (optionally) the output.  Pass ``out`` to allocate nothing at all.
        Raises NotImplementedError when the partials would not fit; calls on one device share the
        array and must not overlap on the GPU."""
        self._check_tensor(q, "q")
        if q.dim() != 3 or not q.is_contiguous():
            raise ValueError("q must be a contiguous [n_seqs, q_heads, head_dim] tensor")
        n_seqs, hq, _ = q.shape
        if out is None:
            out = torch.empty_like(q)
        self._check(lib.skv_decode_attn_static(self._h, layer, i32_array(seq_ids), n_seqs, q.data_ptr(), out.data_ptr(),
                                               i32_array(q_pos), hq, float(eps), self.stream))
        return out

    # -- K4 over pages ------------------------------------------------------------------------------------
    def prefill_attention(self, layer: int, q: torch.Tensor, *, seq_ids=None, positions: Optional[torch.Tensor] = None,
                          causal: bool = True, eps: float = 1e-12) -> torch.Tensor:
        """``q`` ``[n_seqs, q_heads, Lq, head_dim]`` against each sequence's cached tokens."""
        self._check_tensor(q, "q")
        q = q.contiguous()
        n_seqs, hq, lq, _ = q.shape
        out = torch.empty_like(q)
        pos_ptr = None
        if positions is not None:
            positions = positions.to(device=self.torch_device, dtype=torch.int32).contiguous()
            pos_ptr = positions.data_ptr()
        self._check(lib.skv_prefill_attn_paged(self._h, layer, i32_array(seq_ids), n_seqs, q.data_ptr(), out.data_ptr(),
                                               pos_ptr, hq, lq, 1 if causal else 0, float(eps), self.stream))
        return out

    # -- K5 ---------------------------------------------------------------------------------------------------
    def evict(self, seq: int, first_slot: int, n_slots: int):
        self._check(lib.skv_evict(self._h, seq, first_slot, n_slots, self.stream))

    def prefetch(self, seq: int, first_slot: int, n_slots: int):
        self._check(lib.skv_prefetch(self._h, seq, first_slot, n_slots, self.stream))

    def sync_transfers(self):
        self._check(lib.skv_sync_transfers(self._h, self.stream))

    def wait_resident(self, timeout_ms: int = 10000):
        self._check(lib.skv_wait_resident(self._h, timeout_ms))

    def transfers_done(self) -> bool:
        """True when the copy stream has drained (a poll: never blocks)."""
        try:
            self.wait_resident(0)
            return True
        except TimeoutError:
            return False

    def check_device_status(self) -> int:
        flag = C.c_int32()
        self._check(lib.skv_check_device_status(self._h, self.stream, C.byref(flag)))
        return flag.value


def _alias(ptr: int, shape, dtype: torch.dtype, device: int) -> torch.Tensor:
    """Torch tensor aliasing device memory owned by the library (no copy, no ownership)."""
    esize = 2 if dtype == torch.bfloat16 else 4
    n = int(np.prod(shape))

    class _Mem:
        __cuda_array_interface__ = {
            "shape": (n * esize,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }

    raw = torch.as_tensor(_Mem(), device=torch.device("cuda", device))
    return raw.view(dtype).view(*shape)


def merge_partials(parts: torch.Tensor, *, eps: float = 1e-12, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Merge ``parts`` ``[n_parts, n_seqs, q_heads, head_dim + 2]`` (float32 rows from ``decode_partial``, one per key
    range) into the attention output ``[n_seqs, q_heads, head_dim]`` with the reference's chunk-merge rule
    (src/ollm/backends/mlx_ops.py:125-146)."""
    if not parts.is_cuda:
        raise RuntimeError("merge_partials needs a CUDA tensor; there is no CPU path")
    if parts.dim() != 4 or parts.dtype != torch.float32 or not parts.is_contiguous():
        raise ValueError("parts must be a contiguous float32 [n_parts, n_seqs, q_heads, head_dim + 2] tensor")
    n_parts, n_seqs, hq, d2 = parts.shape
    out = torch.empty((n_seqs, hq, d2 - 2), dtype=dtype, device=parts.device)
    st = lib.skv_merge_partials(parts.data_ptr(), n_parts, n_seqs * hq * d2, n_seqs * hq, d2 - 2, float(eps), out.data_ptr(),
                                _lib.BF16 if dtype == torch.bfloat16 else _lib.F32,
                                torch.cuda.current_stream(parts.device).cuda_stream)
    raise_for_status(st)
    return out


def rope_rows(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, scaling_factor: float = 1.0,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RoPE on ``x`` ``[n_rows, n_heads, head_dim]`` with one absolute position per row
    (apply_rotary_pos_emb_mlx, src/ollm/llama_mlx.py:149-182)."""
    if not x.is_cuda:
        raise RuntimeError("rope_rows needs a CUDA tensor; there is no CPU path")
    if x.dim() != 3 or x.stride(-1) != 1:
        raise ValueError("x must be [n_rows, n_heads, head_dim] with contiguous head_dim")
    if out is None:
        out = torch.empty_like(x)
    if out.stride() != x.stride():
        raise ValueError("out must share x's strides")
    positions = positions.to(device=x.device, dtype=torch.int32).contiguous()
    inv_freq = inv_freq.to(device=x.device, dtype=torch.float32).contiguous()
    dt = _lib.BF16 if x.dtype == torch.bfloat16 else _lib.F32
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("x must be float32 or bfloat16")
    st = lib.skv_rope_rows(x.data_ptr(), out.data_ptr(), positions.data_ptr(), inv_freq.data_ptr(), x.shape[0],
                           x.shape[1], x.shape[2], x.stride(0), x.stride(1), float(scaling_factor), dt,
                           torch.cuda.current_stream(x.device).cuda_stream)
    raise_for_status(st)
    return out
