"""PagedKVCache: the reference's KV-cache duck type on top of the paged pool.

Same call surface as ``MLXKVCache`` (src/ollm/mlx_kvcache.py:21-307): ``update`` with replay
rejection, per-layer ``get_seq_length``, ``__getitem__`` / ``__len__`` / ``__contains__``,
``save_to_disk`` / ``offload_layers_to_disk`` / ``clear`` with the same ``.npz`` fields and the same
error messages.  What differs is underneath: ``update`` writes only the new tokens into pages
(the reference re-concatenates the whole history, :107-118) and returns paged views that the
attention callable consumes directly; a dense tensor exists only when someone asks for one.

The pool is created at the first ``update`` (the reference also learns batch, heads and head_dim
from the first tensors it sees); pass ``pool=`` or the geometry keywords to size it up front.
"""
from __future__ import annotations

import os
import time
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from .attention import PagedView
from .pool import PagedKVConfig, PagedPool


def _positions_to_list(cache_position) -> List[int]:
    if isinstance(cache_position, torch.Tensor):
        return [int(x) for x in cache_position.reshape(-1).tolist()]
    return [int(x) for x in np.asarray(cache_position).reshape(-1).tolist()]


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0") not in ("", "0")


def _rows_packed(t: torch.Tensor) -> bool:
    """``[B, H, 1, D]`` whose heads lie back to back inside each batch row (contiguous, or a slice of a wider row)."""
    return t.dim() == 4 and t.shape[2] == 1 and t.stride(3) == 1 and t.stride(1) == t.shape[3]


class PagedKVCache:
    def __init__(self, config: Any, cache_dir: Optional[str] = None, stats: Optional[Any] = None, *,
                 pool: Optional[PagedPool] = None, device: Optional[int] = None, page_size: int = 16,
                 max_tokens: Optional[int] = None, host_pages: int = 0):
        self.config = config
        self.cache_dir = cache_dir
        self.stats = stats
        self.pool = pool
        self._device = device
        self._page_size = page_size
        self._max_tokens = max_tokens
        self._host_pages = host_pages
        self.seq_ids: Optional[List[int]] = None      # batch row -> pool sequence id
        self.batch_size = 0
        self._resident: set = set()                   # layers whose history sits in pages
        self._disk_offloaded: Dict[int, str] = {}
        self._layer_lengths: Dict[int, int] = {}
        self._managed_disk_files: set = set()
        self._seen_tokens = 0
        # layer files: float32 `key` / `value` / `seen_tokens`, readable by the reference's loader; SKV_COMPACT_KV_FILES=1
        # (or this attribute) stores bfloat16 layers as raw 16-bit patterns instead, which only this loader reads
        self.compact_bf16_files = _env_flag("SKV_COMPACT_KV_FILES")
        if cache_dir is not None:
            os.makedirs(cache_dir, exist_ok=True)

    # -- validators: messages of mlx_kvcache.py:127-158 -------------------------------------------
    def _validate_layer_index(self, layer_idx):
        if not isinstance(layer_idx, int) or layer_idx < 0:
            raise ValueError("layer_idx must be a non-negative integer")
        count = getattr(self.config, "num_hidden_layers", None)
        if count is not None and layer_idx >= count:
            raise ValueError(f"layer_idx {layer_idx} is outside configured layer count {count}")

    @staticmethod
    def _validate_state_shapes(key_states, value_states):
        if key_states.ndim != 4 or value_states.ndim != 4:
            raise ValueError("key and value states must have rank 4")
        if tuple(key_states.shape) != tuple(value_states.shape):
            raise ValueError("key and value states must have identical shapes")

    @staticmethod
    def _validate_cache_position(cache_kwargs, previous_length: int, new_length: int):
        if not cache_kwargs or cache_kwargs.get("cache_position") is None:
            return
        got = _positions_to_list(cache_kwargs["cache_position"])
        want = list(range(previous_length, previous_length + new_length))
        if got != want:
            raise ValueError(
                "cache_position must append exactly after the cached sequence; "
                f"expected {want}, got {got}"
            )

    # -- pool creation ----------------------------------------------------------------------------------
    def _ensure_pool(self, key_states: torch.Tensor):
        B, Hkv, _, D = key_states.shape
        if self.pool is None:
            max_tokens = self._max_tokens
            if max_tokens is None:
                max_tokens = min(int(getattr(self.config, "max_position_embeddings", 4096) or 4096), 8192)
            pages_per_seq = -(-max_tokens // self._page_size)
            layers = getattr(self.config, "num_hidden_layers", None)
            if layers is None:
                raise ValueError("config.num_hidden_layers is required")
            dev = key_states.device.index if self._device is None else self._device
            self.pool = PagedPool(PagedKVConfig(
                num_layers=layers, num_kv_heads=Hkv, head_dim=D, num_pages=B * pages_per_seq, max_seqs=B,
                max_pages_per_seq=pages_per_seq, page_size=self._page_size, dtype=key_states.dtype,
                device=dev, host_pages=self._host_pages))
        if self.seq_ids is None:
            # sorted: on a pool of its own the cache then owns sequences 0..B-1 in batch order, which is what the
            # one-call decode step needs (the allocator hands ids back in LIFO order after a clear)
            self.seq_ids = sorted(self.pool.alloc_sequence() for _ in range(B))
            self.batch_size = B

    # -- update (mlx_kvcache.py:65-125) ----------------------------------------------------------------------
    def _prepare_update(self, key_states, value_states, layer_idx, cache_kwargs) -> int:
        self._validate_layer_index(layer_idx)
        self._validate_state_shapes(key_states, value_states)
        if not isinstance(key_states, torch.Tensor) or not key_states.is_cuda:
            raise RuntimeError("PagedKVCache.update needs CUDA tensors; there is no CPU path")
        if layer_idx in self._disk_offloaded:
            self._load_layer_from_disk(layer_idx)
        previous = self._layer_lengths.get(layer_idx, 0)
        self._validate_cache_position(cache_kwargs, previous, key_states.shape[2])
        self._ensure_pool(key_states)
        c = self.pool.cfg
        if (key_states.shape[0], key_states.shape[1], key_states.shape[3]) != (self.batch_size, c.num_kv_heads, c.head_dim):
            raise ValueError("new key states must match cached batch, head, and feature dimensions")
        return previous

    def _finish_update(self, layer_idx: int, previous: int, n_new: int):
        self._resident.add(layer_idx)
        self._layer_lengths[layer_idx] = previous + n_new
        self._seen_tokens = max(self._layer_lengths.values(), default=0)
        return PagedView(self, layer_idx, "key"), PagedView(self, layer_idx, "value")

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[Dict[str, Any]] = None) -> Tuple[PagedView, PagedView]:
        previous = self._prepare_update(key_states, value_states, layer_idx, cache_kwargs)
        if key_states.shape[2] > 0:
            self.pool.append(layer_idx, key_states, value_states, seq_ids=self.seq_ids,
                             start_pos=[previous] * self.batch_size)
        return self._finish_update(layer_idx, previous, key_states.shape[2])

    def _ensure_rope(self, inv_freq: np.ndarray, scaling_factor: float) -> None:
        """Hand the RoPE table to the pool when it changes (same array object and factor: nothing to compare)."""
        if inv_freq is getattr(self, "_rope_arr", None) and scaling_factor == getattr(self, "_rope_scale", None):
            return
        rope_key = (inv_freq.tobytes(), float(scaling_factor))
        if getattr(self, "_rope_key", None) != rope_key:
            self.pool.set_rope(inv_freq, scaling_factor)
            self._rope_key = rope_key
        self._rope_arr, self._rope_scale = inv_freq, scaling_factor

    def update_with_rope(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                         layer_idx: int, cache_kwargs: Optional[Dict[str, Any]] = None, *, inv_freq: np.ndarray,
                         scaling_factor: float = 1.0) -> Tuple[PagedView, PagedView]:
        """``update`` for un-rotated K: RoPE is applied on the way into the pages, and ``query_states``
        is rotated in place by the same launch (apply_rotary_pos_emb_mlx + update, llama_mlx.py:284-297)."""
        previous = self._prepare_update(key_states, value_states, layer_idx, cache_kwargs)
        self._ensure_rope(inv_freq, scaling_factor)
        if key_states.shape[2] > 0:
            self.pool.append(layer_idx, key_states, value_states, seq_ids=self.seq_ids,
                             start_pos=[previous] * self.batch_size, rope_k=True, q=query_states)
        return self._finish_update(layer_idx, previous, key_states.shape[2])

    def decode_step_with_rope(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                              layer_idx: int, cache_kwargs: Optional[Dict[str, Any]] = None, *, inv_freq: np.ndarray,
                              scaling_factor: float = 1.0, eps: float = 1e-12,
                              out: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """The cached decode step of a layer (one new token per sequence) in ONE library call:
        ``update_with_rope`` followed by the attention call with ``query_positions = [past]``
        (llama_mlx.py:284-308 for L == 1).  Same validation and bookkeeping as ``update``; ``query_states``
        is rotated in place; returns ``[B, Hq, 1, D]`` (written into ``out`` when given), or ``None`` when the step
        does not apply (more than one token) and the caller should make the two calls."""
        if key_states.dim() != 4 or key_states.shape[2] != 1 or query_states.dim() != 4 or query_states.shape[2] != 1:
            return None
        if self.seq_ids is None or not all(_rows_packed(t) for t in (query_states, key_states, value_states)):
            return None
        previous = self._prepare_update(key_states, value_states, layer_idx, cache_kwargs)
        self._ensure_rope(inv_freq, scaling_factor)
        B, Hq, _, D = query_states.shape
        # [B, H, 1, D] -> [B, H, D] without a copy: the tensors may be strided slices of one fused projection output
        out = self.pool.decode_step(layer_idx, query_states[:, :, 0], key_states[:, :, 0], value_states[:, :, 0], eps=eps,
                                    out=None if out is None else out[:, :, 0],
                                    seq_ids=None if list(self.seq_ids) == list(range(B)) else self.seq_ids)
        self._finish_update(layer_idx, previous, 1)
        return out.unsqueeze(2)

    def bind_decode_step(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                         out: torch.Tensor, *, inv_freq: np.ndarray, scaling_factor: float = 1.0, eps: float = 1e-12):
        """``decode_step_with_rope`` for tensors that stay put (static buffers of a CUDA graph): shapes, dtypes and
        the RoPE table are checked once; the returned ``step(layer, position, stream)`` rejects a position that does
        not append exactly after the cached sequence, makes the library call and does the bookkeeping of
        ``update``.  Returns ``None`` when a per-update policy has to run (a layer window), so that the caller keeps
        using ``decode_step_with_rope``."""
        if self.pool is None or self.seq_ids is None or type(self)._finish_update is not PagedKVCache._finish_update:
            return None
        self._validate_state_shapes(key_states, value_states)
        B, Hq, L, D = query_states.shape
        Hkv = key_states.shape[1]
        c = self.pool.cfg
        if L != 1 or key_states.shape[2] != 1 or (B, Hkv, D) != (self.batch_size, c.num_kv_heads, c.head_dim):
            raise ValueError("new key states must match cached batch, head, and feature dimensions")
        self._ensure_rope(inv_freq, scaling_factor)
        call = self.pool.decode_step_binder(query_states[:, :, 0], key_states[:, :, 0], value_states[:, :, 0], out[:, :, 0], eps=eps,
                                            seq_ids=None if list(self.seq_ids) == list(range(B)) else self.seq_ids)
        lengths, resident, offloaded = self._layer_lengths, self._resident, self._disk_offloaded

        def step(layer_idx: int, position: int, stream: int) -> None:
            if layer_idx in offloaded:
                self._load_layer_from_disk(layer_idx)
            previous = lengths.get(layer_idx, 0)
            if position != previous:
                raise ValueError("cache_position must append exactly after the cached sequence; "
                                 f"expected {[previous]}, got {[position]}")
            call(layer_idx, stream)
            resident.add(layer_idx)
            lengths[layer_idx] = previous + 1
            if previous + 1 > self._seen_tokens:
                self._seen_tokens = previous + 1
        return step

    # -- lengths (mlx_kvcache.py:160-181) ----------------------------------------------------------------------
    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        if layer_idx is None:
            return max(self._layer_lengths.values(), default=0)
        return self._layer_lengths.get(layer_idx, 0)

    def get_max_cache_shape(self) -> Optional[int]:
        return None

    # -- dense view ------------------------------------------------------------------------------------------------
    def materialize(self, layer_idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense ``[B, Hkv, T, D]`` K and V of a resident layer (gather kernel)."""
        if layer_idx in self._disk_offloaded:
            self._load_layer_from_disk(layer_idx)
        if layer_idx not in self._resident:
            raise KeyError(layer_idx)
        return self.pool.gather(layer_idx, seq_ids=self.seq_ids, max_len=self._layer_lengths[layer_idx])

    # -- disk round trip (mlx_kvcache.py:183-284) ---------------------------------------------------------------------
    def save_to_disk(self, layer_idx: int, filename: Optional[str] = None):
        if layer_idx not in self._resident:
            return
        if filename is None:
            if self.cache_dir is None:
                raise ValueError("filename is required for a memory-only KV cache")
            filename = os.path.join(self.cache_dir, f"kvcache_layer_{layer_idx}.npz")
        dest = Path(filename)
        dest.parent.mkdir(parents=True, exist_ok=True)
        t0 = time.perf_counter()
        k, v = self.materialize(layer_idx)
        extra = {}
        if k.dtype == torch.bfloat16 and self.compact_bf16_files:
            # NumPy has no bfloat16: the raw 16-bit patterns plus a tag.  Half the bytes, but only this loader reads it
            # (the reference's loader, mlx_kvcache.py:232-247, would take the patterns for integers).
            k_np = k.view(torch.int16).cpu().numpy().view(np.uint16)
            v_np = v.view(torch.int16).cpu().numpy().view(np.uint16)
            extra["stored_dtype"] = "bfloat16"
        else:
            # float32 holds every bfloat16 value exactly: a file either side can read, like the reference's own
            k_np, v_np = k.float().cpu().numpy(), v.float().cpu().numpy()
        np.savez_compressed(dest, key=k_np, value=v_np, seen_tokens=self._seen_tokens, **extra)
        if self.stats:
            self.stats.set("kv_save_to_disk", t0)
        self._disk_offloaded[layer_idx] = os.fspath(dest)
        self._managed_disk_files.add(os.fspath(dest))
        self._resident.discard(layer_idx)
        # the pages stay owned by the sequences (a page holds every layer); the layer's rows are
        # rewritten from the file on reload, so stale bytes can never be observed
        self._reset_layer_length(layer_idx)

    def _reset_layer_length(self, layer_idx: int):
        # lengths of this layer back to 0 (pages stay) so that the reload appends from position 0
        self.pool.truncate(layer_idx, 0, seq_ids=self.seq_ids)

    def _load_layer_from_disk(self, layer_idx: int):
        if layer_idx not in self._disk_offloaded:
            return
        filename = self._disk_offloaded[layer_idx]
        t0 = time.perf_counter()
        with np.load(filename) as data:
            key_np, value_np = data["key"], data["value"]
            if "seen_tokens" in data:
                self._seen_tokens = int(data["seen_tokens"])
            bf16 = "stored_dtype" in data and str(data["stored_dtype"]) == "bfloat16"
        dev = self.pool.torch_device
        if bf16:
            k = torch.from_numpy(key_np.view(np.int16)).to(dev).view(torch.bfloat16)
            v = torch.from_numpy(value_np.view(np.int16)).to(dev).view(torch.bfloat16)
        else:
            k = torch.from_numpy(key_np).to(dev)
            v = torch.from_numpy(value_np).to(dev)
        if k.dtype != self.pool.cfg.dtype:      # e.g. a float32 file written by the reference for a bfloat16 pool
            k, v = k.to(self.pool.cfg.dtype), v.to(self.pool.cfg.dtype)
        if k.shape[2] > 0:
            self.pool.append(layer_idx, k.contiguous(), v.contiguous(), seq_ids=self.seq_ids, start_pos=[0] * self.batch_size)
        self._resident.add(layer_idx)
        self._layer_lengths[layer_idx] = k.shape[2]
        if self.stats:
            self.stats.set("kv_load_from_disk", t0)
        del self._disk_offloaded[layer_idx]

    def offload_layers_to_disk(self, layer_indices: Optional[List[int]] = None):
        if layer_indices is None:
            layer_indices = sorted(self._resident)
        for idx in layer_indices:
            if idx in self._resident:
                self.save_to_disk(idx)

    def clear(self):
        if self.pool is not None and self.seq_ids is not None:
            for s in self.seq_ids:
                self.pool.free_sequence(s)
        self.seq_ids = None
        self.batch_size = 0
        self._resident.clear()
        for name in self._managed_disk_files:
            if os.path.exists(name):
                os.remove(name)
        self._disk_offloaded.clear()
        self._managed_disk_files.clear()
        self._layer_lengths.clear()
        self._seen_tokens = 0

    # -- container protocol (mlx_kvcache.py:286-307) ----------------------------------------------------------------------
    def __len__(self) -> int:
        return len(self._resident) + len(self._disk_offloaded)

    def __getitem__(self, layer_idx: int) -> Dict[str, Optional[torch.Tensor]]:
        if layer_idx in self._disk_offloaded:
            self._load_layer_from_disk(layer_idx)
        if layer_idx not in self._resident:
            return {"key": None, "value": None}
        k, v = self.materialize(layer_idx)
        return {"key": k, "value": v}

    def __contains__(self, layer_idx: int) -> bool:
        return layer_idx in self._resident or layer_idx in self._disk_offloaded

    # -- host tier (no reference counterpart; stands in for the disk tier at page granularity) -------------------------------
    def evict_oldest(self, fraction: float):
        """Park the oldest ``fraction`` of every sequence's full pages in pinned host memory."""
        T = self.get_seq_length(None)
        n = int((T // self.pool.cfg.page_size) * fraction)
        for s in self.seq_ids or []:
            if n > 0:
                self.pool.evict(s, 0, n)
        return n

    def prefetch_all(self):
        for s in self.seq_ids or []:
            n = len(self.pool.page_table(s))
            if n:
                self.pool.prefetch(s, 0, n)
        self.pool.sync_transfers()


class PagedLlamaDiskCache(PagedKVCache):
    """Keeps at most ``max_layers_in_memory`` layers in pages, spilling the lowest-index layers to
    ``.npz`` files, never the layer just written (MLXLlamaDiskCache, mlx_kvcache.py:310-367).
    ``None`` disables the spill: a B200 holds every layer of the configurations this library targets."""

    def __init__(self, config: Any, cache_dir: str = "./kvcache", stats: Optional[Any] = None,
                 max_layers_in_memory: Optional[int] = 4, **kw):
        super().__init__(config, cache_dir, stats, **kw)
        if max_layers_in_memory is not None and max_layers_in_memory <= 0:
            raise ValueError("max_layers_in_memory must be positive")
        self.max_layers_in_memory = max_layers_in_memory

    def _finish_update(self, layer_idx: int, previous: int, n_new: int):
        # every way of appending (update, update_with_rope, decode_step_with_rope) ends here
        result = super()._finish_update(layer_idx, previous, n_new)
        if self.max_layers_in_memory is not None and len(self._resident) > self.max_layers_in_memory:
            for idx in sorted(self._resident)[: -self.max_layers_in_memory]:
                if idx != layer_idx:
                    self.save_to_disk(idx)
        return result


class PagedQwen3NextDiskCache(PagedKVCache):
    """Cache for Qwen3-Next models: the base cache plus the layer count the reference records
    (``config.num_hidden_layers``, 80 when the config has none; MLXQwen3NextDiskCache, mlx_kvcache.py:370-396)."""

    def __init__(self, config: Any, cache_dir: str = "./kvcache", stats: Optional[Any] = None, **kw):
        super().__init__(config, cache_dir, stats, **kw)
        self.num_layers = getattr(config, "num_hidden_layers", None) or 80


def create_paged_kv_cache(model_id: str, config: Any, cache_dir: str = "./kvcache", stats: Optional[Any] = None,
                          **kw) -> PagedKVCache:
    """Factory by model-id prefix (create_mlx_kv_cache, mlx_kvcache.py:399-425)."""
    if model_id.startswith("llama"):
        kw.setdefault("max_layers_in_memory", None)
        return PagedLlamaDiskCache(config, cache_dir, stats, **kw)
    if model_id.startswith("qwen"):
        return PagedQwen3NextDiskCache(config, cache_dir, stats, **kw)
    return PagedKVCache(config, cache_dir, stats, **kw)          # "gemma" and everything else: the base class
