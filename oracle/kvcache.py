"""NumPy restatement of the reference's concatenating KV cache.

Test infrastructure only (see ``oracle/__init__.py``).

Follows ``src/ollm/mlx_kvcache.py`` of the reference, with ``np.concatenate``
standing in for ``mx.concatenate``:
  * ``ConcatKVCache``       -> MLXKVCache             :21-307
  * ``LayerWindowKVCache``  -> MLXLlamaDiskCache      :310-367
  * ``create_kv_cache``     -> create_mlx_kv_cache    :399-425
"""
from __future__ import annotations

import os
from pathlib import Path
from typing import Any, Dict, Optional

import numpy as np


class ConcatKVCache:
    def __init__(self, config: Any, cache_dir: Optional[str] = None, stats: Optional[Any] = None):
        self.config = config
        self.cache_dir = cache_dir
        self.stats = stats
        self._cache: Dict[int, Dict[str, np.ndarray]] = {}
        self._disk_offloaded: Dict[int, str] = {}
        self._layer_lengths: Dict[int, int] = {}
        self._managed_disk_files: set = set()
        if cache_dir is not None:
            os.makedirs(cache_dir, exist_ok=True)
        self._seen_tokens = 0

    # -- validators (mlx_kvcache.py:127-158) ---------------------------------
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
        if key_states.shape != value_states.shape:
            raise ValueError("key and value states must have identical shapes")

    @staticmethod
    def _validate_cache_position(cache_kwargs, previous_length, new_length):
        if not cache_kwargs or cache_kwargs.get("cache_position") is None:
            return
        got = np.asarray(cache_kwargs["cache_position"]).reshape(-1)
        want = np.arange(previous_length, previous_length + new_length)
        if got.shape != want.shape or not np.array_equal(got, want):
            raise ValueError(
                "cache_position must append exactly after the cached sequence; "
                f"expected {want.tolist()}, got {got.tolist()}"
            )

    # -- update (mlx_kvcache.py:65-125) ---------------------------------------
    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self._validate_layer_index(layer_idx)
        self._validate_state_shapes(key_states, value_states)
        if layer_idx in self._disk_offloaded:
            self._load_layer_from_disk(layer_idx)
        self._validate_cache_position(
            cache_kwargs, self._layer_lengths.get(layer_idx, 0), key_states.shape[2]
        )
        entry = self._cache.get(layer_idx)
        if entry is not None:
            ck, cv = entry["key"], entry["value"]
            if ck.shape[:2] + ck.shape[3:] != key_states.shape[:2] + key_states.shape[3:]:
                raise ValueError("new key states must match cached batch, head, and feature dimensions")
            if cv.shape[:2] + cv.shape[3:] != value_states.shape[:2] + value_states.shape[3:]:
                raise ValueError("new value states must match cached batch, head, and feature dimensions")
            entry["key"] = np.concatenate([ck, key_states], axis=2)
            entry["value"] = np.concatenate([cv, value_states], axis=2)
        else:
            entry = self._cache[layer_idx] = {"key": key_states, "value": value_states}
        self._layer_lengths[layer_idx] = entry["key"].shape[2]
        self._seen_tokens = max(self._layer_lengths.values(), default=0)
        return entry["key"], entry["value"]

    # -- lengths (mlx_kvcache.py:160-181) --------------------------------------
    def get_seq_length(self, layer_idx: Optional[int] = 0) -> int:
        if layer_idx is None:
            return max(self._layer_lengths.values(), default=0)
        return self._layer_lengths.get(layer_idx, 0)

    def get_max_cache_shape(self):
        return None

    # -- disk round trip (mlx_kvcache.py:183-284) -------------------------------
    def save_to_disk(self, layer_idx: int, filename: Optional[str] = None):
        if layer_idx not in self._cache:
            return
        if filename is None:
            if self.cache_dir is None:
                raise ValueError("filename is required for a memory-only KV cache")
            filename = os.path.join(self.cache_dir, f"kvcache_layer_{layer_idx}.npz")
        dest = Path(filename)
        dest.parent.mkdir(parents=True, exist_ok=True)
        np.savez_compressed(
            dest,
            key=np.asarray(self._cache[layer_idx]["key"]),
            value=np.asarray(self._cache[layer_idx]["value"]),
            seen_tokens=self._seen_tokens,
        )
        self._disk_offloaded[layer_idx] = os.fspath(dest)
        self._managed_disk_files.add(os.fspath(dest))
        del self._cache[layer_idx]

    def _load_layer_from_disk(self, layer_idx: int):
        if layer_idx not in self._disk_offloaded:
            return
        with np.load(self._disk_offloaded[layer_idx]) as data:
            key, value = data["key"], data["value"]
            if "seen_tokens" in data:
                self._seen_tokens = int(data["seen_tokens"])
        self._cache[layer_idx] = {"key": key, "value": value}
        self._layer_lengths[layer_idx] = key.shape[2]
        del self._disk_offloaded[layer_idx]

    def offload_layers_to_disk(self, layer_indices=None):
        if layer_indices is None:
            layer_indices = list(self._cache.keys())
        for idx in layer_indices:
            if idx in self._cache:
                self.save_to_disk(idx)

    def clear(self):
        self._cache.clear()
        for name in self._managed_disk_files:
            if os.path.exists(name):
                os.remove(name)
        self._disk_offloaded.clear()
        self._managed_disk_files.clear()
        self._layer_lengths.clear()
        self._seen_tokens = 0

    # -- container protocol (mlx_kvcache.py:286-307) -----------------------------
    def __len__(self):
        return len(self._cache) + len(self._disk_offloaded)

    def __getitem__(self, layer_idx):
        if layer_idx in self._disk_offloaded:
            self._load_layer_from_disk(layer_idx)
        return self._cache.get(layer_idx, {"key": None, "value": None})

    def __contains__(self, layer_idx):
        return layer_idx in self._cache or layer_idx in self._disk_offloaded


class LayerWindowKVCache(ConcatKVCache):
    """Keeps at most ``max_layers_in_memory`` layers resident (mlx_kvcache.py:310-367)."""

    def __init__(self, config, cache_dir="./kvcache", stats=None, max_layers_in_memory: int = 4):
        super().__init__(config, cache_dir, stats)
        if max_layers_in_memory <= 0:
            raise ValueError("max_layers_in_memory must be positive")
        self.max_layers_in_memory = max_layers_in_memory

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        result = super().update(key_states, value_states, layer_idx, cache_kwargs)
        if len(self._cache) > self.max_layers_in_memory:
            for idx in sorted(self._cache.keys())[: -self.max_layers_in_memory]:
                if idx != layer_idx:
                    self.save_to_disk(idx)
        return result


def create_kv_cache(model_id: str, config, cache_dir: str = "./kvcache", stats=None):
    """Factory by model-id prefix (mlx_kvcache.py:399-425)."""
    if model_id.startswith("llama"):
        return LayerWindowKVCache(config, cache_dir, stats)
    return ConcatKVCache(config, cache_dir, stats)
