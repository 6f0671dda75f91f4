"""RoPE and concat-KV oracle against the reference's test expectations
(tests/test_mlx_generation.py:259-280, tests/test_mlx_kvcache.py:22-93)."""
import os
from types import SimpleNamespace

import numpy as np
import pytest

from oracle import rope as orope
from oracle.kvcache import ConcatKVCache, LayerWindowKVCache, create_kv_cache


def test_rope_matches_half_rotation_fixture(golden_dir):
    with np.load(os.path.join(golden_dir, "rope_half_rotation.npz")) as d:
        cos, sin = orope.cos_sin(d["positions"], int(d["dim"]), float(d["base"]))
        q_rot, k_rot = orope.apply_qk(d["q"], d["k"], cos, sin)
        assert cos.shape == (1, 3, 4) and cos.dtype == np.float32
        assert np.allclose(q_rot, d["q_out"], atol=1e-6)
        assert np.allclose(k_rot, d["k_out"], atol=1e-6)


def test_rope_linear_scaling_divides_positions():
    cos_a, sin_a = orope.cos_sin(np.array([[0, 4, 8]]), 8, 100000.0, scaling_factor=4.0)
    cos_b, sin_b = orope.cos_sin(np.array([[0, 1, 2]]), 8, 100000.0)
    assert np.array_equal(cos_a, cos_b) and np.array_equal(sin_a, sin_b)


def _states(start, length):
    values = np.arange(start, start + length * 8, dtype=np.float32).reshape(1, 2, length, 4)
    return values, values + 100


CONFIG = SimpleNamespace(num_hidden_layers=2)


def test_update_appends_and_tracks_each_layer_length():
    cache = ConcatKVCache(CONFIG, cache_dir=None)
    k0, v0 = _states(0, 3)
    k1, v1 = _states(24, 1)
    cache.update(k0, v0, 0, {"cache_position": np.arange(0, 3)})
    keys, values = cache.update(k1, v1, 0, {"cache_position": np.array([3])})
    assert cache.get_seq_length(0) == 4 and cache.get_seq_length(1) == 0
    assert cache.get_seq_length(None) == 4 and cache.get_max_cache_shape() is None
    assert keys.shape == (1, 2, 4, 4)
    assert np.array_equal(keys[:, :, :3], k0) and np.array_equal(values[:, :, 3:], v1)
    assert len(cache) == 1 and 0 in cache and 1 not in cache
    assert cache[1] == {"key": None, "value": None}


def test_update_rejects_replayed_positions_and_bad_shapes():
    cache = ConcatKVCache(CONFIG, cache_dir=None)
    k, v = _states(0, 2)
    cache.update(k, v, 0, {"cache_position": np.array([0, 1])})
    with pytest.raises(ValueError, match="append exactly"):
        cache.update(k, v, 0, {"cache_position": np.array([0, 1])})
    with pytest.raises(ValueError, match="non-negative integer"):
        cache.update(k, v, -1)
    with pytest.raises(ValueError, match="outside configured layer count"):
        cache.update(k, v, 2)
    with pytest.raises(ValueError, match="rank 4"):
        cache.update(k[0], v[0], 0)
    with pytest.raises(ValueError, match="identical shapes"):
        cache.update(k, v[:, :, :1], 0)
    with pytest.raises(ValueError, match="must match cached batch, head, and feature"):
        cache.update(k[:, :1], v[:, :1], 0)


def test_disk_round_trip_preserves_values_and_length(tmp_path):
    cache = ConcatKVCache(CONFIG, cache_dir=str(tmp_path))
    k, v = _states(0, 2)
    cache.update(k, v, 1, {"cache_position": np.array([0, 1])})
    cache.save_to_disk(1)
    path = tmp_path / "kvcache_layer_1.npz"
    assert cache.get_seq_length(1) == 2 and 1 not in cache._cache and path.exists()
    restored = cache[1]
    assert np.array_equal(restored["key"], k) and np.array_equal(restored["value"], v)
    assert cache.get_seq_length(1) == 2
    cache.clear()
    assert not path.exists() and cache.get_seq_length(None) == 0


def test_memory_only_cache_requires_explicit_destination():
    cache = ConcatKVCache(CONFIG, cache_dir=None)
    k, v = _states(0, 1)
    cache.update(k, v, 0)
    with pytest.raises(ValueError, match="filename is required"):
        cache.save_to_disk(0)


def test_layer_window_cache_offloads_lowest_layers(tmp_path):
    cfg = SimpleNamespace(num_hidden_layers=6)
    cache = LayerWindowKVCache(cfg, cache_dir=str(tmp_path), max_layers_in_memory=2)
    k, v = _states(0, 1)
    for layer in range(4):
        cache.update(k, v, layer)
    assert sorted(cache._cache) == [2, 3] and sorted(cache._disk_offloaded) == [0, 1]
    assert len(cache) == 4
    with pytest.raises(ValueError, match="must be positive"):
        LayerWindowKVCache(cfg, cache_dir=str(tmp_path), max_layers_in_memory=0)
    assert isinstance(create_kv_cache("llama3-1B", cfg, str(tmp_path)), LayerWindowKVCache)
    assert type(create_kv_cache("gemma", cfg, str(tmp_path))) is ConcatKVCache
