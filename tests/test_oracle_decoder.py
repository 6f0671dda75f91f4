"""Decoder-glue oracle: arithmetic against the reference CPU executor's outputs
(fixture), and the reference's model-level relations
(tests/test_mlx_generation.py:140-156, 249-257, 282-323)."""
import os
from types import SimpleNamespace

import numpy as np
import pytest

from oracle import decoder as od
from oracle.kvcache import ConcatKVCache


def test_glue_arithmetic_matches_reference_cpu_executor(golden_dir):
    with np.load(os.path.join(golden_dir, "decoder_glue.npz")) as d:
        assert np.allclose(od.linear(d["x"], d["w"]), d["linear"], atol=1e-6, rtol=1e-6)
        assert np.allclose(od.rms_norm(d["x"], d["scale"], float(d["eps"])), d["rms"], atol=1e-6, rtol=1e-6)
        assert np.allclose(od.silu(d["x"]), d["silu"], atol=1e-6, rtol=1e-6)


def tiny_config(**kw):
    # tests/test_mlx_generation.py:49-61
    return od.make_config(vocab_size=17, hidden_size=8, intermediate_size=12, num_hidden_layers=2,
                          num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=32, **kw)


@pytest.mark.parametrize("mha", [False, True])
def test_cached_decode_matches_full_causal_forward(mha):
    cfg = tiny_config()
    if mha:
        cfg.num_key_value_heads = None   # DeepSeek default: MHA
    model = od.DecoderOracle(cfg, od.random_weights(cfg, seed=7, std=0.15))
    ids = np.array([[2, 5, 3, 11]], dtype=np.int32)
    full = model(ids, use_cache=False)
    cache = ConcatKVCache(cfg, cache_dir=None)
    model(ids[:, :3], past_key_values=cache, use_cache=True)
    dec = model(ids[:, 3:], past_key_values=cache, use_cache=True)
    assert cache.get_seq_length() == 4
    assert np.allclose(full[:, -1, :], dec[:, -1, :], atol=1e-5, rtol=1e-5)


def test_cache_untouched_when_use_cache_false():
    cfg = tiny_config()
    model = od.DecoderOracle(cfg, od.random_weights(cfg, seed=7, std=0.15))
    cache = ConcatKVCache(cfg, cache_dir=None)
    model(np.array([[2, 5, 3]]), past_key_values=cache, use_cache=False)
    assert cache.get_seq_length() == 0


def test_generation_prefills_once_then_decodes_one_token_at_a_time():
    class RecordingModel:
        def __init__(self):
            self.config = SimpleNamespace(num_hidden_layers=1)
            self.input_lengths, self.cache_lengths = [], []

        def __call__(self, input_ids, past_key_values=None, use_cache=False):
            self.input_lengths.append(input_ids.shape[1])
            self.cache_lengths.append(past_key_values.get_seq_length())
            B, L = input_ids.shape
            st = np.broadcast_to(input_ids[:, None, :, None].astype(np.float32), (B, 1, L, 2))
            start = past_key_values.get_seq_length()
            past_key_values.update(st, st, 0, {"cache_position": np.arange(start, start + L)})
            return np.broadcast_to(np.array([0.0, 0.0, 0.0, 1.0, 0.0]), (B, L, 5))

    m = RecordingModel()
    out = od.greedy_generate(m, np.array([[1, 2, 4, 2]], dtype=np.int32), max_new_tokens=3, temperature=1.0)
    assert m.input_lengths == [4, 1, 1] and m.cache_lengths == [0, 4, 5]
    assert out.shape == (1, 7) and np.array_equal(out[:, -3:], [[3, 3, 3]])
    with pytest.raises(ValueError, match="non-negative"):
        od.greedy_generate(m, np.array([[1]]), max_new_tokens=-1, temperature=1.0)
    with pytest.raises(ValueError, match="temperature must be positive"):
        od.greedy_generate(m, np.array([[1]]), max_new_tokens=1, temperature=0.0)
    with pytest.raises(ValueError, match="shape"):
        od.greedy_generate(m, np.array([1]), max_new_tokens=1, temperature=1.0)
    same = np.array([[1, 2]])
    assert od.greedy_generate(m, same, max_new_tokens=0, temperature=1.0) is same
