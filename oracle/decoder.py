"""NumPy restatement of the reference's Llama / DeepSeek decoder around the hot path.

Test infrastructure only (see ``oracle/__init__.py``).

Follows the reference's ``src/ollm/llama_mlx.py`` (DeepSeek twin in
``src/ollm/deepseek_mlx.py`` differs only in defaults, see ``DecoderOracle``):
  * ``rms_norm``            -> MLXRMSNorm.__call__        :86-92
  * ``linear``              -> _linear (unquantised)      :53-63
  * ``mlp``                 -> MLXLlamaMLP.__call__       :390-408
  * ``DecoderOracle.attention`` -> MLXLlamaAttention.__call__ :220-316
  * ``DecoderOracle.forward``   -> MLXLlamaModel.__call__ :740-833 and
                                   MLXLlamaForCausalLM.__call__ :863-912
  * ``greedy_generate``     -> src/ollm/generation.py:7-50
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import Dict, Optional

import numpy as np

from . import attention as _attn
from . import rope as _rope
from .kvcache import ConcatKVCache


def rms_norm(x, weight, eps):
    x = np.asarray(x, dtype=np.float32)
    var = np.mean(np.square(x), axis=-1, keepdims=True, dtype=np.float32)
    return (weight * (x * (np.float32(1.0) / np.sqrt(var + np.float32(eps))))).astype(np.float32)


def linear(x, weight):
    return np.matmul(np.asarray(x, dtype=np.float32), np.asarray(weight, dtype=np.float32).T)


def silu(x):
    x = np.asarray(x, dtype=np.float32)
    return (x * (np.float32(1.0) / (np.float32(1.0) + np.exp(-x)))).astype(np.float32)


def mlp(x, gate_w, up_w, down_w):
    return linear(silu(linear(x, gate_w)) * linear(x, up_w), down_w)


def make_config(**kw) -> SimpleNamespace:
    base = dict(pad_token_id=0, rms_norm_eps=1e-6, max_position_embeddings=2048, rope_theta=10000.0,
                rope_scaling_factor=1.0)
    base.update(kw)
    return SimpleNamespace(**base)


def random_weights(config, seed: int, std: float = 0.02) -> Dict[str, np.ndarray]:
    """Seeded N(0, std) float32 weights in the key order of the reference's
    ``tiny_weights`` fixture (tests/test_mlx_generation.py:64-88); norm weights are 1."""
    rng = np.random.default_rng(seed)
    H = config.hidden_size
    D = H // config.num_attention_heads
    Hkv = getattr(config, "num_key_value_heads", None) or config.num_attention_heads
    I = config.intermediate_size

    def mat(shape):
        return rng.normal(0.0, std, shape).astype(np.float32)

    w: Dict[str, np.ndarray] = {}
    for i in range(config.num_hidden_layers):
        b = f"model.layers.{i}"
        w[f"{b}.self_attn.q_proj.weight"] = mat((config.num_attention_heads * D, H))
        w[f"{b}.self_attn.k_proj.weight"] = mat((Hkv * D, H))
        w[f"{b}.self_attn.v_proj.weight"] = mat((Hkv * D, H))
        w[f"{b}.self_attn.o_proj.weight"] = mat((H, config.num_attention_heads * D))
        w[f"{b}.mlp.gate_proj.weight"] = mat((I, H))
        w[f"{b}.mlp.up_proj.weight"] = mat((I, H))
        w[f"{b}.mlp.down_proj.weight"] = mat((H, I))
        w[f"{b}.input_layernorm.weight"] = np.ones((H,), dtype=np.float32)
        w[f"{b}.post_attention_layernorm.weight"] = np.ones((H,), dtype=np.float32)
    w["model.embed_tokens.weight"] = mat((config.vocab_size, H))
    w["lm_head.weight"] = mat((config.vocab_size, H))
    w["model.norm.weight"] = np.ones((H,), dtype=np.float32)
    return w


class DecoderOracle:
    """Float32 decoder forward with the reference's call sequence around the cache."""

    def __init__(self, config, weights: Dict[str, np.ndarray], round_dtype=None, round_glue: bool = False):
        self.config = config
        self.w = weights
        self.H = config.hidden_size
        self.Hq = config.num_attention_heads
        # deepseek_mlx.py:235 defaults KV heads to the attention-head count (MHA).
        self.Hkv = getattr(config, "num_key_value_heads", None) or self.Hq
        self.D = self.H // self.Hq
        self.eps = getattr(config, "rms_norm_eps", 1e-6)
        self.theta = getattr(config, "rope_theta", 10000.0)
        self.rope_scale = getattr(config, "rope_scaling_factor", 1.0)
        # Optional rounding of stored K/V and of attention inputs/outputs to a
        # storage dtype (e.g. ml_dtypes.bfloat16) at the points where the CUDA
        # path stores that dtype.
        self.round_dtype = round_dtype
        # round_glue additionally rounds after every linear layer, norm, activation product and residual
        # add, which is where a decoder whose glue runs in that storage dtype (cuBLAS, fp32 accumulate,
        # one rounding per output) rounds.
        self.round_glue = round_glue and round_dtype is not None

    def _g(self, x):
        return self._round(x) if self.round_glue else x

    def _mlp(self, x, b):
        gate = self._g(linear(x, self.w[f"{b}.mlp.gate_proj.weight"]))
        up = self._g(linear(x, self.w[f"{b}.mlp.up_proj.weight"]))
        act = self._g(self._g(silu(gate)) * up)
        return self._g(linear(act, self.w[f"{b}.mlp.down_proj.weight"]))

    def _round(self, x):
        if self.round_dtype is None:
            return x
        return np.asarray(x).astype(self.round_dtype).astype(np.float32)

    def attention(self, layer, hidden, cos, sin, position_ids, cache, cache_position):
        B, L, _ = hidden.shape
        b = f"model.layers.{layer}.self_attn"
        q = self._g(linear(hidden, self.w[f"{b}.q_proj.weight"])).reshape(B, L, self.Hq, self.D).transpose(0, 2, 1, 3)
        k = self._g(linear(hidden, self.w[f"{b}.k_proj.weight"])).reshape(B, L, self.Hkv, self.D).transpose(0, 2, 1, 3)
        v = self._g(linear(hidden, self.w[f"{b}.v_proj.weight"])).reshape(B, L, self.Hkv, self.D).transpose(0, 2, 1, 3)
        q, k = _rope.apply_qk(self._round(q), self._round(k), cos, sin)
        q, k, v = self._round(q), self._round(k), self._round(v)
        if cache is not None:
            k, v = cache.update(k, v, layer, {"sin": sin, "cos": cos, "cache_position": cache_position})
        o = _attn.chunked_grouped_attention(
            q, k, v, query_positions=position_ids, causal=True, q_block_size=32768,
            k_block_size=(1024 if L > 128 else 1000000),
        )
        o = self._round(o).transpose(0, 2, 1, 3).reshape(B, L, -1)
        return self._g(linear(o, self.w[f"{b}.o_proj.weight"]))

    def forward(self, input_ids, past_key_values: Optional[ConcatKVCache] = None, use_cache: bool = False):
        input_ids = np.asarray(input_ids)
        B, L = input_ids.shape
        hidden = self.w["model.embed_tokens.weight"][input_ids].astype(np.float32)
        cache = past_key_values if use_cache else None
        past = cache.get_seq_length() if cache is not None else 0
        cache_position = np.arange(past, past + L, dtype=np.int32)
        position_ids = cache_position[None, :]
        cos, sin = _rope.cos_sin(position_ids, self.D, self.theta, self.rope_scale)
        for i in range(self.config.num_hidden_layers):
            b = f"model.layers.{i}"
            x = self._g(rms_norm(hidden, self.w[f"{b}.input_layernorm.weight"], self.eps))
            hidden = self._g(hidden + self.attention(i, x, cos, sin, position_ids, cache, cache_position))
            x = self._g(rms_norm(hidden, self.w[f"{b}.post_attention_layernorm.weight"], self.eps))
            hidden = self._g(hidden + self._mlp(x, b))
        hidden = self._g(rms_norm(hidden, self.w["model.norm.weight"], self.eps))
        head = self.w.get("lm_head.weight")
        if head is None:  # tied-embedding fallback, llama_mlx.py:886-890
            head = self.w["model.embed_tokens.weight"]
        return self._g(linear(hidden, head))

    __call__ = forward


def greedy_generate(model, input_ids, *, max_new_tokens: int, temperature: float, past_key_values=None):
    """Prefill once, then one-token cached decode calls (generation.py:7-50)."""
    if max_new_tokens < 0:
        raise ValueError("max_new_tokens must be non-negative")
    if temperature <= 0:
        raise ValueError("temperature must be positive")
    input_ids = np.asarray(input_ids)
    if input_ids.ndim != 2 or input_ids.shape[1] == 0:
        raise ValueError("input_ids must have shape [batch, sequence] with sequence > 0")
    if max_new_tokens == 0:
        return input_ids
    cache = past_key_values if past_key_values is not None else ConcatKVCache(model.config, cache_dir=None)
    generated, step_input = input_ids, input_ids
    for _ in range(max_new_tokens):
        logits = model(step_input, past_key_values=cache, use_cache=True)
        nxt = np.argmax(logits[:, -1, :] / temperature, axis=-1, keepdims=True).astype(input_ids.dtype)
        generated = np.concatenate([generated, nxt], axis=1)
        step_input = nxt
    return generated
