"""Prefill once, then one-token cached decode calls (greedy), with the reference's contract.

Mirrors ``greedy_generate_mx`` (src/ollm/generation.py:7-50): same validation and messages, the
prompt is never replayed, a fresh memory-only cache is made when none is passed.
"""
from __future__ import annotations

from typing import Any, Optional

import torch

from .kvcache import PagedKVCache


def greedy_generate(model: Any, input_ids: torch.Tensor, *, max_new_tokens: int, temperature: float,
                    past_key_values: Optional[Any] = None) -> torch.Tensor:
    if max_new_tokens < 0:
        raise ValueError("max_new_tokens must be non-negative")
    if temperature <= 0:
        raise ValueError("temperature must be positive")
    if input_ids.ndim != 2 or input_ids.shape[1] == 0:
        raise ValueError("input_ids must have shape [batch, sequence] with sequence > 0")
    if max_new_tokens == 0:
        return input_ids
    cache = past_key_values
    if cache is None:
        cache = PagedKVCache(model.config, cache_dir=None)
    generated = input_ids
    model_input = input_ids
    for _ in range(max_new_tokens):
        logits = model(model_input, past_key_values=cache, use_cache=True)
        next_token = torch.argmax(logits[:, -1, :] / temperature, dim=-1, keepdim=True).to(input_ids.dtype)
        generated = torch.cat([generated, next_token.to(generated.device)], dim=1)
        model_input = next_token
    return generated
