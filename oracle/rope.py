"""NumPy restatement of the reference's rotary position embedding.

Test infrastructure only (see ``oracle/__init__.py``).

Follows ``src/ollm/llama_mlx.py`` of the reference:
  * ``inv_freq``                   -> MLXRotaryEmbedding.__init__  :111-114
  * ``cos_sin``                    -> MLXRotaryEmbedding.__call__  :116-146
  * ``rotate_half`` / ``apply``    -> :149-182
``scaling_factor`` (linear position scaling, positions divided by the factor
before the multiplication with ``inv_freq``) has no reference counterpart: the
reference reads only ``rope_theta`` (llama_mlx.py:698-702).  It is the Hugging
Face "linear" convention and is defined here once for both sides.
"""
from __future__ import annotations

import numpy as np


def inv_freq(dim: int, base: float = 10000.0) -> np.ndarray:
    """``1 / base ** (arange(0, dim, 2) / dim)`` in float32 (llama_mlx.py:111-114)."""
    exponent = np.arange(0, dim, 2, dtype=np.float32) / np.float32(dim)
    return (np.float32(1.0) / np.power(np.float32(base), exponent, dtype=np.float32)).astype(np.float32)


def cos_sin(position_ids, dim: int, base: float = 10000.0, scaling_factor: float = 1.0):
    """cos, sin of shape ``[B, L, dim]`` float32 from ``[B, L]`` positions (llama_mlx.py:132-146)."""
    position_ids = np.asarray(position_ids)
    B, L = position_ids.shape
    pos = position_ids.reshape(-1).astype(np.float32)
    if scaling_factor != 1.0:
        pos = (pos / np.float32(scaling_factor)).astype(np.float32)
    freqs = np.outer(pos, inv_freq(dim, base)).astype(np.float32)
    emb = np.concatenate([freqs, freqs], axis=-1)
    return (
        np.cos(emb).astype(np.float32).reshape(B, L, dim),
        np.sin(emb).astype(np.float32).reshape(B, L, dim),
    )


def rotate_half(x: np.ndarray) -> np.ndarray:
    """``concat(-x[D/2:], x[:D/2])`` (llama_mlx.py:179-182)."""
    half = x.shape[-1] // 2
    return np.concatenate([-x[..., half:], x[..., :half]], axis=-1)


def apply(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """``x * cos + rotate_half(x) * sin`` for ``x`` of shape ``[B, H, L, D]`` (llama_mlx.py:170-175).

    Float32 arithmetic (MLX promotes bf16 * fp32 to fp32); the caller rounds to
    the storage dtype.
    """
    x32 = np.asarray(x, dtype=np.float32)
    c = cos[:, None, :, :]
    s = sin[:, None, :, :]
    return (x32 * c + rotate_half(x32) * s).astype(np.float32)


def apply_qk(q, k, cos, sin):
    """Rotated (q, k) as ``apply_rotary_pos_emb_mlx`` returns them (llama_mlx.py:149-176)."""
    return apply(q, cos, sin), apply(k, cos, sin)
