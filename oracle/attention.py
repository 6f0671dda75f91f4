"""NumPy restatement of the reference's chunked grouped-query attention.

Test infrastructure only (see ``oracle/__init__.py``).

Follows ``src/ollm/backends/mlx_ops.py`` of the reference:
  * ``normalize_query_positions``  -> mlx_ops.py:17-29
  * ``chunked_grouped_attention``  -> mlx_ops.py:32-152
  * ``chunked_grouped_attention_no_mask`` -> mlx_ops.py:155-178
``full_softmax_attention`` is an independent one-shot softmax used to
cross-check the chunked form; it states the same mathematics as the
reference's test oracle (tests/test_mlx_attention.py:17-40) in float64.
"""
from __future__ import annotations

import numpy as np

_NEG_INF = np.float32(-np.inf)


def normalize_query_positions(query_positions, batch_size: int, query_length: int) -> np.ndarray:
    """Broadcast ``[Lq]`` / ``[1, Lq]`` positions to ``[B, Lq]`` int32 (mlx_ops.py:17-29)."""
    pos = np.asarray(query_positions).astype(np.int32)
    if pos.ndim == 1:
        pos = pos[None, :]
    if pos.shape == (1, query_length) and batch_size > 1:
        pos = np.broadcast_to(pos, (batch_size, query_length))
    if pos.shape != (batch_size, query_length):
        raise ValueError(
            "query_positions must have shape [query_length] or "
            f"[batch, query_length], got {pos.shape}"
        )
    return pos


def _check_shapes(q, k, v, causal, q_block_size, k_block_size):
    # mlx_ops.py:48-67, same order and the same message fragments.
    if q_block_size <= 0 or k_block_size <= 0:
        raise ValueError("attention block sizes must be positive")
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
    return B, Hq, Lq, D, Hkv, Lk


def chunked_grouped_attention(
    q,
    k,
    v,
    query_positions=None,
    causal: bool = True,
    q_block_size: int = 32768,
    k_block_size: int = 1024,
    eps: float = 1e-12,
    out_dtype=None,
):
    """Blockwise online-softmax GQA with absolute query positions (mlx_ops.py:32-152).

    All arithmetic is float32, as in the reference (``astype(mx.float32)`` at
    :82-86).  A query row with no allowed key returns exactly 0 (``s == 0`` so
    ``wv / max(s, eps)`` is ``0 / eps``, :118 and :146).  The result is cast to
    ``out_dtype`` (default: ``q.dtype``, :147).
    """
    B, Hq, Lq, D, Hkv, Lk = _check_shapes(q, k, v, causal, q_block_size, k_block_size)
    positions = None
    if causal:
        if query_positions is None:
            query_positions = np.arange(Lk - Lq, Lk, dtype=np.int32)  # :69-71
        positions = normalize_query_positions(query_positions, B, Lq)
    G = Hq // Hkv
    scale = np.float32(1.0 / (D ** 0.5))
    out_dtype = q.dtype if out_dtype is None else out_dtype
    out = np.empty((B, Hq, Lq, D), dtype=out_dtype)

    for h in range(Hkv):  # :81
        kh = np.asarray(k[:, h], dtype=np.float32)
        vh = np.asarray(v[:, h], dtype=np.float32)
        qg = np.asarray(q[:, h * G:(h + 1) * G], dtype=np.float32)
        for q0 in range(0, Lq, q_block_size):  # :90
            q1 = min(Lq, q0 + q_block_size)
            qb = qg[:, :, q0:q1, :]
            m = np.full((B, G, q1 - q0), _NEG_INF, dtype=np.float32)
            s = np.zeros((B, G, q1 - q0), dtype=np.float32)
            wv = np.zeros((B, G, q1 - q0, D), dtype=np.float32)
            for k0 in range(0, Lk, k_block_size):  # :101
                k1 = min(Lk, k0 + k_block_size)
                scores = np.einsum("bhqd,bkd->bhqk", qb, kh[:, k0:k1]).astype(np.float32) * scale
                if causal:
                    kpos = np.arange(k0, k1, dtype=np.int32)
                    allowed = kpos[None, None, None, :] <= positions[:, None, q0:q1, None]
                    scores = np.where(allowed, scores, _NEG_INF)
                    local_valid = np.broadcast_to(allowed.any(axis=-1), s.shape)
                else:
                    allowed = None
                    local_valid = np.ones(s.shape, dtype=bool)
                raw_max = scores.max(axis=-1)
                local_max = np.where(local_valid, raw_max, np.float32(0.0)).astype(np.float32)
                with np.errstate(invalid="ignore"):
                    p = np.exp(scores - local_max[..., None]).astype(np.float32)
                if allowed is not None:
                    p = np.where(allowed, p, np.float32(0.0))
                sum_p = p.sum(axis=-1, dtype=np.float32)
                pv = np.einsum("bhqk,bkd->bhqd", p, vh[:, k0:k1]).astype(np.float32)

                prev_valid = s > 0  # :128
                both = prev_valid & local_valid
                new_m = np.where(both, np.maximum(m, local_max), np.where(prev_valid, m, local_max))
                with np.errstate(invalid="ignore", over="ignore"):
                    alpha = np.where(prev_valid, np.exp(m - new_m), np.float32(0.0)).astype(np.float32)
                    beta = np.where(local_valid, np.exp(local_max - new_m), np.float32(0.0)).astype(np.float32)
                s = (alpha * s + beta * sum_p).astype(np.float32)
                wv = (alpha[..., None] * wv + beta[..., None] * pv).astype(np.float32)
                m = new_m.astype(np.float32)
            denom = np.maximum(s[..., None], np.float32(eps))
            out[:, h * G:(h + 1) * G, q0:q1, :] = (wv / denom).astype(out_dtype)
    return out


def chunked_grouped_attention_no_mask(
    q, k, v, position_ids=None, q_block_size: int = 32768, k_block_size: int = 1024, eps: float = 1e-12
):
    """Unmasked compatibility entry point; ``position_ids`` is ignored (mlx_ops.py:155-178)."""
    del position_ids
    return chunked_grouped_attention(
        q, k, v, causal=False, q_block_size=q_block_size, k_block_size=k_block_size, eps=eps
    )


def full_softmax_attention(q, k, v, query_positions=None) -> np.ndarray:
    """One-shot softmax GQA in float64; rows with no allowed key give 0.

    Independent cross-check of the chunked form.  ``query_positions`` is
    ``[B, Lq]`` absolute positions or ``None`` for no mask.
    """
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    B, Hq, Lq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    out = np.zeros((B, Hq, Lq, D), dtype=np.float64)
    for hq in range(Hq):
        sc = q[:, hq] @ np.swapaxes(k[:, hq // G], 1, 2) / np.sqrt(D)
        if query_positions is not None:
            allowed = np.arange(Lk)[None, None, :] <= np.asarray(query_positions)[:, :, None]
            sc = np.where(allowed, sc, -np.inf)
        mx = sc.max(axis=-1, keepdims=True)
        mx = np.where(np.isfinite(mx), mx, 0.0)
        w = np.exp(sc - mx)
        den = w.sum(axis=-1, keepdims=True)
        w = np.divide(w, den, out=np.zeros_like(w), where=den > 0)
        out[:, hq] = w @ v[:, hq // G]
    return out


def attention_partial(q, k, v, query_positions):
    """Un-normalised state (m, s, wv) of the reference's online softmax over ONE key block, i.e. what
    mlx_ops.py:106-123 computes for a block before the merge of :125-144; rows with no allowed key have s = 0.
    q [B, Hq, Lq, D]; k, v [B, Hkv, Lk, D]; query_positions [B, Lq] in this block's own key numbering."""
    q = np.asarray(q, dtype=np.float32)
    B, Hq, Lq, D = q.shape
    Hkv, Lk = k.shape[1], k.shape[2]
    G = Hq // Hkv
    scale = np.float32(1.0 / (D ** 0.5))
    pos = normalize_query_positions(query_positions, B, Lq)
    kk = np.repeat(np.asarray(k, dtype=np.float32), G, axis=1)
    vv = np.repeat(np.asarray(v, dtype=np.float32), G, axis=1)
    scores = np.einsum("bhqd,bhkd->bhqk", q, kk).astype(np.float32) * scale
    allowed = np.arange(Lk, dtype=np.int32)[None, None, None, :] <= pos[:, None, :, None]
    scores = np.where(allowed, scores, _NEG_INF)
    valid = allowed.any(axis=-1)
    valid = np.broadcast_to(valid, scores.shape[:3])
    m = np.where(valid, scores.max(axis=-1) if Lk else _NEG_INF, np.float32(0.0)).astype(np.float32)
    with np.errstate(invalid="ignore"):
        p = np.where(allowed, np.exp(scores - m[..., None]), np.float32(0.0)).astype(np.float32)
    s = p.sum(axis=-1, dtype=np.float32)
    wv = np.einsum("bhqk,bhkd->bhqd", p, vv).astype(np.float32)
    return m, s, wv


def merge_partials(states, eps: float = 1e-12):
    """Merge (m, s, wv) states of disjoint key blocks with the rule of mlx_ops.py:125-146 and normalise."""
    m, s, wv = states[0]
    for lm, ls, lwv in states[1:]:
        prev_valid, local_valid = s > 0, ls > 0
        both = prev_valid & local_valid
        new_m = np.where(both, np.maximum(m, lm), np.where(prev_valid, m, lm))
        with np.errstate(invalid="ignore", over="ignore"):
            alpha = np.where(prev_valid, np.exp(m - new_m), np.float32(0.0)).astype(np.float32)
            beta = np.where(local_valid, np.exp(lm - new_m), np.float32(0.0)).astype(np.float32)
        s = (alpha * s + beta * ls).astype(np.float32)
        wv = (alpha[..., None] * wv + beta[..., None] * lwv).astype(np.float32)
        m = new_m.astype(np.float32)
    return (wv / np.maximum(s[..., None], np.float32(eps))).astype(np.float32)
