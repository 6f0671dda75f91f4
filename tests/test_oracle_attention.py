"""The attention oracle against the reference's own NumPy oracle outputs (golden
fixtures) and against an independent float64 softmax.  Tolerance is the
reference's: atol = rtol = 1e-5 (tests/test_mlx_attention.py:67-69)."""
import glob
import os

import numpy as np
import pytest

from oracle import attention as oa

TOL = dict(atol=1e-5, rtol=1e-5)


def _load(golden_dir, name):
    with np.load(os.path.join(golden_dir, f"attention_{name}.npz")) as d:
        return {k: d[k] for k in d.files}


@pytest.mark.parametrize("name", ["unmasked", "causal_prefill", "decode_abs_position", "gqa_d128_offsets"])
def test_chunked_matches_reference_oracle(golden_dir, name):
    c = _load(golden_dir, name)
    pos = c.get("positions")
    if int(c["causal"]):
        out = oa.chunked_grouped_attention(c["q"], c["k"], c["v"], query_positions=pos, causal=True,
                                           q_block_size=int(c["q_block"]), k_block_size=int(c["k_block"]))
    else:
        out = oa.chunked_grouped_attention_no_mask(c["q"], c["k"], c["v"], position_ids=[1, 2, 3],
                                                   q_block_size=int(c["q_block"]), k_block_size=int(c["k_block"]))
    assert out.dtype == c["q"].dtype
    assert np.allclose(c["out"], out, **TOL)
    assert np.allclose(oa.full_softmax_attention(c["q"], c["k"], c["v"], pos if int(c["causal"]) else None),
                       out, **TOL)


def test_future_values_do_not_change_earlier_outputs(golden_dir):
    c = _load(golden_dir, "future_values")
    a = oa.chunked_grouped_attention(c["q"], c["k"], c["v"], k_block_size=2)
    b = oa.chunked_grouped_attention(c["q"], c["k"], c["v_changed"], k_block_size=2)
    assert np.allclose(a, c["out"], **TOL) and np.allclose(b, c["out_changed"], atol=1e-2, rtol=1e-5)
    assert np.allclose(a[:, :, :3], b[:, :, :3])
    assert not np.allclose(a[:, :, 3:], b[:, :, 3:])


def test_default_positions_are_bottom_right_aligned():
    rng = np.random.default_rng(3)
    q = rng.standard_normal((1, 2, 3, 8), dtype=np.float32)
    k = rng.standard_normal((1, 1, 10, 8), dtype=np.float32)
    v = rng.standard_normal((1, 1, 10, 8), dtype=np.float32)
    a = oa.chunked_grouped_attention(q, k, v, k_block_size=4)
    b = oa.chunked_grouped_attention(q, k, v, query_positions=[7, 8, 9], k_block_size=3)
    assert np.allclose(a, b, **TOL)


def test_fully_masked_row_is_zero_not_nan():
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 2, 2, 4), dtype=np.float32)
    k = rng.standard_normal((1, 2, 5, 4), dtype=np.float32)
    out = oa.chunked_grouped_attention(q, k, k, query_positions=[[-1, 2]], k_block_size=2)
    assert np.array_equal(out[:, :, 0], np.zeros_like(out[:, :, 0]))
    assert np.isfinite(out).all() and np.abs(out[:, :, 1]).max() > 0


def test_block_size_independence():
    rng = np.random.default_rng(5)
    q = rng.standard_normal((2, 4, 9, 16), dtype=np.float32)
    k = rng.standard_normal((2, 2, 21, 16), dtype=np.float32)
    v = rng.standard_normal((2, 2, 21, 16), dtype=np.float32)
    base = oa.chunked_grouped_attention(q, k, v, q_block_size=32768, k_block_size=1000000)
    for qb, kb in [(1, 1), (2, 5), (4, 8), (9, 21)]:
        assert np.allclose(base, oa.chunked_grouped_attention(q, k, v, q_block_size=qb, k_block_size=kb), **TOL)


def test_rejections_carry_reference_messages():
    one = np.ones((1, 3, 2, 4), dtype=np.float32)
    kv = np.ones((1, 2, 2, 4), dtype=np.float32)
    with pytest.raises(ValueError, match="divisible"):
        oa.chunked_grouped_attention(one, kv, kv)
    q = np.ones((1, 2, 3, 4), dtype=np.float32)
    with pytest.raises(ValueError, match="key length >= query length"):
        oa.chunked_grouped_attention(q, kv, kv)
    with pytest.raises(ValueError, match="block sizes must be positive"):
        oa.chunked_grouped_attention(q, kv, kv, k_block_size=0)
    with pytest.raises(ValueError, match="query_positions must have shape"):
        oa.chunked_grouped_attention(q[:, :, :2], kv, kv, query_positions=np.zeros((3, 2)))
    with pytest.raises(ValueError, match="share last-dim"):
        oa.chunked_grouped_attention(np.ones((1, 2, 2, 8), dtype=np.float32), kv, kv)


def test_all_fixture_files_are_covered(golden_dir):
    names = {os.path.basename(p) for p in glob.glob(os.path.join(golden_dir, "attention_*.npz"))}
    assert names == {f"attention_{n}.npz" for n in
                     ["unmasked", "causal_prefill", "decode_abs_position", "future_values", "gqa_d128_offsets"]}
