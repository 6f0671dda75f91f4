"""Attention kernels on the GPU, through the C ABI, against the oracle, the reference's own oracle
outputs (golden fixtures) and the reference's attention tests (tests/test_mlx_attention.py:53-137)."""
import os

import numpy as np
import pytest
import torch

import lokahi_b200 as L
from oracle import attention as oattn
from oracle import paged as opaged
from parity import TOL_BF16, TOL_F32, assert_parity, bf16_round, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def _load(golden_dir, name):
    with np.load(os.path.join(golden_dir, f"attention_{name}.npz")) as d:
        return {k: d[k] for k in d.files}


# ---- dense attention: reference fixtures (tolerance of the reference's tests: 1e-5) ----------------
@pytest.mark.parametrize("name", ["unmasked", "causal_prefill", "decode_abs_position", "gqa_d128_offsets"])
def test_dense_attention_matches_reference_fixtures(golden_dir, name):
    c = _load(golden_dir, name)
    q, k, v = _t(c["q"]), _t(c["k"]), _t(c["v"])
    if int(c["causal"]):
        out = L.chunked_grouped_attention(q, k, v, query_positions=c["positions"], causal=True,
                                          q_block_size=int(c["q_block"]), k_block_size=int(c["k_block"]))
    else:
        out = L.chunked_grouped_attention_no_mask(q, k, v, position_ids=[0], q_block_size=int(c["q_block"]),
                                                  k_block_size=int(c["k_block"]))
    assert out.dtype == q.dtype and out.shape == q.shape
    assert np.allclose(c["out"], to_np(out), atol=1e-5, rtol=1e-5)


def test_future_values_do_not_change_earlier_outputs(golden_dir):
    c = _load(golden_dir, "future_values")
    q, k = _t(c["q"]), _t(c["k"])
    a = to_np(L.chunked_grouped_attention(q, k, _t(c["v"]), k_block_size=2))
    b = to_np(L.chunked_grouped_attention(q, k, _t(c["v_changed"]), k_block_size=2))
    assert np.allclose(a, c["out"], atol=1e-5, rtol=1e-5)
    assert np.allclose(a[:, :, :3], b[:, :, :3]) and not np.allclose(a[:, :, 3:], b[:, :, 3:])


def test_rejections_carry_reference_messages():
    ones = lambda *s: torch.ones(*s, device=DEV)
    with pytest.raises(ValueError, match="divisible"):
        L.chunked_grouped_attention(ones(1, 3, 2, 4), ones(1, 2, 2, 4), ones(1, 2, 2, 4))
    with pytest.raises(ValueError, match="key length >= query length"):
        L.chunked_grouped_attention(ones(1, 2, 3, 4), ones(1, 2, 2, 4), ones(1, 2, 2, 4))
    with pytest.raises(ValueError, match="block sizes must be positive"):
        L.chunked_grouped_attention(ones(1, 2, 2, 4), ones(1, 2, 2, 4), ones(1, 2, 2, 4), k_block_size=0)
    with pytest.raises(ValueError, match="query_positions must have shape"):
        L.chunked_grouped_attention(ones(1, 2, 2, 4), ones(1, 2, 2, 4), ones(1, 2, 2, 4), query_positions=np.zeros((3, 2)))
    with pytest.raises(ValueError, match="share last-dim"):
        L.chunked_grouped_attention(ones(1, 2, 2, 8), ones(1, 2, 2, 4), ones(1, 2, 2, 4))


def test_fully_masked_rows_are_zero():
    rng = np.random.default_rng(4)
    q = rng.standard_normal((1, 2, 2, 4), dtype=np.float32)
    k = rng.standard_normal((1, 2, 5, 4), dtype=np.float32)
    out = to_np(L.chunked_grouped_attention(_t(q), _t(k), _t(k), query_positions=[[-1, 2]]))
    ref = oattn.chunked_grouped_attention(q, k, k, query_positions=[[-1, 2]])
    assert np.array_equal(out[:, :, 0], np.zeros_like(out[:, :, 0])) and np.allclose(out, ref, atol=1e-5)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
@pytest.mark.parametrize("shape", [(2, 4, 2, 33, 70, 64), (1, 8, 2, 130, 130, 128), (1, 2, 2, 1, 257, 96)])
def test_dense_attention_matches_oracle(dtype, tol, shape):
    B, Hq, Hkv, Lq, Lk, D = shape
    rng = np.random.default_rng(Lq * 7 + D)
    rnd = (lambda a: a) if dtype == torch.float32 else bf16_round
    q = rnd(rng.standard_normal((B, Hq, Lq, D), dtype=np.float32))
    k = rnd(rng.standard_normal((B, Hkv, Lk, D), dtype=np.float32))
    v = rnd(rng.standard_normal((B, Hkv, Lk, D), dtype=np.float32))
    for causal in (True, False):
        out = L.chunked_grouped_attention(_t(q, dtype), _t(k, dtype), _t(v, dtype), causal=causal)
        ref = oattn.chunked_grouped_attention(q, k, v, causal=causal, k_block_size=64)
        assert_parity(out, ref, tol, f"dense causal={causal}")


# ---- paged decode ----------------------------------------------------------------------------------------
def _paged_setup(rng, dtype, n_seqs, Hkv, D, P, lens, n_pages=None, layers=1, headroom=0):
    pages_per_seq = max(1, max(-(-(t + 1 + headroom) // P) for t in lens))
    n_pages = n_pages or n_seqs * pages_per_seq + 3
    pool = L.PagedPool(L.PagedKVConfig(num_layers=layers, num_kv_heads=Hkv, head_dim=D, num_pages=n_pages, max_seqs=n_seqs,
                                       max_pages_per_seq=pages_per_seq, page_size=P, dtype=dtype))
    perm = rng.permutation(n_pages)
    rnd = (lambda a: a) if dtype == torch.float32 else bf16_round
    k_ref = rnd(rng.standard_normal((n_pages, Hkv, P, D), dtype=np.float32))
    v_ref = rnd(rng.standard_normal((n_pages, Hkv, P, D), dtype=np.float32))
    table = np.full((n_seqs, pages_per_seq), -1, np.int32)
    for s in range(n_seqs):
        assert pool.alloc_sequence() == s
        pages = perm[s * pages_per_seq:(s + 1) * pages_per_seq]
        table[s] = pages
        pool.set_page_table(s, pages.tolist(), lens[s])
    kp, vp = pool.layer_views(layers - 1)
    kp.copy_(_t(k_ref, dtype)); vp.copy_(_t(v_ref, dtype))
    return pool, k_ref, v_ref, table, rnd


@pytest.mark.parametrize("dtype,tol,D,Hq,Hkv", [
    (torch.bfloat16, TOL_BF16, 128, 32, 8),     # tensor-core kernel, the benchmark's head geometry
    (torch.bfloat16, TOL_BF16, 128, 16, 16),    # MHA through the tensor-core kernel
    (torch.bfloat16, TOL_BF16, 64, 8, 2),       # CUDA-core kernel, bf16
    (torch.float32, TOL_F32, 64, 4, 2),         # two-layer fixture geometry, float32
    (torch.float32, TOL_F32, 6, 4, 2),          # the reference tests' head_dim
])
def test_paged_decode_matches_oracle_on_ragged_lengths(dtype, tol, D, Hq, Hkv):
    rng = np.random.default_rng(D + Hq)
    P = 16
    lens = [1, 2, 15, 16, 17, 31, 32, 33, 64, 100, 257, 700, 1024, 1500]
    pool, k_ref, v_ref, table, rnd = _paged_setup(rng, dtype, len(lens), Hkv, D, P, lens, layers=2)
    q = rnd(rng.standard_normal((len(lens), Hq, D), dtype=np.float32))
    out = pool.decode_attention(1, _t(q, dtype))
    ref = opaged.paged_decode_attention(q, k_ref, v_ref, table, np.array(lens), out_dtype=np.float32)
    assert pool.check_device_status() == 0
    assert_parity(out, ref, tol, "paged decode")
    # absolute query positions below the newest token restrict the keys (mlx_ops.py:107-112)
    qpos = [max(0, t - 1 - (i % 5) * 3) for i, t in enumerate(lens)]
    out2 = pool.decode_attention(1, _t(q, dtype), q_pos=qpos)
    ref2 = opaged.paged_decode_attention(q, k_ref, v_ref, table, np.array(lens), q_positions=qpos, out_dtype=np.float32)
    assert_parity(out2, ref2, tol, "paged decode with absolute positions")
    # a subset of sequences in another order
    ids = [13, 0, 7]
    out3 = pool.decode_attention(1, _t(q[:3], dtype), seq_ids=ids)
    ref3 = opaged.paged_decode_attention(q[:3], k_ref, v_ref, table, np.array(lens), seq_ids=ids, out_dtype=np.float32)
    assert_parity(out3, ref3, tol, "paged decode with sequence ids")


def test_paged_decode_kernels_agree_and_empty_sequences_give_zero(skv_switch):
    rng = np.random.default_rng(3)
    lens = [0, 5, 48, 333]
    pool, k_ref, v_ref, table, rnd = _paged_setup(rng, torch.bfloat16, len(lens), 8, 128, 16, lens)
    q = _t(rnd(rng.standard_normal((len(lens), 32, 128), dtype=np.float32)), torch.bfloat16)
    a = pool.decode_attention(0, q)
    assert not to_np(a[0]).any()
    skv_switch("SKV_DECODE_GENERIC", "1")
    b = pool.decode_attention(0, q)
    skv_switch("SKV_DECODE_GENERIC", None)
    assert_parity(a, to_np(b), TOL_BF16, "tensor-core vs CUDA-core decode")
    ref = opaged.paged_decode_attention(to_np(q), k_ref, v_ref, table, np.array(lens), out_dtype=np.float32)
    assert_parity(b, ref, TOL_BF16, "CUDA-core decode")
    q_neg = pool.decode_attention(0, q, q_pos=[-1, -1, -1, -1])
    assert not to_np(q_neg).any()


def test_cache_update_then_attention_like_the_reference_call_site():
    """QKV -> RoPE -> cache.update -> attention with position_ids, as llama_mlx.py:284-308, prefill then decode."""
    from types import SimpleNamespace
    rng = np.random.default_rng(12)
    B, Hq, Hkv, D, Lp = 2, 4, 2, 64, 37
    cfg = SimpleNamespace(num_hidden_layers=1, max_position_embeddings=128)
    cache = L.PagedKVCache(cfg, cache_dir=None)
    from oracle.kvcache import ConcatKVCache
    ref_cache = ConcatKVCache(cfg, cache_dir=None)
    attn = L.B200Backend().attention_kernel()
    for step, Lnew in enumerate([Lp, 1, 1, 1]):
        past = cache.get_seq_length(0)
        q = rng.standard_normal((B, Hq, Lnew, D), dtype=np.float32)
        k = rng.standard_normal((B, Hkv, Lnew, D), dtype=np.float32)
        v = rng.standard_normal((B, Hkv, Lnew, D), dtype=np.float32)
        pos = np.arange(past, past + Lnew, dtype=np.int32)
        kk, vv = cache.update(_t(k), _t(v), 0, {"cache_position": torch.from_numpy(pos)})
        rk, rv = ref_cache.update(k, v, 0, {"cache_position": pos})
        out = attn(_t(q), kk, vv, query_positions=pos[None], causal=True, q_block_size=32768,
                   k_block_size=(1024 if Lnew > 128 else 1000000))
        ref = oattn.chunked_grouped_attention(q, rk, rv, query_positions=pos[None], causal=True,
                                              k_block_size=(1024 if Lnew > 128 else 1000000))
        assert_parity(out, ref, TOL_F32, f"step {step}")
        assert np.array_equal(to_np(kk.materialize()), rk)
    assert cache.get_seq_length() == Lp + 3


def test_full_size_paged_decode_properties():
    """At the benchmark's full size (64 sequences, contexts 512..8192, 32/8 heads, D 128, bf16):
    oracle parity on a sample of sequences and the sum-to-one property of the softmax weights."""
    rng = np.random.default_rng(2024)
    n_seqs, Hq, Hkv, D, P = 64, 32, 8, 128, 16
    lens = rng.integers(512, 8193, size=n_seqs)
    pages_per_seq = int(-(-(lens.max() + 1) // P))
    n_pages = int(sum(-(-(int(t) + 1) // P) for t in lens)) + 8
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=n_pages, max_seqs=n_seqs,
                                       max_pages_per_seq=pages_per_seq, page_size=P, dtype=torch.bfloat16))
    perm = rng.permutation(n_pages)
    table = np.full((n_seqs, pages_per_seq), -1, np.int32)
    at = 0
    for s in range(n_seqs):
        n = -(-(int(lens[s]) + 1) // P)
        table[s, :n] = perm[at:at + n]
        at += n
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, table[s, :n].tolist(), int(lens[s]))
    kp, vp = pool.layer_views(0)
    gen = torch.Generator(device=DEV).manual_seed(7)
    kp.copy_(torch.randn(kp.shape, generator=gen, device=DEV, dtype=torch.float32))
    vp.copy_(torch.randn(vp.shape, generator=gen, device=DEV, dtype=torch.float32))
    q = bf16_round(rng.standard_normal((n_seqs, Hq, D), dtype=np.float32))
    out = pool.decode_attention(0, _t(q, torch.bfloat16))
    assert pool.check_device_status() == 0
    sample = [0, 17, int(np.argmax(lens)), int(np.argmin(lens))]
    for s in sample:   # the oracle reads only this sequence's pages
        n = -(-int(lens[s]) // P)
        pages = torch.from_numpy(table[s, :n].astype(np.int64)).to(DEV)
        k_s, v_s = to_np(kp[pages]), to_np(vp[pages])
        local = np.arange(n, dtype=np.int32)[None]
        ref = opaged.paged_decode_attention(q[s:s + 1], k_s, v_s, local, np.array([lens[s]]), out_dtype=np.float32)
        assert_parity(out[s:s + 1], ref, TOL_BF16, f"full-size sequence {s}")
    # softmax weights sum to one: with V == 1 everywhere every output element is 1 (up to bf16 rounding of P)
    vp.fill_(1.0)
    ones = to_np(pool.decode_attention(0, _t(q, torch.bfloat16)))
    assert np.abs(ones - 1.0).max() <= 2e-2
    assert pool.check_device_status() == 0


# ---- tensor-core (tcgen05) prefill kernel ---------------------------------------------------------------
@pytest.mark.parametrize("shape,causal", [
    ((1, 8, 2, 256, 256, 128), True),       # GQA, two query tiles, diagonal tiles masked
    ((2, 4, 4, 200, 333, 128), True),       # ragged tile tails on both axes, bottom-right alignment
    ((1, 4, 2, 130, 130, 128), False),      # unmasked twin
    ((1, 2, 1, 64, 700, 128), True),        # chunked prefill against a long history
])
def test_tensor_core_prefill_matches_oracle(shape, causal):
    B, Hq, Hkv, Lq, Lk, D = shape
    rng = np.random.default_rng(Lq + Lk)
    q = bf16_round(rng.standard_normal((B, Hq, Lq, D), dtype=np.float32))
    k = bf16_round(rng.standard_normal((B, Hkv, Lk, D), dtype=np.float32))
    v = bf16_round(rng.standard_normal((B, Hkv, Lk, D), dtype=np.float32))
    out = L.chunked_grouped_attention(_t(q, torch.bfloat16), _t(k, torch.bfloat16), _t(v, torch.bfloat16), causal=causal)
    ref = oattn.chunked_grouped_attention(q, k, v, causal=causal, k_block_size=128)
    assert_parity(out, ref, TOL_BF16, "tcgen05 prefill")


def test_tensor_core_prefill_absolute_positions_and_masked_rows(skv_switch):
    rng = np.random.default_rng(77)
    B, Hq, Hkv, Lq, Lk, D = 2, 4, 2, 96, 300, 128
    q = bf16_round(rng.standard_normal((B, Hq, Lq, D), dtype=np.float32))
    k = bf16_round(rng.standard_normal((B, Hkv, Lk, D), dtype=np.float32))
    v = bf16_round(rng.standard_normal((B, Hkv, Lk, D), dtype=np.float32))
    pos = rng.integers(-1, Lk + 5, size=(B, Lq)).astype(np.int32)     # includes rows with no allowed key and rows past Lk
    pos[0, 0] = -1
    out = L.chunked_grouped_attention(_t(q, torch.bfloat16), _t(k, torch.bfloat16), _t(v, torch.bfloat16), query_positions=pos)
    ref = oattn.chunked_grouped_attention(q, k, v, query_positions=pos, k_block_size=64)
    assert_parity(out, ref, TOL_BF16, "tcgen05 prefill, per-row positions")
    assert not to_np(out[0, :, 0]).any(), "a row with no allowed key is exactly 0"
    skv_switch("SKV_PREFILL_GENERIC", "1")
    gen = L.chunked_grouped_attention(_t(q, torch.bfloat16), _t(k, torch.bfloat16), _t(v, torch.bfloat16), query_positions=pos)
    assert_parity(out, to_np(gen), TOL_BF16, "tcgen05 vs CUDA-core prefill")


def test_tensor_core_prefill_at_full_sequence_4096(skv_switch):
    """The stand-alone chunked-GQA configuration (32 query heads, 8 KV heads, head_dim 128, sequence 4096, bf16):
    oracle parity on a sample of heads / row blocks, agreement with the CUDA-core kernel on all of it, and
    causality (changing future V leaves earlier rows untouched)."""
    gen = torch.Generator(device=DEV).manual_seed(4096)
    B, Hq, Hkv, S, D = 1, 32, 8, 4096, 128
    q = torch.randn((B, Hq, S, D), generator=gen, device=DEV).to(torch.bfloat16)
    k = torch.randn((B, Hkv, S, D), generator=gen, device=DEV).to(torch.bfloat16)
    v = torch.randn((B, Hkv, S, D), generator=gen, device=DEV).to(torch.bfloat16)
    pos = np.arange(S, dtype=np.int32)
    out = L.chunked_grouped_attention(q, k, v, query_positions=pos, causal=True, q_block_size=512, k_block_size=512)
    for hq, r0 in [(0, 0), (13, 1900), (31, 3968)]:      # oracle on 128-row blocks of three heads
        hk = hq // 4
        ref = oattn.chunked_grouped_attention(to_np(q[:, hq:hq + 1, r0:r0 + 128]), to_np(k[:, hk:hk + 1]), to_np(v[:, hk:hk + 1]),
                                              query_positions=pos[r0:r0 + 128], q_block_size=512, k_block_size=512)
        assert_parity(out[:, hq:hq + 1, r0:r0 + 128], ref, TOL_BF16, f"S=4096 head {hq} rows {r0}")
    v2 = v.clone()
    v2[:, :, 3000:] += 1000.0
    out2 = L.chunked_grouped_attention(q, k, v2, query_positions=pos, causal=True)
    assert torch.equal(out[:, :, :3000], out2[:, :, :3000]) and not torch.equal(out[:, :, 3000:], out2[:, :, 3000:])
    skv_switch("SKV_PREFILL_GENERIC", "1")
    ref_all = L.chunked_grouped_attention(q[:, ::8], k[:, ::2], v[:, ::2], query_positions=pos, causal=True)
    # both sides are bf16-rounded, so element-wise they may sit two roundings apart: normalised error only
    from parity import parity_errors
    assert parity_errors(out[:, ::8], to_np(ref_all))[0] <= TOL_BF16, "tcgen05 vs CUDA-core at S=4096"


@pytest.mark.parametrize("P", [16, 32, 48, 64])
def test_tensor_core_prefill_over_pages_matches_oracle_and_the_dense_kernel(skv_switch, P):
    """bf16, head_dim 128, pages of a multiple of 16 tokens, at least 32 query rows: the tcgen05 kernel reads K/V
    straight from the scattered pages (in groups of 16 tokens, which never straddle a page).  Ragged lengths (one
    shorter than a key tile, one not a multiple of the page size), default bottom-right positions and explicit
    ones (with fully masked rows), against the oracle on the logical history and against the float32 CUDA-core
    kernel."""
    rng = np.random.default_rng(91)
    lens = [40, 64, 200, 777, 1030]
    n, Hq, Hkv, D, Lq = len(lens), 8, 2, 128, 40
    pool, k_ref, v_ref, table, rnd = _paged_setup(rng, torch.bfloat16, n, Hkv, D, P, lens)
    q = _t(rnd(rng.standard_normal((n, Hq, Lq, D), dtype=np.float32)), torch.bfloat16)
    before = L._lib.lib.skv_launch_count()
    out = pool.prefill_attention(0, q)                                   # positions default to Lk - Lq + i
    assert L._lib.lib.skv_launch_count() - before == 1
    skv_switch("SKV_PREFILL_GENERIC", "1")
    out_generic = pool.prefill_attention(0, q)
    skv_switch("SKV_PREFILL_GENERIC", None)
    from parity import parity_errors
    assert parity_errors(out, to_np(out_generic))[0] <= TOL_BF16
    for i, t in enumerate(lens):
        k_log = opaged.logical_kv(k_ref, table[i], t)[None]
        v_log = opaged.logical_kv(v_ref, table[i], t)[None]
        ref = oattn.chunked_grouped_attention(to_np(q[i:i + 1]), k_log, v_log, q_block_size=16, k_block_size=64)
        assert_parity(out[i:i + 1], ref, TOL_BF16, f"paged tensor-core prefill, sequence {i} (length {t})")
    # explicit absolute positions: some rows see nothing (-1), some see everything, the rest are scattered
    pos = rng.integers(-1, 1100, size=(n, Lq)).astype(np.int32)
    pos[:, 0] = -1
    pos[:, 1] = 5000
    out2 = pool.prefill_attention(0, q, positions=_t(pos, torch.int32))
    assert pool.check_device_status() == 0
    for i, t in enumerate(lens):
        k_log = opaged.logical_kv(k_ref, table[i], t)[None]
        v_log = opaged.logical_kv(v_ref, table[i], t)[None]
        ref = oattn.chunked_grouped_attention(to_np(q[i:i + 1]), k_log, v_log, query_positions=pos[i:i + 1],
                                              q_block_size=16, k_block_size=64)
        assert_parity(out2[i:i + 1], ref, TOL_BF16, f"paged tensor-core prefill with positions, sequence {i}")
        assert torch.count_nonzero(out2[i, :, 0]) == 0, "a row with no allowed key is exactly 0"


def test_decode_step_equals_append_then_attention(skv_switch):
    skv_switch("SKV_STEP_FUSED", "0")     # the two-call form of the step: bit-identical to its parts
    rng = np.random.default_rng(55)
    lens = [5, 16, 300, 1025]
    pool_a, k_ref, v_ref, table, rnd = _paged_setup(rng, torch.bfloat16, len(lens), 8, 128, 16, lens)
    rng = np.random.default_rng(55)
    pool_b, _, _, _, _ = _paged_setup(rng, torch.bfloat16, len(lens), 8, 128, 16, lens)
    for p in (pool_a, pool_b):
        p.set_rope(L.rope_inv_freq(128, 500000.0))
    q = _t(rnd(rng.standard_normal((len(lens), 32, 128), dtype=np.float32)), torch.bfloat16)
    k = _t(rnd(rng.standard_normal((len(lens), 8, 128), dtype=np.float32)), torch.bfloat16)
    v = _t(rnd(rng.standard_normal((len(lens), 8, 128), dtype=np.float32)), torch.bfloat16)
    qa, qb = q.clone(), q.clone()
    pool_a.append(0, k, v, start_pos=lens, rope_k=True, q=qa, layout="bhd")
    out_a = pool_a.decode_attention(0, qa)
    out_b = pool_b.decode_step(0, qb, k, v)
    assert torch.equal(qa, qb) and torch.equal(out_a, out_b)
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0)) and pool_b.check_device_status() == 0


def test_fused_append_step_matches_the_two_launch_step_and_the_oracle(skv_switch):
    """The one-kernel step (RoPE of q and of the new K row, the store into the page and the new token's score all
    inside the decode kernel) against append + attention, over 20 steps that cross page, chunk and empty-sequence
    boundaries: rotated q and the stored pages bit-equal, outputs within bf16 tolerance of each other and of the
    oracle on the logical history."""
    lens = [0, 5, 15, 16, 255, 256, 300, 1023, 2047, 2048]
    n, Hq, Hkv, D, P = len(lens), 32, 8, 128, 16
    rng = np.random.default_rng(56)
    pool_a, k_ref, v_ref, table, rnd = _paged_setup(rng, torch.bfloat16, n, Hkv, D, P, lens, headroom=20)
    rng = np.random.default_rng(56)
    pool_b, _, _, _, _ = _paged_setup(rng, torch.bfloat16, n, Hkv, D, P, lens, headroom=20)
    inv = L.rope_inv_freq(D, 500000.0)
    for p in (pool_a, pool_b):
        p.set_rope(inv)
    from parity import parity_errors
    launches = []
    for step in range(20):
        q = _t(rnd(rng.standard_normal((n, Hq, D), dtype=np.float32)), torch.bfloat16)
        k = _t(rnd(rng.standard_normal((n, Hkv, D), dtype=np.float32)), torch.bfloat16)
        v = _t(rnd(rng.standard_normal((n, Hkv, D), dtype=np.float32)), torch.bfloat16)
        qa, qb = q.clone(), q.clone()
        skv_switch("SKV_STEP_FUSED", "0")
        out_a = pool_a.decode_step(0, qa, k, v)
        skv_switch("SKV_STEP_FUSED", "1")
        before = L._lib.lib.skv_launch_count()
        out_b = pool_b.decode_step(0, qb, k, v)
        launches.append(L._lib.lib.skv_launch_count() - before)
        assert torch.equal(qa, qb), f"rotated q differs at step {step}"
        assert parity_errors(out_b, to_np(out_a))[0] <= TOL_BF16, f"step {step}"
        assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0))
    assert max(launches) == 2, "the fused step is the decode kernel and the merge kernel, nothing else"
    ka, va = pool_a.gather(0, n_seqs=n)
    kb, vb = pool_b.gather(0, n_seqs=n)
    final = [t + 20 for t in lens]
    for i in range(n):
        assert torch.equal(ka[i, :, :final[i]], kb[i, :, :final[i]]) and torch.equal(va[i, :, :final[i]], vb[i, :, :final[i]]), \
            f"stored pages of sequence {i} differ"
    assert pool_b.check_device_status() == 0
    # last step against the oracle on the logical history read back from the pages
    k_np, v_np = to_np(kb), to_np(vb)
    for i in (0, 3, 9):
        ref = oattn.chunked_grouped_attention(to_np(qb[i])[None, :, None, :], k_np[i:i + 1, :, :final[i]], v_np[i:i + 1, :, :final[i]],
                                              query_positions=np.array([final[i] - 1], dtype=np.int32))
        assert_parity(out_b[i], ref[0, :, 0, :], TOL_BF16, f"fused step vs oracle, sequence {i}")


def test_fused_gather_path_on_one_gpu_matches_plain_decode():
    """world == 1 runs the same merge-kernel code (stores into the receive buffer, polling, unpacking) against
    local buffers."""
    rng = np.random.default_rng(71)
    lens = [1, 40, 777, 2050, 0]
    pool, k_ref, v_ref, table, rnd = _paged_setup(rng, torch.bfloat16, len(lens), 8, 128, 16, lens)
    q = _t(rnd(rng.standard_normal((len(lens), 32, 128), dtype=np.float32)), torch.bfloat16)
    expect = pool.decode_attention(0, q)
    gather = L.PeerGather(L.HeadShard(0, 1, 32, 8), len(lens), 128, torch.bfloat16, torch.device(DEV))
    for _ in range(3):     # epochs 1..3 alternate between the two gathered buffers
        view = pool.decode_attention_xchg(0, q, gather)
        torch.cuda.synchronize()
        assert torch.equal(view[0], expect)
    assert gather.epoch == 3 and pool.check_device_status() == 0


def test_sequence_sharding_partials_merge_to_the_unsharded_result():
    """Three pools on one GPU stand in for three ranks that each hold a contiguous, page-aligned token range of
    every sequence: local partials + merge must equal decode attention over the whole history, and each local
    partial must equal the oracle's block state."""
    rng = np.random.default_rng(123)
    R, n, Hq, Hkv, D, P, span = 3, 4, 32, 8, 128, 16, 512
    lens = [5, 512, 700, 1400]
    qpos = [4, 511, 650, 1399]
    rnd = bf16_round
    k_hist = [rnd(rng.standard_normal((Hkv, t, D), dtype=np.float32)) for t in lens]
    v_hist = [rnd(rng.standard_normal((Hkv, t, D), dtype=np.float32)) for t in lens]
    q = rnd(rng.standard_normal((n, Hq, D), dtype=np.float32))
    qt = _t(q, torch.bfloat16)

    def pool_for(first, count_of):
        pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=n * 100, max_seqs=n,
                                           max_pages_per_seq=100, page_size=P, dtype=torch.bfloat16))
        for s in range(n):
            assert pool.alloc_sequence() == s
            cnt = count_of(s)
            if cnt > 0:
                pool.append(0, _t(k_hist[s][None, :, first:first + cnt], torch.bfloat16),
                            _t(v_hist[s][None, :, first:first + cnt], torch.bfloat16), seq_ids=[s], start_pos=[0])
        return pool

    whole = pool_for(0, lambda s: lens[s]).decode_attention(0, qt, q_pos=qpos)
    parts, states = [], [[] for _ in range(n)]
    for r in range(R):
        sh = L.SequenceShard(r, R, span, P)
        pool = pool_for(r * span, lambda s: sh.local_range(lens[s])[1])
        parts.append(pool.decode_partial(0, qt, q_pos=[sh.local_position(p) for p in qpos]))
        for s in range(n):
            first, cnt = sh.local_range(lens[s])
            states[s].append(oattn.attention_partial(q[s][None, :, None, :], k_hist[s][None, :, first:first + cnt],
                                                     v_hist[s][None, :, first:first + cnt], [[sh.local_position(qpos[s])]]))
        assert pool.check_device_status() == 0
    merged = L.merge_partials(torch.stack(parts).contiguous())
    assert_parity(merged, to_np(whole), TOL_BF16, "merged partials vs unsharded decode")
    ref = np.stack([oattn.merge_partials(states[s])[0, :, 0, :] for s in range(n)])
    assert_parity(merged, ref, TOL_BF16, "merged partials vs oracle merge")
    # the l of a rank that holds none of the allowed keys is exactly 0
    assert float(parts[2][0, :, D + 1].abs().max()) == 0.0 and float(parts[1][0, :, D + 1].abs().max()) == 0.0
    # world == 1 path of the helper
    one = L.sequence_sharded_decode(pool_for(0, lambda s: lens[s]), 0, qt, qpos, L.SequenceShard(0, 1, 2048, P))
    assert_parity(one, to_np(whole), TOL_BF16, "single-rank sequence sharding")


def test_fused_step_is_all_or_nothing_when_pages_run_out():
    """A step that needs a fresh page for some sequences while the pool has too few free ones fails with
    OutOfPagesError before anything is launched or changed; after a sequence is freed the same step succeeds."""
    rng = np.random.default_rng(57)
    n, Hq, Hkv, D, P = 3, 8, 2, 128, 16
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=4, max_seqs=4,
                                       max_pages_per_seq=4, page_size=P, dtype=torch.bfloat16))
    pool.set_rope(L.rope_inv_freq(D, 10000.0))
    rnd = bf16_round
    for s in range(n):                                  # 16 tokens each: three full pages, one page left
        assert pool.alloc_sequence() == s
        kv = _t(rnd(rng.standard_normal((1, Hkv, P, D), dtype=np.float32)), torch.bfloat16)
        pool.append(0, kv, kv, seq_ids=[s], start_pos=[0])
    q = _t(rnd(rng.standard_normal((n, Hq, D), dtype=np.float32)), torch.bfloat16)
    k = _t(rnd(rng.standard_normal((n, Hkv, D), dtype=np.float32)), torch.bfloat16)
    v = _t(rnd(rng.standard_normal((n, Hkv, D), dtype=np.float32)), torch.bfloat16)
    q_before, lens_before, free_before = q.clone(), pool.lengths(0).copy(), pool.counters()["free_pages"]
    with pytest.raises(L.OutOfPagesError):
        pool.decode_step(0, q, k, v)                    # needs three pages, one is free
    torch.cuda.synchronize()
    assert torch.equal(q, q_before) and np.array_equal(pool.lengths(0), lens_before)
    assert pool.counters()["free_pages"] == free_before and pool.check_device_status() == 0
    # two sequences fit: the step runs for 0..1 after sequence 2 gave its page back
    pool.free_sequence(2)
    out = pool.decode_step(0, q[:2].contiguous(), k[:2].contiguous(), v[:2].contiguous())
    assert out.shape == (2, Hq, D) and list(pool.lengths(0)[:2]) == [P + 1, P + 1] and pool.check_device_status() == 0


def test_one_call_step_with_a_sequence_list_matches_the_two_calls(monkeypatch):
    """A subset of the live sequences in a shuffled order: the two-launch step against append + attention with the
    same list, for five steps; stored pages, lengths (also of the untouched sequences) and rotated q identical,
    outputs within bf16 tolerance; a repeated id is rejected."""
    lens = [3, 700, 16, 255, 1024, 90]
    ids = [4, 1, 5, 2]
    n, Hq, Hkv, D, P = len(lens), 32, 8, 128, 16
    rng = np.random.default_rng(58)
    pool_a, _, _, _, rnd = _paged_setup(rng, torch.bfloat16, n, Hkv, D, P, lens, headroom=8)
    rng = np.random.default_rng(58)
    pool_b, _, _, _, _ = _paged_setup(rng, torch.bfloat16, n, Hkv, D, P, lens, headroom=8)
    inv = L.rope_inv_freq(D, 500000.0)
    for p in (pool_a, pool_b):
        p.set_rope(inv)
    from parity import parity_errors
    for step in range(5):
        q = _t(rnd(rng.standard_normal((len(ids), Hq, D), dtype=np.float32)), torch.bfloat16)
        k = _t(rnd(rng.standard_normal((len(ids), Hkv, D), dtype=np.float32)), torch.bfloat16)
        v = _t(rnd(rng.standard_normal((len(ids), Hkv, D), dtype=np.float32)), torch.bfloat16)
        qa, qb = q.clone(), q.clone()
        pool_a.append(0, k, v, seq_ids=ids, start_pos=[lens[s] + step for s in ids], rope_k=True, q=qa, layout="bhd")
        out_a = pool_a.decode_attention(0, qa, seq_ids=ids)
        before = L._lib.lib.skv_launch_count()
        out_b = pool_b.decode_step(0, qb, k, v, seq_ids=ids)
        assert L._lib.lib.skv_launch_count() - before == 2
        assert torch.equal(qa, qb) and parity_errors(out_b, to_np(out_a))[0] <= TOL_BF16
        assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0))
    assert list(pool_b.lengths(0)) == [lens[s] + (5 if s in ids else 0) for s in range(n)]
    ka, va = pool_a.gather(0, n_seqs=n)
    kb, vb = pool_b.gather(0, n_seqs=n)
    for s in range(n):
        t = lens[s] + (5 if s in ids else 0)
        assert torch.equal(ka[s, :, :t], kb[s, :, :t]) and torch.equal(va[s, :, :t], vb[s, :, :t])
    with pytest.raises(ValueError, match="listed twice"):
        pool_b.decode_step(0, qb[:2].contiguous(), k[:2].contiguous(), v[:2].contiguous(), seq_ids=[1, 1])
    assert pool_b.check_device_status() == 0


def test_paged_tensor_core_prefill_at_2048_tokens_matches_the_oracle_on_sampled_blocks():
    """The prefill shape of the DeepSeek-1.3B-shaped decoder (16 MHA heads of 128, 2048-token prompt, bf16, 16-token
    pages dealt out in a random order): the paged tcgen05 kernel against the oracle on 128-row blocks sampled over
    sequences, heads and positions (the first block, one across the middle, the last), after a RoPE-on-write append."""
    rng = np.random.default_rng(2048)
    n, H, S, D, P = 2, 16, 2048, 128, 16
    pps = S // P
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=H, head_dim=D, num_pages=n * pps + 5, max_seqs=n,
                                       max_pages_per_seq=pps, page_size=P, dtype=torch.bfloat16, rope_theta=100000.0,
                                       rope_scaling_factor=4.0))
    perm = rng.permutation(n * pps + 5)
    for s in range(n):
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, perm[s * pps:(s + 1) * pps].tolist(), 0)
    g = torch.Generator(device=DEV).manual_seed(7)
    q = torch.randn((n, H, S, D), generator=g, device=DEV).to(torch.bfloat16)
    k = torch.randn((n, H, S, D), generator=g, device=DEV).to(torch.bfloat16)
    v = torch.randn((n, H, S, D), generator=g, device=DEV).to(torch.bfloat16)
    k0, q0 = to_np(k), to_np(q)
    pool.append(0, k, v, start_pos=[0, 0], rope_k=True, q=q)              # rotates q in place, K on the way into the pages
    out = pool.prefill_attention(0, q)
    assert pool.check_device_status() == 0
    kd, vd = pool.gather(0, n_seqs=n)
    pos = np.arange(S)
    for s, h, r0 in [(0, 0, 0), (1, 7, 960), (0, 15, S - 128), (1, 3, 1500)]:
        k_rot = bf16_round(opaged.rope_rows(k0[s].transpose(1, 0, 2), pos, 100000.0, 4.0)).transpose(1, 0, 2)
        assert np.all(np.abs(to_np(kd[s, h]) - k_rot[h]) <= np.abs(k_rot[h]) * 2.0 ** -7 + 1e-30), "stored K against the oracle's RoPE"
        ref = oattn.chunked_grouped_attention(to_np(q[s:s + 1, h:h + 1, r0:r0 + 128]), to_np(kd[s:s + 1, h:h + 1]), to_np(vd[s:s + 1, h:h + 1]),
                                              query_positions=pos[r0:r0 + 128].astype(np.int32), q_block_size=512, k_block_size=512)
        assert_parity(out[s:s + 1, h:h + 1, r0:r0 + 128], ref, TOL_BF16, f"paged prefill S=2048, sequence {s} head {h} rows {r0}")
