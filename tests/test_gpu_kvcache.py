"""Paged KV cache on the GPU, through the C ABI: the reference's cache tests
(tests/test_mlx_kvcache.py:28-93) and bit-exact comparison of copied KV bytes, page tables and
lengths with the oracle."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import lokahi_b200 as L
from oracle import paged as opaged
from oracle import rope as orope
from oracle.kvcache import ConcatKVCache
from parity import TOL_BF16, TOL_F32, assert_parity, bf16_round, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CONFIG = SimpleNamespace(num_hidden_layers=2, max_position_embeddings=64)


def _states(start, length):
    values = np.arange(start, start + length * 8, dtype=np.float32).reshape(1, 2, length, 4)
    return values, values + 100


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def test_update_appends_values_and_tracks_each_layer_length():
    cache = L.PagedKVCache(CONFIG, cache_dir=None, page_size=2)
    ref = ConcatKVCache(CONFIG, cache_dir=None)
    k0, v0 = _states(0, 3)
    k1, v1 = _states(24, 1)
    cache.update(_t(k0), _t(v0), 0, {"cache_position": torch.arange(0, 3)})
    ref.update(k0, v0, 0, {"cache_position": np.arange(0, 3)})
    keys, values = cache.update(_t(k1), _t(v1), 0, {"cache_position": torch.tensor([3])})
    rk, rv = ref.update(k1, v1, 0, {"cache_position": np.array([3])})
    assert cache.get_seq_length(0) == 4 and cache.get_seq_length(1) == 0 and cache.get_seq_length(None) == 4
    assert keys.shape == (1, 2, 4, 4)
    assert np.array_equal(to_np(keys.materialize()), rk) and np.array_equal(to_np(values.materialize()), rv)
    assert np.array_equal(to_np(keys[:, :, :3]), k0) and np.array_equal(to_np(values[:, :, 3:]), v1)
    assert len(cache) == 1 and 0 in cache and 1 not in cache and cache[1] == {"key": None, "value": None}
    assert cache.pool.page_table(cache.seq_ids[0]).tolist() == [0, 1]
    assert cache.pool.check_device_status() == 0


def test_update_rejects_replay_and_bad_shapes():
    cache = L.PagedKVCache(CONFIG, cache_dir=None)
    k, v = (_t(x) for x in _states(0, 2))
    cache.update(k, v, 0, {"cache_position": torch.tensor([0, 1])})
    with pytest.raises(ValueError, match="append exactly"):
        cache.update(k, v, 0, {"cache_position": torch.tensor([0, 1])})
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
    assert cache.get_seq_length(0) == 2


def test_disk_round_trip_preserves_values_and_length(tmp_path):
    for dtype in (torch.float32, torch.bfloat16):
        cache = L.PagedKVCache(CONFIG, cache_dir=str(tmp_path))
        k, v = _states(0, 2)
        cache.update(_t(k, dtype), _t(v, dtype), 1, {"cache_position": torch.tensor([0, 1])})
        cache.save_to_disk(1)
        path = tmp_path / "kvcache_layer_1.npz"
        assert cache.get_seq_length(1) == 2 and 1 not in cache._resident and path.exists() and 1 in cache
        restored = cache[1]
        assert np.array_equal(to_np(restored["key"]), k) and np.array_equal(to_np(restored["value"]), v)
        assert cache.get_seq_length(1) == 2
        # appending after a reload continues the same history
        k2, v2 = _states(16, 1)
        keys, _ = cache.update(_t(k2, dtype), _t(v2, dtype), 1, {"cache_position": torch.tensor([2])})
        assert np.array_equal(to_np(keys.materialize()), np.concatenate([k, k2], axis=2))
        cache.clear()
        assert not path.exists() and cache.get_seq_length(None) == 0


def test_memory_only_cache_requires_explicit_destination():
    cache = L.PagedKVCache(CONFIG, cache_dir=None)
    k, v = (_t(x) for x in _states(0, 1))
    cache.update(k, v, 0)
    with pytest.raises(ValueError, match="filename is required"):
        cache.save_to_disk(0)


def test_layer_window_cache_spills_lowest_layers(tmp_path):
    cfg = SimpleNamespace(num_hidden_layers=6, max_position_embeddings=32)
    cache = L.PagedLlamaDiskCache(cfg, cache_dir=str(tmp_path), max_layers_in_memory=2)
    k, v = (_t(x) for x in _states(0, 1))
    for layer in range(4):
        cache.update(k, v, layer)
    assert sorted(cache._resident) == [2, 3] and sorted(cache._disk_offloaded) == [0, 1] and len(cache) == 4
    assert np.array_equal(to_np(cache[0]["key"]), to_np(k))
    with pytest.raises(ValueError, match="must be positive"):
        L.PagedLlamaDiskCache(cfg, cache_dir=str(tmp_path), max_layers_in_memory=0)
    assert isinstance(L.create_paged_kv_cache("llama3-1B", cfg, str(tmp_path)), L.PagedLlamaDiskCache)
    qwen = L.create_paged_kv_cache("qwen3-next-80B", SimpleNamespace(max_position_embeddings=32, num_hidden_layers=None), str(tmp_path))
    assert isinstance(qwen, L.PagedQwen3NextDiskCache) and qwen.num_layers == 80
    assert type(L.create_paged_kv_cache("gemma3-12B", cfg, str(tmp_path))) is L.PagedKVCache
    # the window also applies when the tokens arrive through the RoPE-on-write path
    cache2 = L.PagedLlamaDiskCache(cfg, cache_dir=str(tmp_path / "w2"), max_layers_in_memory=2)
    D = 64
    kk = torch.randn((1, 2, 3, D), device=DEV)
    qq = torch.randn((1, 4, 3, D), device=DEV)
    for layer in range(4):
        cache2.update_with_rope(qq.clone(), kk, kk, layer, {"cache_position": [0, 1, 2]}, inv_freq=L.rope_inv_freq(D, 10000.0))
    assert sorted(cache2._resident) == [2, 3] and sorted(cache2._disk_offloaded) == [0, 1]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_ragged_append_with_rope_matches_oracle(dtype, tol):
    """Ragged sequences, external random page table, RoPE-on-write for K and Q in one launch."""
    rng = np.random.default_rng(21)
    n_seqs, Hkv, Hq, D, P = 5, 2, 4, 64, 16
    theta = 500000.0
    lens = [0, 1, 15, 16, 37]
    n_pages = 32
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=n_pages, max_seqs=n_seqs,
                                       max_pages_per_seq=6, page_size=P, dtype=dtype, rope_theta=theta))
    perm = rng.permutation(n_pages)
    tables = []
    for s in range(n_seqs):
        assert pool.alloc_sequence() == s
        pages = perm[s * 6:(s + 1) * 6].tolist()
        pool.set_page_table(s, pages, 0)
        tables.append(pages)
    k_ref = np.zeros((n_pages, Hkv, P, D), np.float32)
    v_ref = np.zeros_like(k_ref)
    rnd = (lambda a: a) if dtype == torch.float32 else bf16_round
    # first a prefill of different lengths per sequence (one call per sequence), then a joint decode append
    for s, n in enumerate(lens):
        if n == 0:
            continue
        k = rnd(rng.standard_normal((1, Hkv, n, D), dtype=np.float32))
        v = rnd(rng.standard_normal((1, Hkv, n, D), dtype=np.float32))
        pool.append(0, _t(k, dtype), _t(v, dtype), seq_ids=[s], start_pos=[0], rope_k=True)
        kr = rnd(orope.apply(k, *orope.cos_sin(np.arange(n)[None], D, theta)))
        opaged.write_tokens(k_ref, np.array(tables[s]), 0, kr[0])
        opaged.write_tokens(v_ref, np.array(tables[s]), 0, v[0])
    k = rnd(rng.standard_normal((n_seqs, Hkv, D), dtype=np.float32))
    v = rnd(rng.standard_normal((n_seqs, Hkv, D), dtype=np.float32))
    q = rnd(rng.standard_normal((n_seqs, Hq, D), dtype=np.float32))
    qt = _t(q, dtype)
    pool.append(0, _t(k, dtype), _t(v, dtype), start_pos=lens, rope_k=True, q=qt, layout="bhd")
    kr = rnd(opaged.rope_rows(k, np.array(lens), theta))
    qr = rnd(opaged.rope_rows(q, np.array(lens), theta))
    for s in range(n_seqs):
        opaged.write_tokens(k_ref, np.array(tables[s]), lens[s], kr[s][:, None, :])
        opaged.write_tokens(v_ref, np.array(tables[s]), lens[s], v[s][:, None, :])
    kp, vp = pool.layer_views(0)
    assert pool.check_device_status() == 0
    assert np.array_equal(pool.lengths(0), np.array(lens) + 1)
    assert np.array_equal(to_np(vp), v_ref), "copied V bytes must be bit-exact"
    assert_parity(kp, k_ref, tol, "rotated K in pages")
    assert_parity(qt, qr, tol, "rotated Q")
    # device copy of the lengths matches the host's
    gk, gv = pool.gather(0, n_seqs=n_seqs)
    for s in range(n_seqs):
        T = lens[s] + 1
        assert np.array_equal(to_np(gv[s, :, :T]), opaged.logical_kv(v_ref, np.array(tables[s]), T))
        assert not to_np(gv[s, :, T:]).any()


def test_rope_rows_matches_reference_fixture(golden_dir):
    with np.load(os.path.join(golden_dir, "rope_half_rotation.npz")) as d:
        q = _t(d["q"][0].transpose(1, 0, 2))            # [rows=3, heads=2, dim=4]
        inv = torch.from_numpy(L.rope_inv_freq(int(d["dim"]), float(d["base"])))
        out = L.rope_rows(q, torch.from_numpy(d["positions"][0]), inv)
        assert np.allclose(to_np(out).transpose(1, 0, 2)[None], d["q_out"], atol=1e-6)


def test_rope_linear_scaling_and_large_positions():
    rng = np.random.default_rng(5)
    x = rng.standard_normal((7, 3, 128), dtype=np.float32)
    pos = np.array([0, 1, 4095, 8192, 65537, 98303, 131071])
    inv = L.rope_inv_freq(128, 100000.0)
    out = L.rope_rows(_t(x), torch.from_numpy(pos), torch.from_numpy(inv), scaling_factor=4.0)
    ref = opaged.rope_rows(x, pos, 100000.0, 4.0)
    assert_parity(out, ref, TOL_F32, "scaled RoPE")


def test_evict_prefetch_round_trip_is_bit_exact_and_moves_pages():
    rng = np.random.default_rng(8)
    Hkv, D, P, T = 2, 32, 4, 26
    pool = L.PagedPool(L.PagedKVConfig(num_layers=3, num_kv_heads=Hkv, head_dim=D, num_pages=12, max_seqs=2,
                                       max_pages_per_seq=8, page_size=P, dtype=torch.bfloat16, host_pages=8))
    model = opaged.PagePoolModel(3, 12, P, 2, 8, 8)
    s = pool.alloc_sequence(); model.alloc_sequence()
    ks, vs = [], []
    for layer in range(3):
        k = bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32))
        v = bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32))
        pool.append(layer, _t(k, torch.bfloat16), _t(v, torch.bfloat16), seq_ids=[s], start_pos=[0])
        model.append(layer, s, 0, T)
        ks.append(k); vs.append(v)
    pool.evict(s, 0, 4); model.evict(s, 0, 4)
    assert np.array_equal(pool.page_table(s), model.page_table[s, :7]) and (pool.page_table(s)[:4] <= -2).all()
    with pytest.raises(L.NotResidentError):
        pool.gather(0, seq_ids=[s])
    q = _t(bf16_round(rng.standard_normal((1, 4, D), dtype=np.float32)), torch.bfloat16)
    with pytest.raises(L.NotResidentError):
        pool.decode_attention(0, q, seq_ids=[s])
    # another sequence takes the freed device pages, so the prefetch must land elsewhere
    s2 = pool.alloc_sequence(); model.alloc_sequence()
    filler = _t(np.ones((1, Hkv, 3 * P, D), np.float32), torch.bfloat16)
    pool.append(0, filler, filler, seq_ids=[s2], start_pos=[0]); model.append(0, s2, 0, 3 * P)
    pool.prefetch(s, 0, 7); model.prefetch(s, 0, 7)
    pool.wait_resident(5000)
    assert np.array_equal(pool.page_table(s), model.page_table[s, :7])
    for layer in range(3):
        gk, gv = pool.gather(layer, seq_ids=[s])
        assert np.array_equal(to_np(gk), ks[layer]) and np.array_equal(to_np(gv), vs[layer])
    c = pool.counters()
    assert c["pages_evicted"] == 4 and c["pages_prefetched"] == 4 and c["bytes_d2h"] == c["bytes_h2d"] == 4 * 3 * 2 * Hkv * P * D * 2
    assert pool.check_device_status() == 0


def test_long_context_decode_with_eviction_every_step():
    """The long-context configuration at reduced scale: 4 sequences, one KV head with its 4 query heads per
    GPU, several layers, bf16; every step appends one token with RoPE, parks the oldest quarter of each
    sequence's pages in pinned host memory, brings them back (they land in other device pages), and attends.
    Outputs must match the oracle every step and the page tables must match the allocator model."""
    rng = np.random.default_rng(96)
    n_seqs, Hq, Hkv, D, P, layers, T0, steps = 4, 4, 1, 128, 16, 3, 1500, 6
    theta = 500000.0
    pages_per_seq = -(-(T0 + steps) // P)
    n_pages = n_seqs * pages_per_seq + 8
    host_pages = n_seqs * (pages_per_seq // 4 + 1)
    pool = L.PagedPool(L.PagedKVConfig(num_layers=layers, num_kv_heads=Hkv, head_dim=D, num_pages=n_pages, max_seqs=n_seqs,
                                       max_pages_per_seq=pages_per_seq, page_size=P, dtype=torch.bfloat16,
                                       host_pages=host_pages, rope_theta=theta))
    model = opaged.PagePoolModel(layers, n_pages, P, n_seqs, pages_per_seq, host_pages)
    for s in range(n_seqs):
        assert pool.alloc_sequence() == model.alloc_sequence() == s
    # logical history per (layer, sequence) kept on the host for the oracle
    hist_k = np.zeros((layers, n_seqs, Hkv, T0 + steps, D), np.float32)
    hist_v = np.zeros_like(hist_k)
    for layer in range(layers):
        k = bf16_round(rng.standard_normal((n_seqs, Hkv, T0, D), dtype=np.float32))
        v = bf16_round(rng.standard_normal((n_seqs, Hkv, T0, D), dtype=np.float32))
        pool.append(layer, _t(k, torch.bfloat16), _t(v, torch.bfloat16), start_pos=[0] * n_seqs)   # history stored as given
        for s in range(n_seqs):
            model.append(layer, s, 0, T0)
        hist_k[layer, :, :, :T0] = k
        hist_v[layer, :, :, :T0] = v
    for step in range(steps):
        T = T0 + step
        n_old = (T // P) // 4
        for s in range(n_seqs):
            pool.evict(s, 0, n_old); model.evict(s, 0, n_old)
        for s in range(n_seqs):
            pool.prefetch(s, 0, n_old); model.prefetch(s, 0, n_old)
        for s in range(n_seqs):
            assert np.array_equal(pool.page_table(s), model.page_table[s, :model.num_seq_pages[s]])
        for layer in range(layers):
            q = bf16_round(rng.standard_normal((n_seqs, Hq, D), dtype=np.float32))
            k = bf16_round(rng.standard_normal((n_seqs, Hkv, D), dtype=np.float32))
            v = bf16_round(rng.standard_normal((n_seqs, Hkv, D), dtype=np.float32))
            qt = _t(q, torch.bfloat16)
            pool.append(layer, _t(k, torch.bfloat16), _t(v, torch.bfloat16), start_pos=[T] * n_seqs, rope_k=True, q=qt,
                        layout="bhd")
            for s in range(n_seqs):
                model.append(layer, s, T, 1)
            out = pool.decode_attention(layer, qt)
            kr = bf16_round(opaged.rope_rows(k, np.full(n_seqs, T), theta))
            qr = bf16_round(opaged.rope_rows(q, np.full(n_seqs, T), theta))
            hist_k[layer, :, :, T] = kr
            hist_v[layer, :, :, T] = v
            ref = np.stack([
                oattn_decode(qr[s], hist_k[layer, s, :, :T + 1], hist_v[layer, s, :, :T + 1], T) for s in range(n_seqs)])
            assert_parity(out, ref, TOL_BF16, f"step {step} layer {layer}")
    c = pool.counters()
    assert c["pages_evicted"] == c["pages_prefetched"] == sum(((T0 + st) // P) // 4 for st in range(steps)) * n_seqs
    assert pool.check_device_status() == 0


def test_long_context_at_full_length_96k_tokens_with_a_quarter_parked():
    """One sequence of the long-context configuration at its full length (98304 tokens, one KV head with its 4
    query heads, bf16, theta 5e5): three one-call decode steps at positions 98304..98306, with the oldest quarter
    of the pages parked in host memory and brought back before every step, against the oracle on the logical
    history (64 split-K chunks, 6144 pages in a random order, RoPE angles near 1e5 radians)."""
    rng = np.random.default_rng(965)
    Hq, Hkv, D, P, T0, steps, theta = 4, 1, 128, 16, 98304, 3, 500000.0
    pages = T0 // P + 2
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=pages + 8, max_seqs=1,
                                       max_pages_per_seq=pages, page_size=P, dtype=torch.bfloat16,
                                       host_pages=pages // 4 + 2, rope_theta=theta))
    assert pool.alloc_sequence() == 0
    order = rng.permutation(pages + 8)[:pages].tolist()
    pool.set_page_table(0, order, T0)
    k_pages = bf16_round(rng.standard_normal((pages + 8, Hkv, P, D), dtype=np.float32))
    v_pages = bf16_round(rng.standard_normal((pages + 8, Hkv, P, D), dtype=np.float32))
    kp, vp = pool.layer_views(0)
    kp.copy_(_t(k_pages, torch.bfloat16)); vp.copy_(_t(v_pages, torch.bfloat16))
    table = np.array(order, np.int32)
    hist_k = np.zeros((Hkv, T0 + steps, D), np.float32)
    hist_v = np.zeros_like(hist_k)
    hist_k[:, :T0] = opaged.logical_kv(k_pages, table, T0)
    hist_v[:, :T0] = opaged.logical_kv(v_pages, table, T0)
    for step in range(steps):
        T = T0 + step
        n_old = (T // P) // 4
        pool.evict(0, 0, n_old)
        pool.prefetch(0, 0, n_old)
        q = bf16_round(rng.standard_normal((1, Hq, D), dtype=np.float32))
        k = bf16_round(rng.standard_normal((1, Hkv, D), dtype=np.float32))
        v = bf16_round(rng.standard_normal((1, Hkv, D), dtype=np.float32))
        qt = _t(q, torch.bfloat16)
        out = pool.decode_step(0, qt, _t(k, torch.bfloat16), _t(v, torch.bfloat16))
        qr = bf16_round(opaged.rope_rows(q, np.array([T]), theta))
        hist_k[:, T] = bf16_round(opaged.rope_rows(k, np.array([T]), theta))[0]
        hist_v[:, T] = v[0]
        # rotated q may sit one bf16 step from the NumPy rotation (sincosf against numpy at 1e5 radians)
        assert np.max(np.abs(to_np(qt) - qr)) <= 2.0 ** -7 * np.max(np.abs(qr)), f"rotated q, step {step}"
        ref = oattn_decode(to_np(qt)[0], hist_k[:, :T + 1], hist_v[:, :T + 1], T)
        assert_parity(out[0], ref, TOL_BF16, f"96k-token decode step {step}")
    kg, vg = pool.gather(0, n_seqs=1)
    assert np.array_equal(to_np(vg)[0, :, :T0 + steps], hist_v), "stored V after parking and three appended rows"
    assert np.max(np.abs(to_np(kg)[0, :, T0:T0 + steps] - hist_k[:, T0:])) <= 2.0 ** -7 * np.max(np.abs(hist_k[:, T0:]))
    assert np.array_equal(to_np(kg)[0, :, :T0], hist_k[:, :T0])
    c = pool.counters()
    assert c["pages_evicted"] == c["pages_prefetched"] == steps * ((T0 // P) // 4)
    assert pool.check_device_status() == 0


def oattn_decode(q, k_hist, v_hist, pos):
    from oracle import attention as oattn
    return oattn.chunked_grouped_attention(q[None, :, None, :], k_hist[None], v_hist[None],
                                           query_positions=np.array([[pos]], dtype=np.int32), causal=True,
                                           q_block_size=32768, k_block_size=1000000, out_dtype=np.float32)[0, :, 0, :]


def test_residency_manager_keeps_results_exact_under_lru_churn():
    """Three sequences, device budget for two: attending them round-robin forces a park/fetch on every turn;
    every output must still equal the all-resident result bit for bit."""
    rng = np.random.default_rng(17)
    n, Hq, Hkv, D, P, T = 3, 8, 2, 128, 16, 320
    pool = L.PagedPool(L.PagedKVConfig(num_layers=2, num_kv_heads=Hkv, head_dim=D, num_pages=64, max_seqs=n,
                                       max_pages_per_seq=24, page_size=P, dtype=torch.bfloat16, host_pages=64))
    qs = []
    for s in range(n):
        assert pool.alloc_sequence() == s
        for layer in range(2):
            k = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
            v = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
            pool.append(layer, k, v, seq_ids=[s], start_pos=[0])
        qs.append(_t(bf16_round(rng.standard_normal((1, Hq, D), dtype=np.float32)), torch.bfloat16))
    expect = [[pool.decode_attention(layer, qs[s], seq_ids=[s]).clone() for layer in range(2)] for s in range(n)]
    res = L.KVPageResidency(pool, budget_pages=2 * (T // P), group_pages=8)
    for s in range(n):
        res.track(s)
    assert res.snapshot().parked_pages == T // P
    for turn in range(7):
        s = turn % n
        res.ensure_resident(s, 0, T // P)
        res.pin(s, 0, T // P)
        for layer in range(2):
            assert torch.equal(pool.decode_attention(layer, qs[s], seq_ids=[s]), expect[s][layer])
        res.release(s, 0, T // P)
    snap = res.snapshot()
    assert snap.resident_pages <= snap.budget_pages and snap.stalls >= 6 and snap.pinned_pages == 0
    assert pool.check_device_status() == 0


@pytest.mark.gpu
def test_look_ahead_prefetcher_keeps_results_exact_and_counts_its_hits():
    """Same churn as above, driven through the prefetcher: while a sequence is attended (pinned) the next one is
    reserved and copied back on the copy stream; every output equals the all-resident result bit for bit and the
    counters tell demand loads from look-ahead hits."""
    rng = np.random.default_rng(23)
    n, Hq, Hkv, D, P, T = 3, 8, 2, 128, 16, 320
    pool = L.PagedPool(L.PagedKVConfig(num_layers=2, num_kv_heads=Hkv, head_dim=D, num_pages=64, max_seqs=n,
                                       max_pages_per_seq=24, page_size=P, dtype=torch.bfloat16, host_pages=64))
    qs = []
    for s in range(n):
        assert pool.alloc_sequence() == s
        for layer in range(2):
            k = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
            v = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
            pool.append(layer, k, v, seq_ids=[s], start_pos=[0])
        qs.append(_t(bf16_round(rng.standard_normal((1, Hq, D), dtype=np.float32)), torch.bfloat16))
    expect = [[pool.decode_attention(layer, qs[s], seq_ids=[s]).clone() for layer in range(2)] for s in range(n)]
    groups = -(-(T // P) // 10)                                  # 20 pages in groups of 10
    res = L.KVPageResidency(pool, budget_pages=2 * (T // P), group_pages=10)
    for s in range(n):
        res.track(s)
    pf = L.KVPagePrefetcher(res)
    statuses = []
    for turn in range(9):
        s, nxt = turn % n, (turn + 1) % n
        leases = [pf.acquire(s, g) for g in range(groups)]
        statuses += [l.cache_status for l in leases]
        for g in range(groups):                                  # look ahead while this sequence is in use
            pf.prefetch(nxt, g)
        for layer in range(2):
            assert torch.equal(pool.decode_attention(layer, qs[s], seq_ids=[s]), expect[s][layer])
        for l in leases:
            l.release()
    snap = pf.snapshot()
    assert snap.prefetch_ready_hits + snap.prefetch_waits >= 8 and snap.pages_loaded >= 8 * 10
    assert "cold_miss" not in statuses[2 * groups:]              # after the first turns the look-ahead covers every group
    assert res.snapshot().resident_pages <= res.snapshot().budget_pages and res.snapshot().pinned_pages == 0
    assert pool.check_device_status() == 0


@pytest.mark.gpu
def test_one_call_decode_step_of_the_cache_equals_update_then_attention():
    """``decode_step_with_rope`` (one library call, two launches) against ``update_with_rope`` + the attention
    callable on twin caches over several steps: same rotated q, same stored history, same lengths, outputs within
    bf16 tolerance; a replayed position is still rejected with the reference's message."""
    rng = np.random.default_rng(31)
    B, Hq, Hkv, D, T0 = 3, 8, 2, 128, 37
    cfg = SimpleNamespace(num_hidden_layers=2, max_position_embeddings=256)
    inv = L.rope_inv_freq(D, 10000.0)
    caches = [L.PagedKVCache(cfg), L.PagedKVCache(cfg)]
    k0 = _t(bf16_round(rng.standard_normal((B, Hkv, T0, D), dtype=np.float32)), torch.bfloat16)
    v0 = _t(bf16_round(rng.standard_normal((B, Hkv, T0, D), dtype=np.float32)), torch.bfloat16)
    q0 = _t(bf16_round(rng.standard_normal((B, Hq, T0, D), dtype=np.float32)), torch.bfloat16)
    for c in caches:
        for layer in range(2):
            c.update_with_rope(q0.clone(), k0, v0, layer, {"cache_position": list(range(T0))}, inv_freq=inv)
    from parity import parity_errors
    for step in range(5):
        pos = T0 + step
        q = _t(bf16_round(rng.standard_normal((B, Hq, 1, D), dtype=np.float32)), torch.bfloat16)
        k = _t(bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32)), torch.bfloat16)
        v = _t(bf16_round(rng.standard_normal((B, Hkv, 1, D), dtype=np.float32)), torch.bfloat16)
        for layer in range(2):
            qa, qb = q.clone(), q.clone()
            kh, vh = caches[0].update_with_rope(qa, k, v, layer, {"cache_position": [pos]}, inv_freq=inv)
            out_a = L.chunked_grouped_attention(qa, kh, vh, query_positions=np.array([[pos]], dtype=np.int32), causal=True)
            out_b = caches[1].decode_step_with_rope(qb, k, v, layer, {"cache_position": [pos]}, inv_freq=inv)
            assert out_b is not None and out_b.shape == (B, Hq, 1, D)
            assert torch.equal(qa, qb)
            assert parity_errors(out_b, to_np(out_a))[0] <= TOL_BF16
            assert caches[0].get_seq_length(layer) == caches[1].get_seq_length(layer) == pos + 1
    for layer in range(2):
        ka, va = caches[0].materialize(layer)
        kb, vb = caches[1].materialize(layer)
        assert torch.equal(ka, kb) and torch.equal(va, vb)
    with pytest.raises(ValueError, match="append exactly"):
        caches[1].decode_step_with_rope(q.clone(), k, v, 0, {"cache_position": [T0]}, inv_freq=inv)
    assert caches[1].decode_step_with_rope(q0.clone(), k0, v0, 0, {"cache_position": [0]}, inv_freq=inv) is None   # L > 1


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,D", [(torch.bfloat16, 128), (torch.float32, 64)])
def test_vectorised_append_writes_the_same_bytes_as_the_scalar_kernel(skv_switch, dtype, D):
    """The 16-byte-access append (one block per token, cos/sin shared by all heads) against the element-wise
    kernel: stored K/V, rotated q and lengths bit-identical, with ragged starts and several tokens per call."""
    rng = np.random.default_rng(77)
    B, Hq, Hkv, P, n_new = 3, 8, 2, 16, 21
    starts = [0, 5, 30]
    inv = L.rope_inv_freq(D, 500000.0)
    results = []
    for scalar in ("1", "0"):
        skv_switch("SKV_APPEND_SCALAR", scalar)
        pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=32, max_seqs=B,
                                           max_pages_per_seq=8, page_size=P, dtype=dtype))
        pool.set_rope(inv, 2.0)
        r = np.random.default_rng(78)
        rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a)
        for s in range(B):
            assert pool.alloc_sequence() == s
            if starts[s]:
                k0 = _t(rnd(r.standard_normal((1, Hkv, starts[s], D), dtype=np.float32)), dtype)
                pool.append(0, k0, k0, seq_ids=[s], start_pos=[0])
        q = _t(rnd(r.standard_normal((B, Hq, n_new, D), dtype=np.float32)), dtype)
        k = _t(rnd(r.standard_normal((B, Hkv, n_new, D), dtype=np.float32)), dtype)
        v = _t(rnd(r.standard_normal((B, Hkv, n_new, D), dtype=np.float32)), dtype)
        pool.append(0, k, v, start_pos=starts, rope_k=True, q=q)
        kk, vv = pool.gather(0, n_seqs=B, max_len=max(starts) + n_new)
        torch.cuda.synchronize()
        results.append((q.clone(), kk.clone(), vv.clone(), pool.lengths(0).copy()))
        assert pool.check_device_status() == 0
    (qa, ka, va, la), (qb, kb, vb, lb) = results
    assert torch.equal(qa, qb) and np.array_equal(la, lb)
    for s in range(B):
        t = starts[s] + n_new
        assert torch.equal(ka[s, :, :t], kb[s, :, :t]) and torch.equal(va[s, :, :t], vb[s, :, :t])


@pytest.mark.gpu
def test_interleaved_parking_and_fetching_without_synchronisation_stays_bit_exact():
    """Evictions and prefetches of different sequences interleaved without any synchronisation in between, so that
    many copies are queued behind the compute stream and freed device pages and host slots are reused at once
    (more than a staging ring's worth of per-call metadata in flight): after the churn every sequence's K/V
    equals what was written."""
    rng = np.random.default_rng(41)
    n, Hkv, D, P, T = 6, 2, 128, 16, 256            # 16 pages per sequence
    pool = L.PagedPool(L.PagedKVConfig(num_layers=3, num_kv_heads=Hkv, head_dim=D, num_pages=n * 16 + 4, max_seqs=n,
                                       max_pages_per_seq=16, page_size=P, dtype=torch.bfloat16, host_pages=3 * 16))
    truth = []
    for s in range(n):
        assert pool.alloc_sequence() == s
        per_layer = []
        for layer in range(3):
            k = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
            v = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
            pool.append(layer, k, v, seq_ids=[s], start_pos=[0])
            per_layer.append((k.clone(), v.clone()))
        truth.append(per_layer)
    parked = []
    order = rng.permutation(n).tolist()
    for rnd_ in range(12):                           # at most three sequences' worth of host slots
        s = order[rnd_ % n]
        if s in parked:
            pool.prefetch(s, 0, 16)
            parked.remove(s)
        else:
            if len(parked) == 3:
                back = parked.pop(0)
                pool.prefetch(back, 0, 16)           # frees host slots that the eviction below takes straight away
            pool.evict(s, 0, 16)
            parked.append(s)
    for s in list(parked):
        pool.prefetch(s, 0, 16)
    pool.sync_transfers()
    for s in range(n):
        assert (pool.page_table(s) >= 0).all()
        for layer in range(3):
            k, v = pool.gather(layer, seq_ids=[s], max_len=T)
            assert torch.equal(k, truth[s][layer][0]) and torch.equal(v, truth[s][layer][1]), (s, layer)
    c = pool.counters()
    assert c["pages_evicted"] == c["pages_prefetched"] and c["free_host_slots"] == 3 * 16 and pool.check_device_status() == 0


@pytest.mark.gpu
def test_park_after_fetch_without_compute_in_between_leaves_the_device_table_parked():
    """prefetch then evict of the same pages with no compute call between them: the page-table entries that the
    prefetch deferred must not overwrite the eviction's; attention afterwards is refused (not resident) and, once
    fetched again, bit-exact."""
    rng = np.random.default_rng(43)
    Hq, Hkv, D, P, T = 8, 2, 128, 16, 64
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=16, max_seqs=2,
                                       max_pages_per_seq=4, page_size=P, dtype=torch.bfloat16, host_pages=8))
    assert pool.alloc_sequence() == 0
    k = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
    v = _t(bf16_round(rng.standard_normal((1, Hkv, T, D), dtype=np.float32)), torch.bfloat16)
    pool.append(0, k, v, seq_ids=[0], start_pos=[0])
    q = _t(bf16_round(rng.standard_normal((1, Hq, D), dtype=np.float32)), torch.bfloat16)
    expect = pool.decode_attention(0, q, seq_ids=[0]).clone()
    pool.evict(0, 0, 4)
    pool.prefetch(0, 0, 4)
    pool.evict(0, 0, 4)                                  # deferred entries of the prefetch are still unpublished here
    with pytest.raises(L.NotResidentError):
        pool.decode_attention(0, q, seq_ids=[0])
    pool.sync_transfers()
    kp, vp = pool.layer_views(0)
    kp.zero_(); vp.zero_()                               # whatever the device table pointed at is now zeros
    pool.prefetch(0, 0, 4)
    assert torch.equal(pool.decode_attention(0, q, seq_ids=[0]), expect)
    assert pool.check_device_status() == 0


@pytest.mark.gpu
def test_layer_file_in_the_reference_layout_and_float32_loads_into_a_bfloat16_cache(tmp_path):
    """A layer file as the reference writes it (compressed .npz with float32 ``key`` / ``value`` and ``seen_tokens``,
    mlx_kvcache.py:183-222) replaces the file of an offloaded layer: the bfloat16 cache reads it back, rounded."""
    cfg = SimpleNamespace(num_hidden_layers=2, max_position_embeddings=64)
    cache = L.PagedKVCache(cfg, cache_dir=str(tmp_path))
    rng = np.random.default_rng(3)
    k = _t(bf16_round(rng.standard_normal((1, 2, 5, 128), dtype=np.float32)), torch.bfloat16)
    cache.update(k, k, 0, {"cache_position": list(range(5))})
    cache.save_to_disk(0)
    name = cache._disk_offloaded[0]
    k32 = rng.standard_normal((1, 2, 5, 128), dtype=np.float32)
    v32 = rng.standard_normal((1, 2, 5, 128), dtype=np.float32)
    np.savez_compressed(name, key=k32, value=v32, seen_tokens=5)
    got = cache[0]
    assert np.array_equal(to_np(got["key"]), bf16_round(k32)) and np.array_equal(to_np(got["value"]), bf16_round(v32))
    assert cache.get_seq_length(0) == 5 and 0 not in cache._disk_offloaded


@pytest.mark.gpu
def test_saved_bfloat16_layer_is_readable_with_the_reference_loader_logic(tmp_path):
    """What the reference's loader does with a layer file (np.load, ``data["key"]`` / ``data["value"]`` taken as they
    are, ``seen_tokens`` if present; mlx_kvcache.py:232-247): a bfloat16 layer saved here must give it the stored values
    (float32 holds them exactly), and the compact 16-bit form stays available behind its switch and round-trips."""
    cfg = SimpleNamespace(num_hidden_layers=1, max_position_embeddings=64)
    rng = np.random.default_rng(8)
    k_np = bf16_round(rng.standard_normal((2, 2, 7, 128), dtype=np.float32))
    v_np = bf16_round(rng.standard_normal((2, 2, 7, 128), dtype=np.float32))
    for compact in (False, True):
        cache = L.PagedKVCache(cfg, cache_dir=str(tmp_path / ("c" if compact else "f")))
        cache.compact_bf16_files = compact
        cache.update(_t(k_np, torch.bfloat16), _t(v_np, torch.bfloat16), 0, {"cache_position": list(range(7))})
        cache.save_to_disk(0)
        with np.load(cache._disk_offloaded[0]) as data:           # the reference's reading of the file
            key, value, seen = np.asarray(data["key"]), np.asarray(data["value"]), int(data["seen_tokens"])
            tagged = "stored_dtype" in data
        assert seen == 7 and tagged == compact
        if not compact:
            assert key.dtype == np.float32 and np.array_equal(key, k_np) and np.array_equal(value, v_np)
        else:
            assert key.dtype == np.uint16
        got = cache[0]                                           # and this loader reads both forms back bit for bit
        assert np.array_equal(to_np(got["key"]), k_np) and np.array_equal(to_np(got["value"]), v_np)
        cache.clear()


@pytest.mark.gpu
def test_attention_over_other_sequences_runs_beside_page_copies():
    """While the pages of one sequence travel to host memory and back, calls that touch only other sequences are not
    ordered behind the copies (they would find their pages resident anyway); a call on the travelling sequence, or
    one that takes fresh pages, is.  Results are the ones from before the copies either way."""
    rng = np.random.default_rng(21)
    Hq, Hkv, D, P = 8, 2, 128, 16
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=40, max_seqs=3, max_pages_per_seq=12,
                                       page_size=P, dtype=torch.bfloat16, host_pages=16, rope_theta=10000.0))
    lens = [150, 100, 40]
    for s, t in enumerate(lens):
        assert pool.alloc_sequence() == s
        kv = _t(bf16_round(rng.standard_normal((1, Hkv, t, D), dtype=np.float32)), torch.bfloat16)
        pool.append(0, kv, kv, seq_ids=[s], start_pos=[0])
    q = _t(bf16_round(rng.standard_normal((3, Hq, D), dtype=np.float32)), torch.bfloat16)
    before = pool.decode_attention(0, q).clone()
    pool.evict(0, 0, 8)
    pool.prefetch(0, 0, 8)                                     # sequence 0 is on its way out and back
    other = pool.decode_attention(0, q[1:].contiguous(), seq_ids=[1, 2])
    assert torch.equal(other, before[1:])
    k1 = _t(bf16_round(rng.standard_normal((1, Hkv, D), dtype=np.float32)), torch.bfloat16)
    step_out = pool.decode_step(0, q[2:3].clone(), k1, k1, seq_ids=[2])   # stays inside its last page: no fresh page
    assert pool.length(0, 2) == 41 and bool(torch.isfinite(step_out.float()).all())
    again = pool.decode_attention(0, q[:1].contiguous(), seq_ids=[0])     # the travelling sequence: ordered behind the copies
    assert torch.equal(again, before[:1])
    assert pool.check_device_status() == 0 and pool.counters()["pages_prefetched"] == 8
