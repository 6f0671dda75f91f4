"""Host bookkeeping of the C++ pool (device = -1: no GPU needed) against the Python model of the
allocator: page tables, lengths and counters must agree bit for bit after any operation sequence."""
import numpy as np
import pytest

import lokahi_b200 as L
from oracle.paged import OutOfPages, PagePoolModel


def make(num_layers=2, num_pages=24, page_size=4, max_seqs=4, max_pages_per_seq=8, host_pages=0):
    cfg = L.PagedKVConfig(num_layers=num_layers, num_kv_heads=2, head_dim=8, num_pages=num_pages, max_seqs=max_seqs,
                          max_pages_per_seq=max_pages_per_seq, page_size=page_size, device=-1, host_pages=host_pages)
    return L.PagedPool(cfg), PagePoolModel(num_layers, num_pages, page_size, max_seqs, max_pages_per_seq, host_pages)


def same_state(pool, model):
    for s in range(model.max_seqs):
        n = int(model.num_seq_pages[s])
        assert np.array_equal(pool.page_table(s), model.page_table[s, :n]), f"page table of sequence {s}"
    for layer in range(model.num_layers):
        assert np.array_equal(pool.lengths(layer), model.lengths[layer])
    c = pool.counters()
    assert c["free_pages"] == len(model.free_pages) and c["free_host_slots"] == len(model.free_host)
    assert c["live_sequences"] == int(model.live.sum())


def test_pops_yield_ascending_pages_and_sequences():
    pool, model = make()
    assert [pool.alloc_sequence() for _ in range(3)] == [model.alloc_sequence() for _ in range(3)] == [0, 1, 2]
    pool.append(0, None, None, n_new=9, seq_ids=[0, 1], start_pos=[0, 0])
    for s in (0, 1):
        model.append(0, s, 0, 9)
    assert pool.page_table(0).tolist() == [0, 1, 2] and pool.page_table(1).tolist() == [3, 4, 5]
    same_state(pool, model)


def test_replay_and_bad_arguments_are_rejected_without_side_effects():
    pool, model = make()
    s = pool.alloc_sequence(); model.alloc_sequence()
    pool.append(0, None, None, n_new=2, seq_ids=[s], start_pos=[0]); model.append(0, s, 0, 2)
    with pytest.raises(ValueError, match="append exactly"):
        pool.append(0, None, None, n_new=2, seq_ids=[s], start_pos=[0])
    with pytest.raises(ValueError, match="non-negative integer"):
        pool.append(-1, None, None, n_new=1, seq_ids=[s], start_pos=[2])
    with pytest.raises(ValueError, match="outside configured layer count"):
        pool.append(2, None, None, n_new=1, seq_ids=[s], start_pos=[2])
    with pytest.raises(ValueError, match="not live"):
        pool.append(0, None, None, n_new=1, seq_ids=[3], start_pos=[0])
    with pytest.raises(ValueError, match="listed twice"):
        pool.append(0, None, None, n_new=1, seq_ids=[s, s], start_pos=[2, 2])
    same_state(pool, model)
    # layers keep their own lengths (the reference tracks them per layer, mlx_kvcache.py:121-123)
    pool.append(1, None, None, n_new=3, seq_ids=[s], start_pos=[0]); model.append(1, s, 0, 3)
    assert pool.length(0, s) == 2 and pool.length(1, s) == 3
    same_state(pool, model)


def test_out_of_pages_is_all_or_nothing():
    pool, model = make(num_pages=5)
    for _ in range(2):
        pool.alloc_sequence(); model.alloc_sequence()
    pool.append(0, None, None, n_new=8, seq_ids=[0], start_pos=[0]); model.append(0, 0, 0, 8)
    with pytest.raises(L.OutOfPagesError):
        pool.append(0, None, None, n_new=16, seq_ids=[1], start_pos=[0])      # needs 4, 3 free
    with pytest.raises(L.OutOfPagesError):
        pool.append(0, None, None, n_new=4 * 9, seq_ids=[1], start_pos=[0])   # beyond the row
    same_state(pool, model)
    with pytest.raises(L.OutOfPagesError):
        for _ in range(5):
            pool.alloc_sequence()


def test_external_page_table_is_validated():
    pool, model = make()
    a = pool.alloc_sequence(); b = pool.alloc_sequence()
    pool.set_page_table(a, [7, 3, 11], 10)
    assert pool.page_table(a).tolist() == [7, 3, 11] and pool.length(1, a) == 10
    with pytest.raises(ValueError, match="belongs to sequence"):
        pool.set_page_table(b, [3], 1)
    with pytest.raises(ValueError, match="listed twice"):
        pool.set_page_table(b, [5, 5], 1)
    with pytest.raises(ValueError, match="outside the pool"):
        pool.set_page_table(b, [24], 1)
    with pytest.raises(ValueError, match="does not fit"):
        pool.set_page_table(b, [5], 5)
    # the allocator never hands out an adopted page
    pool.append(0, None, None, n_new=4 * 8, seq_ids=[b], start_pos=[0])
    assert not set(pool.page_table(b).tolist()) & {7, 3, 11}


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_random_operation_sequences_match_the_model(seed):
    rng = np.random.default_rng(seed)
    pool, model = make(num_pages=40, max_seqs=5, max_pages_per_seq=10, host_pages=12)
    live = []
    for _ in range(300):
        op = rng.integers(0, 6)
        if op == 0 and len(live) < 5:
            s = pool.alloc_sequence()
            assert s == model.alloc_sequence()
            live.append(s)
        elif op == 1 and live:
            s = live.pop(int(rng.integers(len(live))))
            pool.free_sequence(s); model.free_sequence(s)
        elif op in (2, 3) and live:
            s = int(rng.choice(live)); layer = int(rng.integers(2)); n = int(rng.integers(1, 9))
            start = int(model.lengths[layer, s])
            resident = all(e >= 0 for e in model.page_table[s, start // 4: model.num_seq_pages[s]])
            try:
                model.reserve  # noqa: B018
                if not resident:
                    with pytest.raises(L.NotResidentError):
                        pool.append(layer, None, None, n_new=n, seq_ids=[s], start_pos=[start])
                    continue
                model.append(layer, s, start, n)
            except OutOfPages:
                with pytest.raises(L.OutOfPagesError):
                    pool.append(layer, None, None, n_new=n, seq_ids=[s], start_pos=[start])
            else:
                pool.append(layer, None, None, n_new=n, seq_ids=[s], start_pos=[start])
        elif op == 4 and live:
            s = int(rng.choice(live)); n = int(model.num_seq_pages[s])
            if n:
                first = int(rng.integers(n)); cnt = int(rng.integers(1, n - first + 1))
                try:
                    model.evict(s, first, cnt)
                except OutOfPages:
                    with pytest.raises(L.OutOfPagesError):
                        pool.evict(s, first, cnt)
                else:
                    pool.evict(s, first, cnt)
        elif op == 5 and live:
            s = int(rng.choice(live)); n = int(model.num_seq_pages[s])
            if n:
                try:
                    model.prefetch(s, 0, n)
                except OutOfPages:
                    with pytest.raises(L.OutOfPagesError):
                        pool.prefetch(s, 0, n)
                else:
                    pool.prefetch(s, 0, n)
        same_state(pool, model)


def test_truncate_and_config_validation():
    pool, _ = make()
    s = pool.alloc_sequence()
    pool.append(0, None, None, n_new=6, seq_ids=[s], start_pos=[0])
    pool.truncate(0, 2, seq_ids=[s])
    assert pool.length(0, s) == 2 and len(pool.page_table(s)) == 2
    with pytest.raises(ValueError, match="exceeds"):
        pool.truncate(0, 3, seq_ids=[s])
    with pytest.raises(ValueError, match="positive integer"):
        L.PagedKVConfig(num_layers=0, num_kv_heads=1, head_dim=8, num_pages=1, max_seqs=1, max_pages_per_seq=1)
    with pytest.raises(ValueError, match="even"):
        L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=7, num_pages=1, max_seqs=1, max_pages_per_seq=1)


def test_misaligned_workspace_is_refused_before_anything_is_launched():
    """The merge kernel reads the workspace with 8- and 16-byte loads: a pointer that is not 16-byte aligned is an
    argument error from every entry point that takes one, not a device fault."""
    import ctypes as C
    from lokahi_b200 import _lib
    pool, _ = make()
    s = pool.alloc_sequence()
    pool.append(0, None, None, n_new=3, seq_ids=[s], start_pos=[0])
    before = _lib.lib.skv_launch_count()
    odd = 0x1004                          # never dereferenced: the call is refused first
    ids = _lib.i32_array([s])
    assert _lib.lib.skv_decode_attn(pool._h, 0, ids, 1, 0x2000, 0x3000, None, 2, 1e-12, odd, 1 << 20, None) == _lib.ERR_BAD_ARG
    assert b"16-byte aligned" in _lib.lib.skv_last_error(pool._h)
    assert _lib.lib.skv_decode_partial(pool._h, 0, ids, 1, 0x2000, None, 2, odd, 1 << 20, 0x3000, None) == _lib.ERR_BAD_ARG
    x = _lib.SkvExchange(mode=_lib.XCHG_HEAD_GATHER, rank=0, world=1, epoch=1)
    assert _lib.lib.skv_decode_attn_xchg(pool._h, 0, ids, 1, 0x2000, None, 2, 1e-12, odd, 1 << 20, C.byref(x), None) == _lib.ERR_BAD_ARG
    a = _lib.SkvStepArgs(layer=0, n_seqs=1, q=0x2000, k=0x2000, v=0x2000, out=0x3000, n_q_heads=2, eps=1e-12,
                         workspace=odd, workspace_bytes=1 << 20)
    a.seq_ids = ids
    assert _lib.lib.skv_decode_step_ex(pool._h, C.byref(a), None) == _lib.ERR_BAD_ARG
    assert b"16-byte aligned" in _lib.lib.skv_last_error(pool._h)
    assert _lib.lib.skv_launch_count() == before and pool.length(0, s) == 3


def test_pools_beyond_the_token_limit_per_sequence_are_refused_at_creation():
    """The split-K plan gives a sequence at most 128 chunks of 2048 tokens; a page-table row that could hold more
    used to be accepted and then failed at every decode launch."""
    from lokahi_b200 import _lib
    ok = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=4, max_seqs=1,
                                     max_pages_per_seq=_lib.MAX_TOKENS_PER_SEQ // 16, page_size=16, device=-1))
    assert _lib.lib.skv_decode_workspace_bytes(ok._h, 1, 1) == 128 * (8 + 2) * 4
    with pytest.raises(NotImplementedError, match="exceeds 262144 tokens per sequence"):
        L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=4, max_seqs=1,
                                    max_pages_per_seq=_lib.MAX_TOKENS_PER_SEQ // 16 + 1, page_size=16, device=-1))


def test_step_bookkeeping_on_a_host_only_pool_and_exchange_sizes():
    """The one-call step does the same host bookkeeping as append (lengths, page growth, replay-free), rejects a
    repeated sequence and half-given sharding arguments; exchange buffer sizes follow the documented layout."""
    import ctypes as C
    from lokahi_b200 import _lib
    pool, model = make()
    pool.set_rope(L.rope_inv_freq(8, 10000.0))
    for _ in range(3):
        assert pool.alloc_sequence() == model.alloc_sequence()
    a = _lib.SkvStepArgs(layer=1, n_seqs=2, n_q_heads=4, eps=1e-12)
    a.seq_ids = _lib.i32_array([2, 0])
    for step in range(6):                 # crosses a page boundary (page_size 4)
        assert _lib.lib.skv_decode_step_ex(pool._h, C.byref(a), None) == _lib.OK
        for s in (2, 0):
            model.append(1, s, step, 1)
        same_state(pool, model)
    a.seq_ids = _lib.i32_array([1, 1])
    assert _lib.lib.skv_decode_step_ex(pool._h, C.byref(a), None) == _lib.ERR_BAD_ARG
    assert b"listed twice" in _lib.lib.skv_last_error(pool._h)
    a.seq_ids = _lib.i32_array([1, 0])
    a.positions = _lib.i32_array([5, 6])
    assert _lib.lib.skv_decode_step_ex(pool._h, C.byref(a), None) == _lib.ERR_BAD_ARG
    assert b"together" in _lib.lib.skv_last_error(pool._h)
    same_state(pool, model)
    # head gather: 2 halves x world x rows x (D * esize / 8) 16-byte words
    assert _lib.lib.skv_exchange_bytes(_lib.XCHG_HEAD_GATHER, 8, 64, 4, 128, _lib.BF16) == 2 * 8 * 256 * 32 * 16
    # sequence merge: world x ceil(rows / world) x (D + 2) / 2 partial words + rows x finished-row words
    assert _lib.lib.skv_exchange_bytes(_lib.XCHG_SEQ_MERGE, 8, 64, 32, 128, _lib.BF16) == 2 * 16 * (8 * 256 * 65 + 2048 * 32)
    assert _lib.lib.skv_exchange_bytes(3, 8, 64, 32, 128, _lib.BF16) == 0
    assert _lib.lib.skv_exchange_bytes(_lib.XCHG_HEAD_GATHER, 9, 64, 32, 128, _lib.BF16) == 0
