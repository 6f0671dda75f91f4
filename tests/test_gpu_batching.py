"""The batched-request decode loop: requests of different lengths join and leave while it runs.  Every emitted
token must be the one the NumPy decoder oracle produces for that request alone; page tables must follow the
allocator model; a run with parked pages and look-ahead must give the same tokens."""
import numpy as np
import pytest
import torch

import lokahi_b200 as L
from oracle import decoder as od
from oracle.kvcache import ConcatKVCache
from oracle.paged import PagePoolModel
from parity import TOL_BF16, assert_parity_logits, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _to_torch(weights, dtype):
    return {k: torch.from_numpy(v).to(DEV).to(dtype) for k, v in weights.items()}


def _record_pool_ops(pool):
    """Wrap the three calls that change page ownership so that a test can replay them on the allocator model."""
    ops = []
    alloc, reserve, free = pool.alloc_sequence, pool.reserve, pool.free_sequence

    def alloc_sequence():
        s = alloc()
        ops.append(("alloc", s))
        return s

    def reserve_(seq, total):
        reserve(seq, total)
        ops.append(("reserve", seq, total))

    def free_sequence(seq):
        free(seq)
        ops.append(("free", seq))

    pool.alloc_sequence, pool.reserve, pool.free_sequence = alloc_sequence, reserve_, free_sequence
    return ops


def _replay(ops, model, done):
    for op in ops[done:]:
        if op[0] == "alloc":
            assert model.alloc_sequence() == op[1]
        elif op[0] == "reserve":
            model.reserve(op[1], op[2])
        else:
            model.free_sequence(op[1])
    return len(ops)


def test_requests_join_and_leave_and_every_token_matches_the_oracle_alone():
    cfg = od.make_config(vocab_size=97, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128)
    w = od.random_weights(cfg, seed=21, std=0.15)
    model = L.PagedDecoder(cfg, _to_torch(w, torch.float32))
    oracle = od.DecoderOracle(cfg, w)
    P = 4
    pool = L.PagedPool(L.PagedKVConfig(num_layers=2, num_kv_heads=2, head_dim=16, num_pages=40, max_seqs=4, max_pages_per_seq=12,
                                       page_size=P, dtype=torch.float32))
    amodel = PagePoolModel(2, 40, P, 4, 12)
    ops = _record_pool_ops(pool)
    loop = L.BatchedDecodeLoop(model, pool, max_batch=2, prefill_token_budget=5, record_logits=True)
    rng = np.random.default_rng(3)
    plan = {0: [(rng.integers(0, 97, 7).tolist(), 9), (rng.integers(0, 97, 3).tolist(), 5)],      # quantum -> requests
            3: [(rng.integers(0, 97, 12).tolist(), 6)],
            7: [(rng.integers(0, 97, 1).tolist(), 12), (rng.integers(0, 97, 9).tolist(), 4)]}
    submitted, replayed, live_seen = {}, 0, set()
    cancelled = None
    for quantum in range(200):
        for prompt, n_new in plan.get(quantum, []):
            submitted[loop.submit(prompt, n_new)] = (prompt, n_new)
        if quantum == 9:
            cancelled = 3
            loop.cancel(cancelled)
        if not loop.pending() and quantum > 7:
            break
        loop.step()
        replayed = _replay(ops, amodel, replayed)
        for req in loop.requests.values():            # page-table rows of the live sequences follow the allocator model
            if req.seq is not None:
                live_seen.add(req.request_id)
                assert np.array_equal(pool.page_table(req.seq), amodel.page_table[req.seq, :amodel.num_seq_pages[req.seq]])
        assert len(loop.ready) <= 4 and pool.check_device_status() == 0
    assert not loop.pending() and len(live_seen) == 5
    assert pool.counters()["free_pages"] == 40 and pool.counters()["live_sequences"] == 0, "every page came back"
    assert loop.stats["decode_batches"] > 10 and max(len(r.generated) for r in loop.requests.values()) == 9
    for rid, (prompt, n_new) in submitted.items():
        req = loop.requests[rid]
        expect = od.greedy_generate(oracle, np.array([prompt]), max_new_tokens=n_new, temperature=1.0,
                                    past_key_values=ConcatKVCache(cfg))[0, len(prompt):].tolist()
        if rid == cancelled:
            assert req.finished == "cancelled" and req.generated == expect[:len(req.generated)] and len(req.generated) < n_new
        else:
            assert req.finished == "length" and req.generated == expect, f"request {rid}"
    # logits of one request, step by step, against the oracle run alone (the first entry is the prefill's)
    rid = 2
    prompt, n_new = submitted[rid]
    cache = ConcatKVCache(cfg)
    logits = oracle(np.array([prompt]), past_key_values=cache, use_cache=True)[0, -1]
    for t, got in enumerate(loop.requests[rid].logits):
        assert np.allclose(to_np(got), logits, atol=1e-4, rtol=1e-4), f"logits of request {rid}, token {t}"
        logits = oracle(np.array([[loop.requests[rid].generated[t]]]), past_key_values=cache, use_cache=True)[0, -1]


def test_end_of_sequence_token_retires_a_request_and_zero_new_tokens_is_a_no_op():
    cfg = od.make_config(vocab_size=31, hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                         num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=64)
    w = od.random_weights(cfg, seed=5, std=0.2)
    model = L.PagedDecoder(cfg, _to_torch(w, torch.float32))
    oracle = od.DecoderOracle(cfg, w)
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=16, num_pages=16, max_seqs=2, max_pages_per_seq=8,
                                       page_size=4, dtype=torch.float32))
    prompt = [4, 9, 2]
    alone = od.greedy_generate(oracle, np.array([prompt]), max_new_tokens=10, temperature=1.0,
                               past_key_values=ConcatKVCache(cfg))[0, 3:].tolist()
    eos = alone[4]
    stop = alone.index(eos)
    loop = L.BatchedDecodeLoop(model, pool)
    a = loop.submit(prompt, 10, eos_token_id=eos)
    b = loop.submit([1, 2], 0)
    with pytest.raises(ValueError, match="non-empty"):
        loop.submit([], 3)
    out = loop.run()
    assert out[a] == alone[:stop + 1] and loop.requests[a].finished == "eos"
    assert out[b] == [] and loop.requests[b].finished == "length"
    assert pool.counters()["live_sequences"] == 0


def test_admission_waits_for_pages_and_resumes_when_a_request_leaves():
    """Reservations are all-or-nothing: a request whose prompt + output bound does not fit stays queued (nothing is
    changed) and is admitted once an earlier request has given its pages back."""
    cfg = od.make_config(vocab_size=31, hidden_size=32, intermediate_size=48, num_hidden_layers=1,
                         num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=64)
    w = od.random_weights(cfg, seed=6, std=0.2)
    model = L.PagedDecoder(cfg, _to_torch(w, torch.float32))
    oracle = od.DecoderOracle(cfg, w)
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=16, num_pages=6, max_seqs=4, max_pages_per_seq=6,
                                       page_size=4, dtype=torch.float32))
    loop = L.BatchedDecodeLoop(model, pool)
    first = loop.submit([3, 1, 4, 1, 5, 9, 2, 6], 8)          # 16 tokens: four of the six pages
    second = loop.submit([2, 7, 1, 8, 2, 8], 6)               # 12 tokens: three pages -- has to wait
    loop.step()
    assert loop.requests[second].seq is None and loop.stats["admission_deferrals"] >= 1
    assert pool.counters()["free_pages"] == 2
    out = loop.run()
    for rid, prompt, n in ((first, [3, 1, 4, 1, 5, 9, 2, 6], 8), (second, [2, 7, 1, 8, 2, 8], 6)):
        expect = od.greedy_generate(oracle, np.array([prompt]), max_new_tokens=n, temperature=1.0,
                                    past_key_values=ConcatKVCache(cfg))[0, len(prompt):].tolist()
        assert out[rid] == expect
    assert pool.counters()["free_pages"] == 6


def _bf16_setup(host_pages=0, seed=31):
    cfg = od.make_config(vocab_size=128, hidden_size=512, intermediate_size=768, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512, rope_theta=500000.0)
    w = od.random_weights(cfg, seed=seed, std=0.05)
    model = L.PagedDecoder(cfg, _to_torch(w, torch.bfloat16))
    pool = L.PagedPool(L.PagedKVConfig(num_layers=2, num_kv_heads=2, head_dim=128, num_pages=64, max_seqs=6, max_pages_per_seq=16,
                                       page_size=16, dtype=torch.bfloat16, host_pages=host_pages))
    rng = np.random.default_rng(seed)
    reqs = [(rng.integers(0, 128, n).tolist(), m) for n, m in ((40, 12), (3, 20), (70, 6), (17, 15), (100, 9))]
    return cfg, model, pool, reqs


def _run_bf16(loop, reqs):
    ids = {}
    for quantum in range(300):
        if quantum == 0:
            for r in reqs[:2]:
                ids[loop.submit(*r)] = r
        if quantum == 4:
            for r in reqs[2:4]:
                ids[loop.submit(*r)] = r
        if quantum == 8:
            ids[loop.submit(*reqs[4])] = reqs[4]
        if not loop.pending() and quantum > 8:
            break
        loop.step()
    assert not loop.pending()
    return ids


def test_bf16_loop_through_the_one_kernel_step_matches_each_sequence_decoded_alone():
    """bf16, head_dim 128: the decode batch goes through the one-kernel step with a sequence list and strided rows of
    one fused projection.  Each request's logits, step by step, against PagedDecoder fed the same tokens alone
    (the GEMMs see another batch size, so the comparison is at bf16 tolerance, not on the argmax)."""
    cfg, model, pool, reqs = _bf16_setup()
    loop = L.BatchedDecodeLoop(model, pool, max_batch=3, prefill_token_budget=64, record_logits=True)
    launches = L._lib.lib.skv_launch_count()
    ids = _run_bf16(loop, reqs)
    assert pool.check_device_status() == 0 and pool.counters()["live_sequences"] == 0
    assert L._lib.lib.skv_launch_count() > launches
    single = L.PagedDecoder(cfg, model.w, decode_graphs=False)
    for rid, (prompt, n_new) in ids.items():
        req = loop.requests[rid]
        assert len(req.generated) == n_new and len(req.logits) == n_new
        cache = L.PagedKVCache(cfg, cache_dir=None)
        logits = single(torch.tensor([prompt]), past_key_values=cache, use_cache=True)[0, -1]
        for t in range(n_new):
            assert_parity_logits(req.logits[t], to_np(logits), TOL_BF16, f"request {rid}, token {t}", max_outlier_fraction=0.02)
            logits = single(torch.tensor([[req.generated[t]]]), past_key_values=cache, use_cache=True)[0, -1]
        cache.clear()


def test_loop_with_parked_pages_and_look_ahead_gives_the_same_tokens():
    """A device-page budget below the working set: sequences that wait for their turn are parked in host memory and
    requested back one batch ahead.  Same tokens and logits as the run with everything resident, bit for bit."""
    cfg, model, pool_a, reqs = _bf16_setup()
    loop_a = L.BatchedDecodeLoop(model, pool_a, max_batch=2, prefill_token_budget=128, record_logits=True)
    ids_a = _run_bf16(loop_a, reqs)
    cfg, model_b, pool_b, _ = _bf16_setup(host_pages=64)
    residency = L.KVPageResidency(pool_b, budget_pages=18, group_pages=4)
    prefetcher = L.KVPagePrefetcher(residency)
    loop_b = L.BatchedDecodeLoop(model_b, pool_b, max_batch=2, prefill_token_budget=128, prefetcher=prefetcher, record_logits=True)
    ids_b = _run_bf16(loop_b, reqs)
    assert pool_b.check_device_status() == 0
    snap = prefetcher.snapshot()
    assert pool_b.counters()["pages_evicted"] > 0 and snap.pages_loaded > 0, "the budget forced parking and loading"
    for rid in ids_a:
        ra, rb = loop_a.requests[rid], loop_b.requests[rid]
        assert ra.generated == rb.generated
        for la, lb in zip(ra.logits, rb.logits):
            assert torch.equal(la, lb)
