"""The one-call decode step (RoPE + append + attention + exchange) through the C ABI: every form of it against the
append + attention pair, the oracle, and itself (packed vs strided rows, early start vs ordinary launch, exchange
vs plain output, inline vs uploaded row metadata, default vs side stream)."""
import numpy as np
import pytest
import torch

import lokahi_b200 as L
from oracle import attention as oattn
from oracle import paged as opaged
from parity import TOL_BF16, assert_parity, bf16_round, parity_errors, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HQ, HKV, D, P, THETA = 32, 8, 128, 16, 500000.0


def _t(a, dtype=torch.bfloat16):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV).to(dtype)


def _pool(seed, lens, headroom, *, hkv=HKV, n_pages=None, assign=True):
    """Pool with `len(lens)` sequences of the given lengths, pages dealt from a seeded permutation and filled with
    bf16-rounded N(0,1); identical for identical arguments."""
    rng = np.random.default_rng(seed)
    n = len(lens)
    pps = max(1, max(-(-(t + 1 + headroom) // P) for t in lens))
    n_pages = n_pages or n * pps + 3
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=hkv, head_dim=D, num_pages=n_pages, max_seqs=n,
                                       max_pages_per_seq=pps, page_size=P, dtype=torch.bfloat16, rope_theta=THETA))
    perm = rng.permutation(n_pages)
    k_ref = bf16_round(rng.standard_normal((n_pages, hkv, P, D), dtype=np.float32))
    v_ref = bf16_round(rng.standard_normal((n_pages, hkv, P, D), dtype=np.float32))
    table = np.full((n, pps), -1, np.int32)
    for s in range(n):
        assert pool.alloc_sequence() == s
        if assign:
            table[s] = perm[s * pps:(s + 1) * pps]
            pool.set_page_table(s, table[s].tolist(), lens[s])
    kp, vp = pool.layer_views(0)
    kp.copy_(_t(k_ref)); vp.copy_(_t(v_ref))
    return pool, k_ref, v_ref, table


def _inputs(seed, steps, n, hq=HQ, hkv=HKV):
    g = torch.Generator(device=DEV).manual_seed(seed)
    mk = lambda *s: torch.randn(s, generator=g, device=DEV).to(torch.bfloat16)
    return mk(steps, n, hq, D), mk(steps, n, hkv, D), mk(steps, n, hkv, D)


def _same_pages(pool_a, pool_b, n, final):
    ka, va = pool_a.gather(0, n_seqs=n)
    kb, vb = pool_b.gather(0, n_seqs=n)
    for i in range(n):
        assert torch.equal(ka[i, :, :final[i]], kb[i, :, :final[i]]) and torch.equal(va[i, :, :final[i]], vb[i, :, :final[i]]), \
            f"stored pages of sequence {i} differ"


LENS = [0, 5, 15, 16, 255, 256, 300, 1023, 2047, 2048]


@pytest.mark.parametrize("mode", ["head_gather", "seq_merge"])
def test_step_with_exchange_on_one_gpu_equals_the_plain_step(mode):
    """world == 1 runs the whole exchange code of the merge kernel (self-validating stores into the receive
    buffer, polling, unpacking; for the sequence merge also the owner's merge and its broadcast) against this GPU's
    own memory: 20 steps across page, chunk and empty-sequence boundaries, result view, rotated q, lengths and
    stored pages bit-equal to the plain step."""
    n, steps = len(LENS), 20
    pool_a, *_ = _pool(56, LENS, steps)
    pool_b, *_ = _pool(56, LENS, steps)
    if mode == "head_gather":
        ex = L.PeerGather(L.HeadShard(0, 1, HQ, HKV), n, D, torch.bfloat16, torch.device(DEV))
    else:
        ex = L.PeerSeqMerge(0, 1, n, HQ, D, torch.bfloat16, torch.device(DEV))
    q_all, k_all, v_all = _inputs(7, steps, n)
    for s in range(steps):
        qa, qb = q_all[s].clone(), q_all[s].clone()
        before = L._lib.lib.skv_launch_count()
        out_a = pool_a.decode_step(0, qa, k_all[s], v_all[s])
        view = pool_b.decode_step(0, qb, k_all[s], v_all[s], exchange=ex)
        assert L._lib.lib.skv_launch_count() - before == 4, "two launches per step, with or without the exchange"
        got = view[0] if mode == "head_gather" else view
        assert torch.equal(got, out_a), f"step {s}"
        assert torch.equal(qa, qb)
        assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0))
    _same_pages(pool_a, pool_b, n, [t + steps for t in LENS])
    assert pool_a.check_device_status() == 0 and pool_b.check_device_status() == 0
    # attention without the append through the same exchange
    q = q_all[0]
    view = pool_b.decode_attention_xchg(0, q, ex)
    assert torch.equal(view[0] if mode == "head_gather" else view, pool_a.decode_attention(0, q))
    # a sequence list in another order
    ids = [7, 2, 9]
    qa, qb = q_all[1, :3].clone(), q_all[1, :3].clone()
    k3, v3 = k_all[1, :3].contiguous(), v_all[1, :3].contiguous()
    if mode == "head_gather":
        ex3 = L.PeerGather(L.HeadShard(0, 1, HQ, HKV), 3, D, torch.bfloat16, torch.device(DEV))
    else:
        ex3 = L.PeerSeqMerge(0, 1, 3, HQ, D, torch.bfloat16, torch.device(DEV))
    out_a = pool_a.decode_step(0, qa, k3, v3, seq_ids=ids)
    view = pool_b.decode_step(0, qb, k3, v3, seq_ids=ids, exchange=ex3)
    assert torch.equal(view[0] if mode == "head_gather" else view, out_a)
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0)) and pool_b.check_device_status() == 0


def test_consecutive_steps_that_start_early_are_bit_identical():
    """With `consecutive=True` and inputs that were complete beforehand the split-K kernel of a step runs ahead of
    the previous step's merge kernel.  40 steps enqueued back to back without a host wait, against the same steps
    launched the ordinary way: outputs, rotated q, lengths and pages bit-equal.  Then steps whose q IS the previous
    step's rotated q (the library has to notice and fall back) give what the ordinary launch gives."""
    n, steps = len(LENS), 40
    pool_a, *_ = _pool(57, LENS, steps + 8)
    pool_b, *_ = _pool(57, LENS, steps + 8)
    q_all, k_all, v_all = _inputs(8, steps, n)
    qa_all, qb_all = q_all.clone(), q_all.clone()
    out_a, out_b = torch.empty_like(q_all), torch.empty_like(q_all)
    torch.cuda.synchronize()
    for s in range(steps):
        pool_a.decode_step(0, qa_all[s], k_all[s], v_all[s], out=out_a[s])
    for s in range(steps):
        pool_b.decode_step(0, qb_all[s], k_all[s], v_all[s], out=out_b[s], consecutive=True)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b) and torch.equal(qa_all, qb_all)
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0))
    _same_pages(pool_a, pool_b, n, [t + steps for t in LENS])
    # aliasing: the rotated q of one step is the input of the next
    qa, qb = q_all[0].clone(), q_all[0].clone()
    oa, ob = torch.empty_like(qa), torch.empty_like(qb)
    torch.cuda.synchronize()
    for s in range(4):
        pool_a.decode_step(0, qa, k_all[s], v_all[s], out=oa)
    for s in range(4):
        pool_b.decode_step(0, qb, k_all[s], v_all[s], out=ob, consecutive=True)
    torch.cuda.synchronize()
    assert torch.equal(qa, qb) and torch.equal(oa, ob)
    # with the exchange (world == 1) as well; its two result buffers alternate, so the last two views stay intact
    ex = L.PeerGather(L.HeadShard(0, 1, HQ, HKV), n, D, torch.bfloat16, torch.device(DEV))
    views = []
    qa_all, qb_all = q_all.clone(), q_all.clone()
    torch.cuda.synchronize()
    for s in range(4):
        pool_a.decode_step(0, qa_all[s], k_all[s], v_all[s], out=out_a[s])
    for s in range(4):
        views.append(pool_b.decode_step(0, qb_all[s], k_all[s], v_all[s], exchange=ex, consecutive=True))
    torch.cuda.synchronize()
    for s in (2, 3):
        assert torch.equal(views[s][0], out_a[s])
    assert pool_a.check_device_status() == 0 and pool_b.check_device_status() == 0


def test_step_takes_strided_rows_of_one_fused_projection_output():
    """q, k and v as slices of one [n, (Hq + 2 Hkv) * D] buffer (the output of one fused QKV projection) and a
    strided output: identical to the packed call, and the bytes between the rows are left alone."""
    lens = [3, 16, 700, 1024, 90]
    n = len(lens)
    pool_a, *_ = _pool(58, lens, 8)
    pool_b, *_ = _pool(58, lens, 8)
    g = torch.Generator(device=DEV).manual_seed(9)
    width = (HQ + 2 * HKV) * D
    for s in range(3):
        fused = torch.randn((n, width), generator=g, device=DEV).to(torch.bfloat16)
        keep = fused.clone()
        q = fused[:, :HQ * D].view(n, HQ, D)
        k = fused[:, HQ * D:(HQ + HKV) * D].view(n, HKV, D)
        v = fused[:, (HQ + HKV) * D:].view(n, HKV, D)
        assert not q.is_contiguous()
        qa, ka, va = q.contiguous(), k.contiguous(), v.contiguous()
        out_wide = torch.full((n, HQ * D + 64), 3.0, device=DEV, dtype=torch.bfloat16)
        out_a = pool_a.decode_step(0, qa, ka, va)
        pool_b.decode_step(0, q, k, v, out=out_wide[:, :HQ * D].view(n, HQ, D))
        assert torch.equal(out_wide[:, :HQ * D].reshape(n, HQ, D), out_a) and bool((out_wide[:, HQ * D:] == 3.0).all())
        assert torch.equal(q, qa), "rotated in place inside the fused buffer"
        assert torch.equal(fused[:, HQ * D:], keep[:, HQ * D:]), "k and v slices are read only"
    _same_pages(pool_a, pool_b, n, [t + 3 for t in lens])
    assert pool_b.check_device_status() == 0


def test_step_grows_pages_through_the_allocator_and_matches_the_oracle():
    """Sequences that start empty and grow by steps only: every 16th step a sequence takes a fresh page from the
    allocator (a page-table update between the two kernels).  Page tables equal the allocator model, lengths equal,
    last outputs equal the oracle on the logical history."""
    n, steps = 5, 40
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=HKV, head_dim=D, num_pages=n * 4, max_seqs=n,
                                       max_pages_per_seq=4, page_size=P, dtype=torch.bfloat16, rope_theta=THETA))
    model = opaged.PagePoolModel(1, n * 4, P, n, 4)
    for s in range(n):
        assert pool.alloc_sequence() == model.alloc_sequence() == s
    q_all, k_all, v_all = _inputs(10, steps, n)
    hist_k = np.zeros((n, HKV, steps, D), np.float32)
    hist_v = np.zeros((n, HKV, steps, D), np.float32)
    for s in range(steps):
        q = q_all[s].clone()
        out = pool.decode_step(0, q, k_all[s], v_all[s])
        for i in range(n):
            model.append(0, i, s, 1)
        hist_k[:, :, s] = bf16_round(opaged.rope_rows(to_np(k_all[s]), np.full(n, s), THETA))
        hist_v[:, :, s] = to_np(v_all[s])
    torch.cuda.synchronize()
    for i in range(n):
        assert np.array_equal(pool.page_table(i), model.page_table[i, :model.num_seq_pages[i]])
    assert list(pool.lengths(0)) == [steps] * n and pool.check_device_status() == 0
    # the kernel's sincosf and NumPy's cos/sin may differ in the last float32 bit, which now and then moves a bf16
    # rounding: the rotated q agrees with the oracle's RoPE to one bf16 step
    qr = bf16_round(opaged.rope_rows(to_np(q_all[steps - 1]), np.full(n, steps - 1), THETA))
    assert np.all(np.abs(to_np(q) - qr) <= np.abs(qr) * 2.0 ** -7 + 1e-30), "rotated q against the oracle's RoPE"
    qr = to_np(q)
    for i in range(n):
        ref = oattn.chunked_grouped_attention(qr[i][None, :, None, :], hist_k[i:i + 1], hist_v[i:i + 1],
                                              query_positions=np.array([steps - 1], dtype=np.int32))
        assert_parity(out[i], ref[0, :, 0, :], TOL_BF16, f"sequence {i}")
    kd, vd = pool.gather(0, n_seqs=n)
    assert np.array_equal(to_np(vd), hist_v), "stored V bytes"
    assert np.all(np.abs(to_np(kd) - hist_k) <= np.abs(hist_k) * 2.0 ** -7 + 1e-30), "stored (rotated) K against the oracle's RoPE"


@pytest.mark.parametrize("split", ["interleaved", "contiguous"])
def test_sequence_sharded_step_on_three_pools_merges_to_the_unsharded_step(split):
    """Three pools on one GPU stand in for three ranks that each hold a share of every sequence's tokens.  Each
    step every pool rotates q at the token's global position, the owner of that position stores the token, all
    write un-normalised partial rows, and the merge of the three equals the step on one pool that holds everything
    (bf16 tolerance: the partial sums are formed in a different order) and the oracle."""
    R, steps = 3, 20
    lens = [0, 5, 40, 100, 517, 1400]
    n = len(lens)
    if split == "interleaved":
        shards = [L.InterleavedShard(r, R, 32, P) for r in range(R)]
        pos_of = lambda sh, t: sh.global_positions(t)
        count = lambda sh, t: sh.local_count(t)
    else:
        shards = [L.SequenceShard(r, R, 512, P) for r in range(R)]
        pos_of = lambda sh, t: list(range(sh.local_range(t)[0], sh.local_range(t)[0] + sh.local_range(t)[1]))
        count = lambda sh, t: sh.local_range(t)[1]
    rng = np.random.default_rng(77)
    cap = max(lens) + steps
    k_hist = [bf16_round(rng.standard_normal((HKV, cap, D), dtype=np.float32)) for _ in lens]
    v_hist = [bf16_round(rng.standard_normal((HKV, cap, D), dtype=np.float32)) for _ in lens]

    def make(positions_of):
        pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=HKV, head_dim=D, num_pages=n * 100, max_seqs=n,
                                           max_pages_per_seq=100, page_size=P, dtype=torch.bfloat16, rope_theta=THETA))
        for s in range(n):
            assert pool.alloc_sequence() == s
            idx = positions_of(s)
            if idx:
                pool.append(0, _t(k_hist[s][None, :, idx]), _t(v_hist[s][None, :, idx]), seq_ids=[s], start_pos=[0])
        return pool

    whole = make(lambda s: list(range(lens[s])))
    parts_pools = [make(lambda s, sh=sh: pos_of(sh, lens[s])) for sh in shards]
    q_all, k_all, v_all = _inputs(11, steps, n)
    for st in range(steps):
        cur = [t + st for t in lens]
        q_ref = q_all[st].clone()
        ref = whole.decode_step(0, q_ref, k_all[st], v_all[st])
        parts = []
        for sh, pool in zip(shards, parts_pools):
            q = q_all[st].clone()
            store = [sh.owner(p) == sh.rank for p in cur]
            parts.append(pool.decode_step(0, q, k_all[st], v_all[st], positions=cur, store=store, partial=True))
            assert torch.equal(q, q_ref), "every rank rotates q at the global position"
            assert list(pool.lengths(0)) == [count(sh, t + 1) for t in cur]
        merged = L.merge_partials(torch.stack(parts).contiguous())
        assert parity_errors(merged, to_np(ref))[0] <= TOL_BF16, f"step {st}"
    for pool in parts_pools:
        assert pool.check_device_status() == 0
    # the union of the shards' pages is the unsharded history, byte for byte
    kw, vw = whole.gather(0, n_seqs=n)
    for sh, pool in zip(shards, parts_pools):
        kl, vl = pool.gather(0, n_seqs=n)
        for s in range(n):
            idx = pos_of(sh, lens[s] + steps)
            assert torch.equal(kl[s, :, :len(idx)], kw[s][:, idx]) and torch.equal(vl[s, :, :len(idx)], vw[s][:, idx])
    # last step against the oracle on the logical history
    final = [t + steps for t in lens]
    k_np, v_np = to_np(kw), to_np(vw)
    for i in (0, 3, 5):
        o = oattn.chunked_grouped_attention(to_np(q_ref[i])[None, :, None, :], k_np[i:i + 1, :, :final[i]], v_np[i:i + 1, :, :final[i]],
                                            query_positions=np.array([final[i] - 1], dtype=np.int32))
        assert_parity(merged[i], o[0, :, 0, :], TOL_BF16, f"merged step vs oracle, sequence {i}")


def test_longest_rows_first_changes_nothing_but_the_order_of_the_work(skv_switch):
    """SKV_DECODE_ORDER=1: the split-K grid works on the rows from the longest to the shortest (what a step does by
    itself when its grid holds more CTAs than the GPU does at once).  Outputs, rotated q, lengths and pages equal the
    unordered step's bit for bit, with a sequence list, over steps that start early."""
    lens = [700, 3, 1024, 0, 88, 2047, 512, 16, 300, 1500]
    n, steps = len(lens), 6
    pool_a, *_ = _pool(77, lens, steps)
    pool_b, *_ = _pool(77, lens, steps)
    q_all, k_all, v_all = _inputs(19, steps, n)
    ids = list(range(n))
    outs = {}
    for name, pool, flag in (("plain", pool_a, "0"), ("ordered", pool_b, "1")):
        skv_switch("SKV_DECODE_ORDER", flag)
        qs = q_all.clone()
        res = torch.empty_like(q_all)
        torch.cuda.synchronize()
        for s in range(steps):
            pool.decode_step(0, qs[s], k_all[s], v_all[s], out=res[s], seq_ids=ids if s % 2 else None, consecutive=s > 0)
        torch.cuda.synchronize()
        outs[name] = (res, qs)
    assert torch.equal(outs["plain"][0], outs["ordered"][0]) and torch.equal(outs["plain"][1], outs["ordered"][1])
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0))
    _same_pages(pool_a, pool_b, n, [t + steps for t in lens])
    assert pool_a.check_device_status() == 0 and pool_b.check_device_status() == 0


def test_step_with_more_rows_than_the_kernel_parameters_hold():
    """300 sequences: the per-row metadata no longer fits the kernel parameters and is uploaded instead; same
    results as the append + attention pair."""
    n = 300
    rng = np.random.default_rng(5)
    lens = [int(x) for x in rng.integers(0, 70, size=n)]
    pool_a, *_ = _pool(59, lens, 4, hkv=2)
    pool_b, *_ = _pool(59, lens, 4, hkv=2)
    q_all, k_all, v_all = _inputs(12, 2, n, hq=8, hkv=2)
    for s in range(2):
        qa, qb = q_all[s].clone(), q_all[s].clone()
        pool_a.append(0, k_all[s], v_all[s], start_pos=[t + s for t in lens], rope_k=True, q=qa, layout="bhd")
        out_a = pool_a.decode_attention(0, qa)
        out_b = pool_b.decode_step(0, qb, k_all[s], v_all[s])
        assert torch.equal(qa, qb) and parity_errors(out_b, to_np(out_a))[0] <= TOL_BF16
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0))
    _same_pages(pool_a, pool_b, n, [t + 2 for t in lens])
    assert pool_b.check_device_status() == 0


def test_pool_driven_from_a_side_stream():
    """Everything, set-up included, enqueued on a non-default (non-blocking) torch stream: table and length changes
    are published on that stream, so the kernels behind them see them.  Results equal the default-stream run."""
    lens = [5, 300, 1023]
    n, steps = len(lens), 6
    q_all, k_all, v_all = _inputs(13, steps, n)
    pool_a, *_ = _pool(60, lens, steps)
    ref = [pool_a.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(steps)]
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=DEV)
    with torch.cuda.stream(side):
        pool_b, *_ = _pool(60, lens, steps)
        got = [pool_b.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(steps)]
        pool_b.free_sequence(1)
        assert pool_b.alloc_sequence() == 1
        pool_b.reserve(1, 40)
        kv = torch.zeros((1, HKV, 33, D), device=DEV, dtype=torch.bfloat16)
        pool_b.append(0, kv, kv, seq_ids=[1], start_pos=[0])
        tail = pool_b.decode_step(0, q_all[0, 1:2].clone(), k_all[0, 1:2].contiguous(), v_all[0, 1:2].contiguous(), seq_ids=[1])
        assert pool_b.check_device_status() == 0
    side.synchronize()
    for s in range(steps):
        assert torch.equal(ref[s], got[s])
    assert list(pool_b.lengths(0)) == [lens[0] + steps, 34, lens[2] + steps] and bool(torch.isfinite(tail.float()).all())


def test_dense_attention_reports_through_its_status_word():
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn((1, 8, 256, 128), generator=g, device=DEV).to(torch.bfloat16)
    k = torch.randn((1, 2, 256, 128), generator=g, device=DEV).to(torch.bfloat16)
    out = L.chunked_grouped_attention(q, k, k)
    assert L.check_dense_attention_status(DEV) == 0 and bool(torch.isfinite(out.float()).all())


def test_consecutive_steps_across_layers_and_after_a_truncation():
    """A decode step of a multi-layer cache is one step per layer, back to back, for every token: early start has to
    hold across layers (a step of layer l may start while the steps of layers l-1 and l-2 are still running, and the
    row it must wait for was stored a whole round of layers ago).  Then the rows are cut back and regrown: the
    stored-length words the steps publish must not satisfy a wait with a value from before the cut."""
    layers, n, tokens = 3, 6, 12
    lens = [0, 7, 15, 16, 700, 2047]
    pps = -(-(max(lens) + 2 * tokens + 4) // P)

    def make():
        rng = np.random.default_rng(91)
        pool = L.PagedPool(L.PagedKVConfig(num_layers=layers, num_kv_heads=HKV, head_dim=D, num_pages=n * pps + 2, max_seqs=n,
                                           max_pages_per_seq=pps, page_size=P, dtype=torch.bfloat16, rope_theta=THETA))
        perm = rng.permutation(n * pps + 2)
        for s in range(n):
            assert pool.alloc_sequence() == s
            pool.set_page_table(s, perm[s * pps:(s + 1) * pps].tolist(), lens[s])
        g = torch.Generator(device=DEV).manual_seed(17)
        for layer in range(layers):
            kp, vp = pool.layer_views(layer)
            kp.normal_(generator=g); vp.normal_(generator=g)
        return pool

    pool_a, pool_b = make(), make()
    g = torch.Generator(device=DEV).manual_seed(18)
    mk = lambda h: torch.randn((tokens, layers, n, h, D), generator=g, device=DEV).to(torch.bfloat16)
    q_all, k_all, v_all = mk(HQ), mk(HKV), mk(HKV)
    qa, qb = q_all.clone(), q_all.clone()
    out_a, out_b = torch.empty_like(q_all), torch.empty_like(q_all)

    def run(pool, q, out, first, count, consecutive):
        for t in range(first, first + count):
            for layer in range(layers):
                pool.decode_step(layer, q[t, layer], k_all[t, layer], v_all[t, layer], out=out[t, layer], consecutive=consecutive)

    torch.cuda.synchronize()
    run(pool_a, qa, out_a, 0, tokens, False)
    run(pool_b, qb, out_b, 0, tokens, True)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b) and torch.equal(qa, qb)
    # cut every layer back to the starting lengths and grow again with other inputs
    for pool in (pool_a, pool_b):
        for layer in range(layers):
            for s in range(n):
                pool.truncate(layer, lens[s], seq_ids=[s])
    q2 = torch.randn((tokens, layers, n, HQ, D), generator=g, device=DEV).to(torch.bfloat16)
    qa, qb = q2.clone(), q2.clone()
    torch.cuda.synchronize()
    run(pool_a, qa, out_a, 0, tokens, False)
    run(pool_b, qb, out_b, 0, tokens, True)
    torch.cuda.synchronize()
    assert torch.equal(out_a, out_b) and torch.equal(qa, qb)
    for layer in range(layers):
        assert np.array_equal(pool_a.lengths(layer), pool_b.lengths(layer))
        ka, va = pool_a.gather(layer, n_seqs=n)
        kb, vb = pool_b.gather(layer, n_seqs=n)
        assert torch.equal(ka, kb) and torch.equal(va, vb)
    assert pool_a.check_device_status() == 0 and pool_b.check_device_status() == 0


@pytest.mark.parametrize("with_exchange", [False, True])
def test_host_fed_pipeline_gives_the_direct_steps_results(with_exchange):
    """`HostStepPipeline`: every step's q | k | v row comes from pinned host memory and every result goes back to it,
    uploads and read-backs overlapping the steps.  Results (through a two-row ring and through a full-length
    output) equal the same steps made directly with device tensors; lengths and pages too."""
    lens = [5, 16, 300, 1023, 2047]
    n, steps = len(lens), 9
    pool_a, *_ = _pool(61, lens, 5 * steps)
    pool_b, *_ = _pool(61, lens, 5 * steps)
    q_all, k_all, v_all = _inputs(14, steps, n)
    ref = torch.stack([pool_a.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(steps)])
    rows = torch.cat([q_all.reshape(steps, -1), k_all.reshape(steps, -1), v_all.reshape(steps, -1)], dim=1).cpu().pin_memory()
    ex = L.PeerGather(L.HeadShard(0, 1, HQ, HKV), n, D, torch.bfloat16, torch.device(DEV)) if with_exchange else None
    pipe = L.HostStepPipeline(pool_b, 0, n, HQ, exchange=ex)
    shape = (1, n, HQ, D) if with_exchange else (n, HQ, D)
    full = torch.empty((steps,) + shape, dtype=torch.bfloat16).pin_memory()
    pipe.run(rows, full)
    assert torch.equal(full.reshape(steps, n, HQ, D), ref.cpu())
    ring = torch.empty((2,) + shape, dtype=torch.bfloat16).pin_memory()
    ref2 = torch.stack([pool_a.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(steps)])
    pipe.run(rows, ring)                                   # a second run on the same pipeline, results through a ring
    assert torch.equal(ring[(steps - 1) % 2].reshape(n, HQ, D), ref2[-1].cpu())
    assert torch.equal(ring[(steps - 2) % 2].reshape(n, HQ, D), ref2[-2].cpu())
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0)) and pool_b.check_device_status() == 0
    _same_pages(pool_a, pool_b, n, [t + 2 * steps for t in lens])
    # the host one step behind instead of two, and steps that never start beside their predecessors: same results
    short = 5
    ref3 = torch.stack([pool_a.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(short)])
    pipe1 = L.HostStepPipeline(pool_b, 0, n, HQ, exchange=ex, lookahead=1, consecutive=False)
    part = torch.empty((short,) + shape, dtype=torch.bfloat16).pin_memory()
    pipe1.run(rows[:short], part)
    assert torch.equal(part.reshape(short, n, HQ, D), ref3.cpu())
    # steps in blocks of three (one event wait before a block, one record after it; 3 + 3 + 2 steps), six buffers in
    # rotation, results through a six-row ring
    more = 8
    ref4 = torch.stack([pool_a.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(more)])
    ex3 = L.PeerGather(L.HeadShard(0, 1, HQ, HKV), n, D, torch.bfloat16, torch.device(DEV), n_results=6) if with_exchange else None
    pipe3 = L.HostStepPipeline(pool_b, 0, n, HQ, exchange=ex3, block=3)
    ring6 = torch.empty((6,) + shape, dtype=torch.bfloat16).pin_memory()
    pipe3.run(rows[:more], ring6)
    for s_ in range(more - 6, more):
        assert torch.equal(ring6[s_ % 6].reshape(n, HQ, D), ref4[s_].cpu()), f"blocks of 3, step {s_}"
    with pytest.raises(ValueError, match="match"):
        pipe3.run(rows[:more], ring)                       # a two-row ring is too short for blocks of three
    assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0)) and pool_b.check_device_status() == 0
    if with_exchange:
        # arguments that vary by step (the positions and store flags of sequence sharding, here with one rank that
        # stores everything), calls bound per step, blocks of two
        base = [int(t) for t in pool_b.lengths(0)]
        extra = 5
        ref5 = torch.stack([pool_a.decode_step(0, q_all[s].clone(), k_all[s], v_all[s]) for s in range(extra)])
        merge = L.PeerSeqMerge(0, 1, n, HQ, D, torch.bfloat16, torch.device(DEV), n_results=4)
        pipe5 = L.HostStepPipeline(pool_b, 0, n, HQ, exchange=merge, block=2, n_steps=extra,
                                   step_args=lambda i: {"positions": [t + i for t in base], "store": [True] * n})
        got5 = torch.empty((extra, n, HQ, D), dtype=torch.bfloat16).pin_memory()
        pipe5.run(rows[:extra], got5)
        assert parity_errors(got5, to_np(ref5))[0] <= TOL_BF16, "per-step arguments, blocks of two"
        assert np.array_equal(pool_a.lengths(0), pool_b.lengths(0)) and pool_b.check_device_status() == 0
    with pytest.raises(ValueError, match="pinned"):
        pipe.run(rows.clone(), ring)


@pytest.mark.parametrize("mode", ["head_gather", "seq_merge"])
def test_exchange_on_a_float32_pool_through_the_cuda_core_kernels(mode):
    """float32 storage, head_dim 64, 4 query heads per KV head... none of it fits the one-kernel step, so the step is
    the append + attention pair and the exchange runs behind the CUDA-core split-K kernel: same rows as without it."""
    n, hq, hkv, d = 4, 8, 2, 64
    lens = [0, 9, 130, 700]

    def make():
        rng = np.random.default_rng(33)
        pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=hkv, head_dim=d, num_pages=4 * 50, max_seqs=n,
                                           max_pages_per_seq=50, page_size=P, dtype=torch.float32, rope_theta=10000.0))
        for s in range(n):
            assert pool.alloc_sequence() == s
            if lens[s]:
                kv = _t(rng.standard_normal((1, hkv, lens[s], d), dtype=np.float32), torch.float32)
                pool.append(0, kv, kv * 0.5, seq_ids=[s], start_pos=[0])
        return pool

    pool_a, pool_b = make(), make()
    dev = torch.device(DEV)
    ex = (L.PeerGather(L.HeadShard(0, 1, hq, hkv), n, d, torch.float32, dev) if mode == "head_gather"
          else L.PeerSeqMerge(0, 1, n, hq, d, torch.float32, dev))
    g = torch.Generator(device=DEV).manual_seed(4)
    for step in range(3):
        q = torch.randn((n, hq, d), generator=g, device=DEV)
        k = torch.randn((n, hkv, d), generator=g, device=DEV)
        v = torch.randn((n, hkv, d), generator=g, device=DEV)
        qa, qb = q.clone(), q.clone()
        out_a = pool_a.decode_step(0, qa, k, v)
        view = pool_b.decode_step(0, qb, k, v, exchange=ex)
        got = view[0] if mode == "head_gather" else view
        assert torch.equal(qa, qb) and torch.equal(got, out_a), f"step {step}"
    q = torch.randn((n, hq, d), generator=g, device=DEV)
    view = pool_b.decode_attention_xchg(0, q, ex, q_pos=[-1, 3, 100, 702])
    ref = pool_a.decode_attention(0, q, q_pos=[-1, 3, 100, 702])
    assert torch.equal(view[0] if mode == "head_gather" else view, ref) and not bool(ref[0].any())
    assert pool_b.check_device_status() == 0
