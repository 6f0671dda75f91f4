"""KV-head sharding host logic on CPU: two gloo ranks each compute their head slice with the oracle,
all-gather, and must reproduce the unsharded result bit for bit (the reference loops over KV heads
independently, mlx_ops.py:81-87, so the split changes no arithmetic)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention as oattn


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q, k, v, pos, full, result_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import importlib.util
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        spec = importlib.util.spec_from_file_location("_sharding", os.path.join(root, "lokahi_b200", "sharding.py"))
        sh = importlib.util.module_from_spec(spec)
        import sys
        sys.modules["_sharding"] = sh
        spec.loader.exec_module(sh)
        shard = sh.HeadShard(rank, world, q.shape[1], k.shape[1])
        ql, kl, vl = shard.take_q(q), shard.take_kv(k), shard.take_kv(v)
        local = oattn.chunked_grouped_attention(ql.numpy(), kl.numpy(), vl.numpy(), query_positions=pos, k_block_size=8)
        out = sh.gather_head_outputs(torch.from_numpy(local), shard)
        ok = bool(np.array_equal(out.numpy(), full))
        # decode layout [n_seqs, heads, D] with a preallocated buffer
        dec = torch.from_numpy(np.ascontiguousarray(local[:, :, -1, :]))
        buf = torch.empty((world,) + tuple(dec.shape))
        out2 = sh.gather_head_outputs(dec, shard, buffer=buf)
        ok = ok and bool(np.array_equal(out2.numpy(), full[:, :, -1, :]))
        result_queue.put((rank, ok, shard.local_q_heads, shard.local_kv_heads))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_head_sharding_reproduces_unsharded_attention():
    rng = np.random.default_rng(31)
    q = rng.standard_normal((2, 8, 5, 16), dtype=np.float32)
    k = rng.standard_normal((2, 4, 19, 16), dtype=np.float32)
    v = rng.standard_normal((2, 4, 19, 16), dtype=np.float32)
    pos = np.arange(14, 19, dtype=np.int32)
    full = oattn.chunked_grouped_attention(q, k, v, query_positions=pos, k_block_size=8)
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), pos, full, queue))
             for r in range(2)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] for r in results) and all(r[2:] == (4, 2) for r in results)


def test_shard_validation():
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("_sharding2", os.path.join(root, "lokahi_b200", "sharding.py"))
    sh = importlib.util.module_from_spec(spec)
    import sys
    sys.modules["_sharding2"] = sh
    spec.loader.exec_module(sh)
    s = sh.HeadShard(3, 4, 32, 8)
    assert (s.local_q_heads, s.local_kv_heads, s.q_slice, s.kv_slice) == (8, 2, slice(24, 32), slice(6, 8))
    with pytest.raises(ValueError, match="divisible by the world size"):
        sh.HeadShard(0, 3, 32, 8)
    with pytest.raises(ValueError, match="divisible by key/value heads"):
        sh.HeadShard(0, 1, 30, 8)
    with pytest.raises(ValueError, match="rank must lie"):
        sh.HeadShard(2, 2, 32, 8)
    x = torch.arange(6.0).reshape(1, 6, 1)
    assert sh.gather_head_outputs(x, sh.HeadShard(0, 1, 6, 6)) is x


def _seq_worker(rank, world, port, q, k, v, qpos, full, queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import importlib.util, sys
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        spec = importlib.util.spec_from_file_location("_sharding3", os.path.join(root, "lokahi_b200", "sharding.py"))
        sh = importlib.util.module_from_spec(spec)
        sys.modules["_sharding3"] = sh
        spec.loader.exec_module(sh)
        shard = sh.SequenceShard(rank, world, 16, 16)
        first, cnt = shard.local_range(k.shape[2])
        m, s, wv = oattn.attention_partial(q.numpy(), k.numpy()[:, :, first:first + cnt], v.numpy()[:, :, first:first + cnt],
                                           qpos - first)
        local = torch.from_numpy(np.concatenate([wv, m[..., None], s[..., None]], axis=-1))   # rows (acc, m, l)
        parts = torch.empty((world,) + tuple(local.shape))
        dist.all_gather_into_tensor(parts.view((-1,) + tuple(local.shape[1:])), local.contiguous())
        p = parts.numpy()
        merged = oattn.merge_partials([(p[r][..., -2], p[r][..., -1], p[r][..., :-2]) for r in range(world)])
        queue.put((rank, bool(np.allclose(merged, full, atol=1e-6, rtol=1e-6)), shard.owner(40), shard.local_position(20)))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_sequence_sharding_merges_to_the_unsharded_result():
    rng = np.random.default_rng(32)
    q = rng.standard_normal((2, 4, 1, 16), dtype=np.float32)
    k = rng.standard_normal((2, 2, 27, 16), dtype=np.float32)
    v = rng.standard_normal((2, 2, 27, 16), dtype=np.float32)
    qpos = np.array([[26], [9]], dtype=np.int32)
    full = oattn.chunked_grouped_attention(q, k, v, query_positions=qpos, k_block_size=1000000)
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_seq_worker, args=(r, 2, port, torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), qpos, full, queue))
             for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(queue.get(timeout=100) for _ in procs)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert results == [(0, True, 1, 20), (1, True, 1, 4)]
