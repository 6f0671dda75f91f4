"""Two-GPU checks (skipped on a one-GPU box), one process per GPU over NCCL + NVLink peer memory:
KV-head sharding (NCCL all-gather; gather fused into the merge kernel; the one-call step with the fused gather, which
is what the scaling benchmark times) and sequence sharding (the one-call step with the cross-rank merge fused in)
against the same work on one unsharded pool and against the oracle."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["SKV_ROOT"]); sys.path.insert(0, os.path.join(os.environ["SKV_ROOT"], "tests"))
import lokahi_b200 as L
from oracle import attention as oattn
from parity import TOL_BF16, assert_parity, parity_errors, to_np
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
os.environ["NCCL_NVLS_ENABLE"] = "0"
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
Hq, Hkv, D, P, THETA = 32, 8, 128, 16, 500000.0
lens = [3, 100, 1000, 2500, 0, 255]
n, steps = len(lens), 12
pps = -(-(max(lens) + steps + 8) // P)
g = torch.Generator().manual_seed(5)
k_full = torch.randn((n * pps, Hkv, P, D), generator=g).to(torch.bfloat16)
v_full = torch.randn((n * pps, Hkv, P, D), generator=g).to(torch.bfloat16)
q_all = torch.randn((steps, n, Hq, D), generator=g).to(torch.bfloat16).to(dev)
kn_all = torch.randn((steps, n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
vn_all = torch.randn((steps, n, Hkv, D), generator=g).to(torch.bfloat16).to(dev)
perm = torch.randperm(n * pps, generator=g).tolist()

def make_pool(kv_heads, k, v):
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=kv_heads, head_dim=D, num_pages=n * pps, max_seqs=n,
                                       max_pages_per_seq=pps, page_size=P, dtype=torch.bfloat16, device=rank, rope_theta=THETA))
    for s in range(n):
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, perm[s * pps:(s + 1) * pps], lens[s])
    kp, vp = pool.layer_views(0)
    kp.copy_(k.to(dev)); vp.copy_(v.to(dev))
    return pool

# ---- KV-head sharding ---------------------------------------------------------------------------------------------
full_pool = make_pool(Hkv, k_full, v_full)                                            # unsharded, on this GPU
full = full_pool.decode_attention(0, q_all[0])
shard = L.HeadShard(rank, world, Hq, Hkv)
pool = make_pool(shard.local_kv_heads, shard.take_kv(k_full).contiguous(), shard.take_kv(v_full).contiguous())
q_loc = shard.take_q(q_all[0]).contiguous()
out_nccl = L.gather_head_outputs(pool.decode_attention(0, q_loc), shard)
assert parity_errors(out_nccl, to_np(full))[0] <= TOL_BF16, "NCCL gather"
gather = L.PeerGather(shard, n, D, torch.bfloat16, dev)
for it in range(4):
    view = pool.decode_attention_xchg(0, q_loc, gather)                               # [world, n, Hq/world, D]
    torch.cuda.synchronize()
    fused = view.movedim(0, 1).reshape(n, Hq, D)
    assert torch.equal(fused, out_nccl), f"fused gather, epoch {it + 1}"
# the one-call step with the fused gather: what `bench.py --gpus N` times
for s in range(steps):
    q_ref = q_all[s].clone()
    ref = full_pool.decode_step(0, q_ref, kn_all[s], vn_all[s])
    q_l = shard.take_q(q_all[s]).contiguous()
    k_l, v_l = shard.take_kv(kn_all[s]).contiguous(), shard.take_kv(vn_all[s]).contiguous()
    ids = None if s % 3 else list(range(n))                                           # with and without a sequence list
    view = pool.decode_step(0, q_l, k_l, v_l, exchange=gather, seq_ids=ids)
    torch.cuda.synchronize()
    got = view.movedim(0, 1).reshape(n, Hq, D)
    assert parity_errors(got, to_np(ref))[0] <= TOL_BF16, f"sharded step {s}"
    assert torch.equal(q_l, shard.take_q(q_ref)), "rotated q"
    assert np.array_equal(pool.lengths(0), full_pool.lengths(0))
kf, vf = full_pool.gather(0, n_seqs=n)
kl, vl = pool.gather(0, n_seqs=n)
assert torch.equal(kl, shard.take_kv(kf)) and torch.equal(vl, shard.take_kv(vf)), "stored pages of the local heads"
# back-to-back steps that start early, every rank's merge kernel waiting for the others inside the next step
q_run = q_all.clone()
ref_out = torch.empty_like(q_all)
views = []
dist.barrier(); torch.cuda.synchronize()
for s in range(steps):
    views.append(pool.decode_step(0, shard.take_q(q_run[s]), shard.take_kv(kn_all[s]), shard.take_kv(vn_all[s]),
                                  exchange=gather, consecutive=True))
q_rot = None
for s in range(steps):
    q_rot = q_all[s].clone()
    full_pool.decode_step(0, q_rot, kn_all[s], vn_all[s], out=ref_out[s])
torch.cuda.synchronize()
for s in (steps - 2, steps - 1):
    got = views[s].movedim(0, 1).reshape(n, Hq, D)
    assert parity_errors(got, to_np(ref_out[s]))[0] <= TOL_BF16, f"early-start sharded step {s}"
assert torch.equal(shard.take_q(q_run[steps - 1]), shard.take_q(q_rot)), "rotated q of the early-start steps"
# the last step against the oracle on the logical history of two sequences
kf, vf = full_pool.gather(0, n_seqs=n)
final = [t + 2 * steps for t in lens]
got = views[steps - 1].movedim(0, 1).reshape(n, Hq, D)
for i in (1, 3):
    o = oattn.chunked_grouped_attention(to_np(q_rot[i])[None, :, None, :], to_np(kf[i:i + 1, :, :final[i]]), to_np(vf[i:i + 1, :, :final[i]]),
                                        query_positions=np.array([final[i] - 1], dtype=np.int32))
    assert_parity(got[i], o[0, :, 0, :], TOL_BF16, f"sharded step vs oracle, sequence {i}")
assert pool.check_device_status() == 0 and full_pool.check_device_status() == 0
gather.close()

# ---- sequence sharding ----------------------------------------------------------------------------------------------
sh = L.InterleavedShard(rank, world, 32, P)
cap = max(lens) + steps
gh = torch.Generator().manual_seed(6)
k_hist = [torch.randn((Hkv, cap, D), generator=gh).to(torch.bfloat16) for _ in lens]
v_hist = [torch.randn((Hkv, cap, D), generator=gh).to(torch.bfloat16) for _ in lens]
def seq_pool(positions_of):
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=Hkv, head_dim=D, num_pages=n * pps, max_seqs=n,
                                       max_pages_per_seq=pps, page_size=P, dtype=torch.bfloat16, device=rank, rope_theta=THETA))
    for s in range(n):
        assert pool.alloc_sequence() == s
        idx = positions_of(s)
        if idx:
            pool.append(0, k_hist[s][None, :, idx].to(dev), v_hist[s][None, :, idx].to(dev), seq_ids=[s], start_pos=[0])
    return pool
whole = seq_pool(lambda s: list(range(lens[s])))
local = seq_pool(lambda s: sh.global_positions(lens[s]))
merge = L.PeerSeqMerge(rank, world, n, Hq, D, torch.bfloat16, dev)
g2 = torch.Generator().manual_seed(8)
q2 = torch.randn((steps, n, Hq, D), generator=g2).to(torch.bfloat16).to(dev)
for s in range(steps):
    cur = [t + s for t in lens]
    q_ref, q_l = q2[s].clone(), q2[s].clone()
    ref = whole.decode_step(0, q_ref, kn_all[s], vn_all[s])
    out = local.decode_step(0, q_l, kn_all[s], vn_all[s], exchange=merge, positions=cur, store=[sh.owner(p) == rank for p in cur])
    torch.cuda.synchronize()
    assert torch.equal(q_l, q_ref) and parity_errors(out, to_np(ref))[0] <= TOL_BF16, f"sequence-sharded step {s}"
    assert list(local.lengths(0)) == [sh.local_count(t + 1) for t in cur]
    both = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(both, out.contiguous())
    assert all(torch.equal(b, both[0]) for b in both), "every rank holds the same merged rows"
assert local.check_device_status() == 0
merge.close()
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.timeout(420)
def test_two_gpu_head_and_sequence_sharding():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        script = os.path.join(tmp, "worker.py")
        with open(script, "w") as f:
            f.write(WORKER)
        env = dict(os.environ, SKV_ROOT=ROOT)
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                            "--master-addr", "127.0.0.1", "--master-port", "29577", script],
                           env=env, capture_output=True, text=True, timeout=400)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
