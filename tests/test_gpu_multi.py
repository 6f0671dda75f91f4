"""Two-GPU checks (skipped on a one-GPU box): KV-head sharding with the NCCL all-gather and with the gather
fused into the merge kernel must both reproduce the unsharded decode output bit for bit."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["SKV_ROOT"])
import lokahi_b200 as L
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
os.environ["NCCL_NVLS_ENABLE"] = "0"
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
Hq, Hkv, D, P = 32, 8, 128, 16
lens = [3, 100, 1000, 2500]
n = len(lens)
pps = -(-(max(lens) + 8) // P)
g = torch.Generator().manual_seed(5)
k_full = torch.randn((n * pps, Hkv, P, D), generator=g).to(torch.bfloat16)
v_full = torch.randn((n * pps, Hkv, P, D), generator=g).to(torch.bfloat16)
q_full = torch.randn((n, Hq, D), generator=g).to(torch.bfloat16)
perm = torch.randperm(n * pps, generator=g).tolist()

def make_pool(kv_heads, k, v):
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=kv_heads, head_dim=D, num_pages=n * pps, max_seqs=n,
                                       max_pages_per_seq=pps, page_size=P, dtype=torch.bfloat16, device=rank))
    for s in range(n):
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, perm[s * pps:(s + 1) * pps], lens[s])
    kp, vp = pool.layer_views(0)
    kp.copy_(k.to(dev)); vp.copy_(v.to(dev))
    return pool

full = make_pool(Hkv, k_full, v_full).decode_attention(0, q_full.to(dev))          # unsharded reference on this GPU
shard = L.HeadShard(rank, world, Hq, Hkv)
pool = make_pool(shard.local_kv_heads, shard.take_kv(k_full).contiguous(), shard.take_kv(v_full).contiguous())
q_loc = shard.take_q(q_full).contiguous().to(dev)
out_nccl = L.gather_head_outputs(pool.decode_attention(0, q_loc), shard)
assert torch.equal(out_nccl, full), "NCCL gather"
gather = L.PeerGather(shard, n, D, torch.bfloat16, dev)
for it in range(4):
    view = pool.decode_attention_gather(0, q_loc, gather)                             # [world, n, Hq/world, D]
    torch.cuda.synchronize()
    fused = view.movedim(0, 1).reshape(n, Hq, D)
    assert torch.equal(fused, full), f"fused gather, epoch {it + 1}"
assert pool.check_device_status() == 0
dist.barrier()
dist.destroy_process_group()
print(f"rank {rank} ok")
'''


@pytest.mark.timeout(300)
def test_two_gpu_head_sharding_nccl_and_fused_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, SKV_ROOT=ROOT)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29577", str(script)],
                       env=env, capture_output=True, text=True, timeout=280)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "rank 0 ok" in r.stdout and "rank 1 ok" in r.stdout
