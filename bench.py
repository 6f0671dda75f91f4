#!/usr/bin/env python
"""Paged grouped-query decode benchmark (the Llama-3-8B attention-layer workload).

Workload "paged_decode_llama3_8b_layer": 32 query heads, 8 KV heads, head_dim 128, bf16, page size 16,
64 sequences with context lengths uniform in [512, 8192], the page table a random permutation of a
shared pool, K/V ~ N(0,1).  One step = append one token per sequence with RoPE (theta 500000) on write,
then attend over the whole paged history: one library call, two launches.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --workload prefill [--kv paged] | decoder | longctx | glue      (secondary workloads, 1 GPU)

Prints one JSON line.  `value` is decode tokens/s with inputs resident in HBM; `e2e` is the same step
driven from pinned host buffers through the public API with the output read back every step;
`roofline` relates the step call's algorithmic HBM bytes to the measured copy bandwidth;
`cpu_baseline` times the NumPy restatement of the reference path on the host.  With N > 1 the KV heads
(and their query heads) are sharded over the ranks and the output slices are gathered by peer stores from the
merge kernel (`--gather nccl`: by an NCCL all-gather).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HQ, HKV, D, P, THETA = 32, 8, 128, 16, 500000.0
N_SEQS, CTX_LO, CTX_HI = 64, 512, 8192
SEED = 1234
WORKLOAD = "paged_decode_llama3_8b_layer"


def workload_lengths():
    return np.random.default_rng(SEED).integers(CTX_LO, CTX_HI + 1, size=N_SEQS).astype(np.int64)


def algorithmic_bytes(lens_after_append, hq, hkv):
    """HBM bytes one attention call must move: K and V of every attended token once, q in, out out,
    and one page-table entry per page touched."""
    kv = int(np.sum(lens_after_append)) * hkv * D * 2 * 2
    qo = 2 * len(lens_after_append) * hq * D * 2
    pt = int(np.sum(-(-lens_after_append // P))) * 4
    return kv + qo + pt


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import lokahi_b200 as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from lokahi_b200.sharding import HeadShard
    shard = HeadShard(rank, world, HQ, HKV)          # raises when the KV heads do not divide over the ranks
    hkv, hq = shard.local_kv_heads, shard.local_q_heads
    if args.emulate_shard > 1 and world == 1:      # one GPU doing the per-GPU share of an N-way head sharding (tuning aid)
        hkv, hq = HKV // args.emulate_shard, HQ // args.emulate_shard

    K, W = args.steps, args.warmup
    total_steps = W + K
    lens0 = workload_lengths()
    rng = np.random.default_rng(SEED + 1)
    cap = lens0 + 3 * total_steps + 2 * P                   # room for the timed leg, the instrumented pass and the e2e leg
    pages_per_seq = int(-(-cap.max() // P))
    pages_each = (-(-cap // P)).astype(np.int64)
    n_pages = int(pages_each.sum()) + 16
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=hkv, head_dim=D, num_pages=n_pages, max_seqs=N_SEQS,
                                       max_pages_per_seq=pages_per_seq, page_size=P, dtype=torch.bfloat16,
                                       device=local_rank, rope_theta=THETA))
    perm = rng.permutation(n_pages)                        # page table = random permutation of the shared pool
    at = 0
    for s in range(N_SEQS):
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, perm[at:at + pages_each[s]].tolist(), int(lens0[s]))
        at += int(pages_each[s])
    kp, vp = pool.layer_views(0)
    gen = torch.Generator(device=dev).manual_seed(SEED + 17 * rank)
    kp.normal_(generator=gen)
    vp.normal_(generator=gen)

    # per-step inputs, resident in HBM (device leg) and in pinned host memory (e2e leg)
    q_all = torch.randn((total_steps, N_SEQS, hq, D), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    k_all = torch.randn((total_steps, N_SEQS, hkv, D), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    v_all = torch.randn((total_steps, N_SEQS, hkv, D), generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    out_buf = torch.empty((N_SEQS, hq, D), device=dev, dtype=torch.bfloat16)
    gathered = torch.empty((world, N_SEQS, hq, D), device=dev, dtype=torch.bfloat16) if world > 1 else None
    fused_gather = world > 1 and args.gather == "fused"
    peer = None
    if fused_gather:
        # peer-mapped buffers need torch symmetric memory on every rank; if any rank cannot set them up,
        # all ranks fall back to the NCCL all-gather together
        try:
            peer = L.PeerGather(shard, N_SEQS, D, torch.bfloat16, dev)
            ok_local = 1
        except Exception as exc:   # noqa: BLE001 - any failure means "no peer mapping here"
            sys.stderr.write(f"[bench] rank {rank}: fused gather unavailable ({exc}); using NCCL all-gather\n")
            ok_local = 0
        flag = torch.tensor([ok_local], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            fused_gather, peer = False, None
    state = {"view": gathered}

    def step_call(q, k, v):
        """The library call of one decode step: RoPE of q and of the new K row, the append and the attention in the
        split-K kernel, then the merge kernel (under sharding with the fused gather: its peer stores and the wait)."""
        if fused_gather:
            state["view"] = pool.decode_step_gather(0, q, k, v, peer)
        else:
            pool.decode_step(0, q, k, v, out=out_buf)

    def step(q, k, v):
        step_call(q, k, v)
        if world > 1 and not fused_gather:
            dist.all_gather_into_tensor(gathered, out_buf)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident leg ---------------------------------------------------------------------------
    for i in range(W):
        step(q_all[i], k_all[i], v_all[i])
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    launches0 = L._lib.lib.skv_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for i in range(K):
        j = W + i
        step(q_all[j], k_all[j], v_all[j])
    ev1.record()
    barrier()
    launches = L._lib.lib.skv_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms_total = ev0.elapsed_time(ev1)
    # instrumented pass (not part of `value`): the same steps with CUDA events around the library call only
    # (split-K kernel + merge kernel, under sharding with the fused gather and its wait), for the roofline
    K2 = min(K, 32)
    attn_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K2)]
    barrier()                                             # rank 0 spent time stopping the clock sampler
    l_inst0 = L._lib.lib.skv_launch_count()
    for i in range(K2):
        j = W + i
        attn_ev[i][0].record()
        step_call(q_all[j], k_all[j], v_all[j])
        attn_ev[i][1].record()
        if world > 1 and not fused_gather:
            dist.all_gather_into_tensor(gathered, out_buf)
    launches_per_call = (L._lib.lib.skv_launch_count() - l_inst0) // K2
    barrier()
    attn_ms = np.array([a.elapsed_time(b) for a, b in attn_ev])
    if K2 > 4:
        attn_ms = attn_ms[2:]                             # the first launches after a barrier absorb rank skew
    if pool.check_device_status() != 0:
        raise SystemExit("device status flag set during the timed region")
    lens_timed = lens0[None, :] + W + K + 1 + np.arange(K2)[:, None]      # attended tokens per instrumented step
    algo_bytes = float(np.mean([algorithmic_bytes(lens_timed[i], hq, hkv) for i in range(K2 - len(attn_ms), K2)]))

    # ---- end-to-end leg: pinned host inputs, output read back every step ----------------------------------
    Ke = K
    nq, nk = N_SEQS * hq * D, N_SEQS * hkv * D
    # one pinned staging buffer per step, [q | k | v], so that a step costs one host->device copy
    qkv_h = torch.cat([q_all[:Ke].reshape(Ke, nq), k_all[:Ke].reshape(Ke, nk), v_all[:Ke].reshape(Ke, nk)], dim=1).cpu().pin_memory()
    qkv_d = torch.empty((nq + 2 * nk,), device=dev, dtype=torch.bfloat16)
    q_d = qkv_d[:nq].view(N_SEQS, hq, D)
    k_d = qkv_d[nq:nq + nk].view(N_SEQS, hkv, D)
    v_d = qkv_d[nq + nk:].view(N_SEQS, hkv, D)
    out_h = torch.empty((world if world > 1 else 1, N_SEQS, hq, D), dtype=torch.bfloat16).pin_memory()

    def e2e_step(i):
        qkv_d.copy_(qkv_h[i], non_blocking=True)
        step(q_d, k_d, v_d)
        out_h.copy_((state["view"] if world > 1 else out_buf).view(out_h.shape), non_blocking=True)
        torch.cuda.current_stream().synchronize()          # a decode loop consumes the result before the next step

    for i in range(min(W, Ke)):
        e2e_step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(Ke):
        e2e_step(i)
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1)
    if pool.check_device_status() != 0:
        raise SystemExit("device status flag set during the end-to-end leg")

    # ---- max over ranks --------------------------------------------------------------------------------------
    stats = torch.tensor([ms_total, ms_e2e, float(attn_ms.mean())], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e, attn_mean_ms = [float(x) for x in stats.tolist()]

    result = None
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        achieved = algo_bytes / (attn_mean_ms * 1e-3) / 1e9
        tokens = N_SEQS * K
        result = {
            "metric": "paged GQA decode tokens/s", "value": tokens / (ms_total * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "n_seqs": N_SEQS, "context": [CTX_LO, CTX_HI], "q_heads": HQ, "kv_heads": HKV,
                       "head_dim": D, "page_size": P, "rope_theta": THETA, "layers": 1,
                       "parallelism": (f"kv_head_shard{world}, output gather " + ("fused into the merge kernel (peer stores)" if fused_gather else "NCCL all-gather")) if world > 1 else "single",
                       "l2": "inputs larger than L2 (KV working set per step >= 1 GB / n_gpus)"},
            "e2e": {"value": N_SEQS * Ke / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e / Ke,
                    "h2d_bytes_per_step": int(q_d.numel() + k_d.numel() + v_d.numel()) * 2,
                    "d2h_bytes_per_step": int(out_h.numel()) * 2},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / 8000.0,
                         "kernel": ("decode step call: split-K kernel with RoPE and the append folded in + merge kernel"
                                    if launches_per_call == 2 + (1 if fused_gather else 0) else
                                    "decode step call: append kernel + split-K kernel + merge kernel")
                                   + (" + gather wait" if fused_gather else ""),
                         "algorithmic_bytes_per_launch": algo_bytes, "launch_ms": attn_mean_ms,
                         "launch_ms_min": float(attn_ms.min()), "launch_ms_median": float(np.median(attn_ms)),
                         "launch_ms_p95": float(np.percentile(attn_ms, 95)), "traffic": algo_bytes * TRAFFIC_RATIO},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline_sample(pool, kp, vp, lens0 + W + K + K2 + min(W, Ke) + Ke, hq, hkv)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def run_prefill(args):
    """Secondary workload "chunked_gqa_prefill_4096": the stand-alone chunked causal GQA op, bf16, batch 1,
    32 query heads, 8 KV heads, head_dim 128, sequence 4096, absolute positions 0..4095 (tensor-core bound).
    One step = one attention call; L2 (126 MB) is flushed between timed calls because q, k, v and out
    together are 84 MB."""
    import torch

    import lokahi_b200 as L
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, S = 1, 4096
    gen = torch.Generator(device=dev).manual_seed(SEED)
    q = torch.randn((B, HQ, S, D), generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn((B, HKV, S, D), generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn((B, HKV, S, D), generator=gen, device=dev).to(torch.bfloat16)
    pos = torch.arange(S, dtype=torch.int32, device=dev)      # positions are an input: resident in HBM like q, k, v
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    K, W = args.steps, args.warmup
    if args.kv == "paged":
        # the same K/V held in a pool of 16-token pages dealt out in a random order: the kernel reads the pages
        n_pages = S // P
        pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=HKV, head_dim=D, num_pages=n_pages + 8, max_seqs=1,
                                           max_pages_per_seq=n_pages, page_size=P, dtype=torch.bfloat16, device=0))
        assert pool.alloc_sequence() == 0
        perm = np.random.default_rng(SEED).permutation(n_pages + 8)[:n_pages]
        pool.set_page_table(0, perm.tolist(), S)
        kp, vp = pool.layer_views(0)
        idx = torch.as_tensor(perm, device=dev, dtype=torch.long)
        kp[idx] = k[0].view(HKV, n_pages, P, D).transpose(0, 1)
        vp[idx] = v[0].view(HKV, n_pages, P, D).transpose(0, 1)
        pos2 = pos.view(1, S)

        def call():
            return pool.prefill_attention(0, q, positions=pos2)
    else:
        def call():
            return L.chunked_grouped_attention(q, k, v, query_positions=pos, causal=True, q_block_size=512, k_block_size=512)
    for _ in range(W):
        call()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    time.sleep(0.3)
    l0 = L._lib.lib.skv_launch_count()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    for a, b in evs:
        flush.zero_()
        a.record()
        call()
        b.record()
    torch.cuda.synchronize()
    launches = L._lib.lib.skv_launch_count() - l0
    clocks = sampler.stop()
    ms = np.array([a.elapsed_time(b) for a, b in evs])
    # end to end: pinned host q, k, v in, out back, every step
    qh, kh, vh = q.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory()
    pos_h = np.arange(S, dtype=np.int32)                      # host positions, copied by the call
    oh = torch.empty_like(qh).pin_memory()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    Ke = max(3, min(K, 20))
    torch.cuda.synchronize()
    e0.record()
    for _ in range(Ke):
        q.copy_(qh, non_blocking=True); k.copy_(kh, non_blocking=True); v.copy_(vh, non_blocking=True)
        o = L.chunked_grouped_attention(q, k, v, query_positions=pos_h, causal=True, q_block_size=512, k_block_size=512)
        oh.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / Ke
    flops = 4.0 * HQ * D * (S * (S + 1) / 2)            # causal-useful flops (dense-equivalent is 2x)
    peak = 1590.0
    kind = "fallback"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak, kind = float(json.load(f)["bf16_tflops"]), "measured"
    achieved = flops / (ms.mean() * 1e-3) / 1e12
    return {
        "metric": "chunked causal GQA prefill tokens/s", "value": B * S / (ms.mean() * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": K, "warmup": W, "ms_per_step": float(ms.mean()), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "chunked_gqa_prefill_4096", "batch": B, "q_heads": HQ, "kv_heads": HKV, "head_dim": D,
                   "seq_len": S, "q_chunk": 512, "k_chunk": 512, "kv": args.kv, "l2": "flushed between timed calls (256 MB write)"},
        "e2e": {"value": B * S / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": int(q.numel() + k.numel() + v.numel()) * 2, "d2h_bytes_per_step": int(q.numel()) * 2},
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "peak_kind": f"of {kind} (burst)", "flops_per_launch": flops, "flops_counted": "causal-useful 4*Hq*D*S(S+1)/2",
                     "launch_ms": float(ms.mean()), "launch_ms_min": float(ms.min()), "launch_ms_median": float(np.median(ms)),
                     "launch_ms_p95": float(np.percentile(ms, 95)), "traffic": None},
        "clocks": clocks,
    }


def run_decoder(args):
    """Secondary workload "deepseek_1p3b_shaped_decoder": random-init decoder, 24 layers, hidden 2048, 16 MHA heads
    of 128, SiLU MLP 5504, vocab 32256, RoPE theta 100000 with linear scaling 4, bf16; batch 8, 2048-token prompt
    prefill then 256 greedy decode tokens with the KV cache held in pages.  The linear layers are torch/cuBLAS
    and are reported separately from the hot path (RoPE + cache update + attention)."""
    import torch
    from types import SimpleNamespace

    import lokahi_b200 as L
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    Bt, Lp, Ld = 8, 2048, max(1, min(args.steps, 256))
    cfg = SimpleNamespace(vocab_size=32256, hidden_size=2048, intermediate_size=5504, num_hidden_layers=24,
                          num_attention_heads=16, num_key_value_heads=16, rms_norm_eps=1e-6, max_position_embeddings=4096,
                          rope_theta=100000.0, rope_scaling_factor=4.0)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    H, I, Dh = cfg.hidden_size, cfg.intermediate_size, 128

    def mat(*shape):
        return (torch.randn(shape, generator=gen, device=dev) * 0.02).to(torch.bfloat16)

    w = {}
    for i in range(cfg.num_hidden_layers):
        b = f"model.layers.{i}"
        for n, shp in (("self_attn.q_proj", (H, H)), ("self_attn.k_proj", (H, H)), ("self_attn.v_proj", (H, H)),
                       ("self_attn.o_proj", (H, H)), ("mlp.gate_proj", (I, H)), ("mlp.up_proj", (I, H)), ("mlp.down_proj", (H, I))):
            w[f"{b}.{n}.weight"] = mat(*shp)
        w[f"{b}.input_layernorm.weight"] = torch.ones(H, device=dev, dtype=torch.bfloat16)
        w[f"{b}.post_attention_layernorm.weight"] = torch.ones(H, device=dev, dtype=torch.bfloat16)
    w["model.embed_tokens.weight"] = mat(cfg.vocab_size, H)
    w["lm_head.weight"] = mat(cfg.vocab_size, H)
    w["model.norm.weight"] = torch.ones(H, device=dev, dtype=torch.bfloat16)
    model = L.PagedDecoder(cfg, w)
    prompt = torch.randint(0, cfg.vocab_size, (Bt, Lp), generator=gen, device=dev)

    # The page pool is created once, ahead of the timed runs (allocating and zeroing its 3.8 GB would otherwise land
    # inside the first layer's hot-path interval); every run gets a fresh cache on it and frees its sequences.
    pages_per_seq = -(-(Lp + Ld + 16) // P)
    shared_pool = L.PagedPool(L.PagedKVConfig(num_layers=cfg.num_hidden_layers, num_kv_heads=16, head_dim=Dh,
                                              num_pages=Bt * pages_per_seq, max_seqs=Bt, max_pages_per_seq=pages_per_seq,
                                              page_size=P, dtype=torch.bfloat16, device=0))

    def one_run(timed):
        cache = L.PagedKVCache(cfg, cache_dir=None, pool=shared_pool)
        model.hot_path_events = [] if timed else None
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        logits = model(prompt, past_key_values=cache, use_cache=True)
        nxt = logits[:, -1, :].argmax(-1, keepdim=True)
        e[1].record()
        n_pre = len(model.hot_path_events) if timed else 0
        for _ in range(Ld):
            logits = model(nxt, past_key_values=cache, use_cache=True)
            nxt = logits[:, -1, :].argmax(-1, keepdim=True)
        e[2].record()
        torch.cuda.synchronize()
        hot = model.hot_path_events or []
        pre_hot = sum(a.elapsed_time(b) for a, b in hot[:n_pre])
        dec_hot = sum(a.elapsed_time(b) for a, b in hot[n_pre:])
        flag = cache.pool.check_device_status()
        cache.clear()
        return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]), pre_hot, dec_hot, flag

    one_run(False)                                   # warm-up (cuBLAS handles, page pool, autotuning)
    l0 = L._lib.lib.skv_launch_count()
    pre_ms, dec_ms, pre_hot, dec_hot, flag = one_run(True)
    launches = L._lib.lib.skv_launch_count() - l0
    if flag:
        raise SystemExit("device status flag set")
    peak_t = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"] if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1590.0
    peak_b, _ = measured_peak_gbs()
    layers = cfg.num_hidden_layers
    pre_flops = layers * Bt * 4.0 * 16 * Dh * (Lp * (Lp + 1) / 2)
    dec_bytes = sum(layers * Bt * (Lp + s + 1) * 16 * Dh * 2 * 2 for s in range(Ld))
    return {
        "metric": "decoder decode tokens/s", "value": Bt * Ld / (dec_ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": Ld,
        "warmup": 1, "ms_per_step": dec_ms / Ld, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "deepseek_1p3b_shaped_decoder", "batch": Bt, "prompt": Lp, "decode_tokens": Ld, "layers": layers,
                   "hidden": H, "heads": 16, "head_dim": Dh, "mlp": I, "vocab": cfg.vocab_size, "rope": "theta 1e5, linear x4"},
        "prefill": {"tokens_per_s": Bt * Lp / (pre_ms * 1e-3), "ms": pre_ms, "hot_path_ms": pre_hot,
                    "hot_path_tflops": pre_flops / (pre_hot * 1e-3) / 1e12, "hot_path_frac_of_bf16_peak": pre_flops / (pre_hot * 1e-3) / 1e12 / peak_t},
        "decode": {"tokens_per_s": Bt * Ld / (dec_ms * 1e-3), "ms": dec_ms, "hot_path_ms": dec_hot,
                   "hot_path_gbs": dec_bytes / (dec_hot * 1e-3) / 1e9, "hot_path_frac_of_hbm_peak": dec_bytes / (dec_hot * 1e-3) / 1e9 / peak_b},
        "gpu_launches": int(launches),
    }


def run_glue(args):
    """Secondary workload "decoder_glue": the RMSNorm (with the residual add fused) and SwiGLU launches at the
    shapes of configs[3]'s prefill (16384 rows, hidden 2048, MLP 5504), bf16: element-wise, HBM roofline.  The
    tensors (64 MB to 180 MB each) rotate through four sets so that consecutive calls do not hit L2."""
    import torch

    import lokahi_b200 as L
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    rows, hidden, inter, sets = 16384, 2048, 5504, 4
    gen = torch.Generator(device=dev).manual_seed(SEED)
    mk = lambda *shape: torch.randn(shape, generator=gen, device=dev).to(torch.bfloat16)
    xs, ds, gs, us = ([mk(rows, n) for _ in range(sets)] for n in (hidden, hidden, inter, inter))
    w = mk(hidden)
    K, W = args.steps, args.warmup
    peak, peak_kind = measured_peak_gbs()

    def timed(fn, bytes_per_call):
        for i in range(W):
            fn(i % sets)
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
        for i, (a, b) in enumerate(evs):
            a.record()
            fn(i % sets)
            b.record()
        torch.cuda.synchronize()
        ms = np.array([a.elapsed_time(b) for a, b in evs])
        gbs = bytes_per_call / (ms.mean() * 1e-3) / 1e9
        return {"launch_ms": float(ms.mean()), "launch_ms_min": float(ms.min()), "algorithmic_bytes": bytes_per_call,
                "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak, "peak_kind": f"of {peak_kind}"}

    l0 = L._lib.lib.skv_launch_count()
    norm = timed(lambda i: L.rms_norm(xs[i], w, 1e-6), 2 * rows * hidden * 2 + hidden * 2)
    add_norm = timed(lambda i: L.add_rms_norm(xs[i], ds[i], w, 1e-6), 4 * rows * hidden * 2 + hidden * 2)
    swi = timed(lambda i: L.swiglu(gs[i], us[i]), 3 * rows * inter * 2)
    launches = L._lib.lib.skv_launch_count() - l0
    return {
        "metric": "decoder glue GB/s (add + RMSNorm)", "value": add_norm["achieved_gbs"], "unit": "GB/s", "n_gpus": 1, "steps": K,
        "warmup": W, "ms_per_step": add_norm["launch_ms"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "decoder_glue", "rows": rows, "hidden": hidden, "mlp": inter,
                   "l2": "four tensor sets in rotation (each set larger than L2 together with its outputs)"},
        "rmsnorm": norm, "add_rmsnorm": add_norm, "swiglu": swi, "gpu_launches": int(launches),
    }


def run_longctx(args):
    """Secondary workload "long_context_llama3_8b_kv": one GPU's share of the 8-way KV-head sharding of a
    Llama-3-8B KV path: 32 layers, 1 KV head with its 4 query heads, head_dim 128, bf16, 4 sequences at 96k
    (98304) tokens of N(0,1) K/V.  Every step parks the oldest 25 % of each sequence's pages in pinned host
    memory, brings them back, then appends one token and attends in all 32 layers.  Two rooflines: HBM for the
    attention bytes, the host link for the parked bytes."""
    import torch

    import lokahi_b200 as L
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    layers, n_seq, hkv, hq, T0 = 32, 4, 1, 4, 98304
    K, W = max(1, min(args.steps, 64)), max(1, min(args.warmup, 3))
    pages_per_seq = -(-(T0 + K + W + 16) // P)
    park = (T0 // P) // 4
    pool = L.PagedPool(L.PagedKVConfig(num_layers=layers, num_kv_heads=hkv, head_dim=D, num_pages=n_seq * pages_per_seq + 8,
                                       max_seqs=n_seq, max_pages_per_seq=pages_per_seq, page_size=P, dtype=torch.bfloat16,
                                       device=0, host_pages=n_seq * park + 8, rope_theta=THETA))
    for s_ in range(n_seq):
        assert pool.alloc_sequence() == s_
        pool.reserve(s_, T0 + K + W + 16)
    gen = torch.Generator(device=dev).manual_seed(SEED)
    pool_set_lengths(pool, layers, n_seq, T0)        # declares the history (writes zeros) ...
    for layer in range(layers):                      # ... which is then filled with N(0,1) K/V in place
        kp, vp = pool.layer_views(layer)
        kp.normal_(generator=gen)
        vp.normal_(generator=gen)
    q = torch.randn((n_seq, hq, D), generator=gen, device=dev).to(torch.bfloat16)
    kn = torch.randn((n_seq, hkv, D), generator=gen, device=dev).to(torch.bfloat16)
    vn = torch.randn((n_seq, hkv, D), generator=gen, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    q_work = torch.empty_like(q)

    def step(timers=None):
        if timers:
            timers[0].record()
        for s_ in range(n_seq):
            pool.evict(s_, 0, park)
        for s_ in range(n_seq):
            pool.prefetch(s_, 0, park)
        pool.sync_transfers()
        if timers:
            timers[1].record()
        for layer in range(layers):
            q_work.copy_(q)                                  # the step rotates q in place
            pool.decode_step(layer, q_work, kn, vn, out=out)  # RoPE + append + attention: one library call
        if timers:
            timers[2].record()

    for _ in range(W):
        step()
    torch.cuda.synchronize()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(K)]
    l0 = L._lib.lib.skv_launch_count()
    c0 = pool.counters()
    for i in range(K):
        step(evs[i])
    torch.cuda.synchronize()
    launches = L._lib.lib.skv_launch_count() - l0
    c1 = pool.counters()
    if pool.check_device_status() != 0:
        raise SystemExit("device status flag set")
    xfer_ms = np.array([e[0].elapsed_time(e[1]) for e in evs])
    attn_ms = np.array([e[1].elapsed_time(e[2]) for e in evs])
    d2h = (c1["bytes_d2h"] - c0["bytes_d2h"]) / K
    h2d = (c1["bytes_h2d"] - c0["bytes_h2d"]) / K
    attn_bytes = float(np.mean([layers * n_seq * (T0 + W + i + 1) * hkv * D * 2 * 2 for i in range(K)]))
    peak, kind = measured_peak_gbs()
    step_ms = float((xfer_ms + attn_ms).mean())
    return {
        "metric": "long-context decode tokens/s per GPU (1 of 8 KV heads)", "value": n_seq / (step_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "long_context_llama3_8b_kv", "layers": layers, "sequences": n_seq, "context": T0, "kv_heads_local": hkv,
                   "q_heads_local": hq, "head_dim": D, "page_size": P, "parked_fraction": 0.25},
        "attention": {"ms_per_step": float(attn_ms.mean()), "algorithmic_bytes": attn_bytes,
                      "achieved_gbs": attn_bytes / (attn_ms.mean() * 1e-3) / 1e9,
                      "frac_of_hbm_peak": attn_bytes / (attn_ms.mean() * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}"},
        "transfers": {"ms_per_step": float(xfer_ms.mean()), "d2h_bytes_per_step": d2h, "h2d_bytes_per_step": h2d,
                      "achieved_gbs_each_way": (d2h + h2d) / 2 / (xfer_ms.mean() * 1e-3 / 2) / 1e9,
                      "note": "evict then prefetch of the same pages, serial on one copy stream; host-link bound"},
        "gpu_launches": int(launches),
    }


def pool_set_lengths(pool, layers, n_seq, length):
    """Give every layer a history of `length` tokens by appending zero rows in blocks (bench set-up only;
    the caller overwrites the pages afterwards)."""
    import torch
    zero = torch.zeros((n_seq, pool.cfg.num_kv_heads, 1, pool.cfg.head_dim), device=pool.torch_device, dtype=pool.cfg.dtype)
    for layer in range(layers):
        done = 0
        while done < length:
            n = min(8192, length - done)
            kv = zero.expand(n_seq, pool.cfg.num_kv_heads, n, pool.cfg.head_dim)   # stride 0 along tokens
            pool.append(layer, kv, kv, start_pos=[done] * n_seq)
            done += n


# ncu dram__bytes_read.sum + dram__bytes_write.sum per decode launch: measured on the 16-sequence capture
# case (293.13 MB of traffic for 287.07 MB algorithmic, profiles/decode_tma_kernel_paged_decode_16seq.md)
# and scaled to this workload by the algorithmic bytes, which is what the traffic grows with.
TRAFFIC_RATIO = 293.13 / 287.07


# ------------------------------------------------------------------------------------------------------
# CPU legs (the only code here that runs the oracle)
# ------------------------------------------------------------------------------------------------------
def _oracle_step(q, k_new, v_new, k_hist, v_hist, length):
    """One sequence, one step of the reference path on the CPU: RoPE on the new q/k, append, attend."""
    from oracle import attention as oattn
    from oracle import paged as opaged
    pos = np.array([length])
    qr = opaged.rope_rows(q[None], pos, THETA)[0]
    kr = opaged.rope_rows(k_new[None], pos, THETA)[0]
    k_hist[:, length] = kr
    v_hist[:, length] = v_new
    T = length + 1
    return oattn.chunked_grouped_attention(qr[None, :, None, :], k_hist[None, :, :T], v_hist[None, :, :T],
                                           query_positions=np.array([[length]], dtype=np.int32), causal=True,
                                           q_block_size=32768, k_block_size=1000000)


def cpu_baseline_sample(pool, kp, vp, lens_now, hq, hkv, budget_s=12.0):
    """Scalar (one core) timing of the oracle on a bounded sample of the same workload."""
    import torch
    rng = np.random.default_rng(SEED + 5)
    order = rng.permutation(N_SEQS)
    done, t_used, steps_per_seq = 0, 0.0, 2
    for s in order:
        T = int(lens_now[s])
        n = -(-(T + steps_per_seq) // P)
        pages = torch.from_numpy(pool.page_table(int(s))[:n].astype(np.int64)).to(kp.device)
        kh = kp[pages].float().permute(1, 0, 2, 3).reshape(hkv, n * P, D).cpu().numpy().copy()
        vh = vp[pages].float().permute(1, 0, 2, 3).reshape(hkv, n * P, D).cpu().numpy().copy()
        for j in range(steps_per_seq):
            q = rng.standard_normal((hq, D), dtype=np.float32)
            k = rng.standard_normal((hkv, D), dtype=np.float32)
            v = rng.standard_normal((hkv, D), dtype=np.float32)
            t0 = time.perf_counter()
            _oracle_step(q, k, v, kh, vh, T + j)
            t_used += time.perf_counter() - t0
            done += 1
        if t_used > budget_s:
            break
    return {"value": done / t_used, "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": f"{done} (sequence, step) pairs of the same workload ({done // steps_per_seq} sequences x "
                      f"{steps_per_seq} steps), NumPy restatement of the reference path, one thread"}


def _ref_worker(conn, seq_ids, lens, seed):
    rng = np.random.default_rng(seed)
    hist = {}
    for s in seq_ids:
        cap = int(lens[s]) + 4096
        hist[s] = [rng.standard_normal((HKV, cap, D), dtype=np.float32), rng.standard_normal((HKV, cap, D), dtype=np.float32),
                   int(lens[s])]
    conn.send("ready")
    while True:
        msg = conn.recv()
        if msg is None:
            break
        step_seed = msg
        r = np.random.default_rng(step_seed)
        for s in seq_ids:
            kh, vh, T = hist[s]
            q = r.standard_normal((HQ, D), dtype=np.float32)
            k = r.standard_normal((HKV, D), dtype=np.float32)
            v = r.standard_normal((HKV, D), dtype=np.float32)
            _oracle_step(q, k, v, kh, vh, T)
            hist[s][2] = T + 1
        conn.send(len(seq_ids))


def run_reference(args):
    """The reference's CPU path (NumPy restatement) on all host cores: one process per core, each owning a
    fixed share of the sequences.  A step is the full workload step (64 sequences, one token each)."""
    import multiprocessing as mp
    if int(os.environ.get("RANK", "0")) != 0:
        return None
    cores = max(1, min(os.cpu_count() or 1, N_SEQS))
    lens0 = workload_lengths()
    ctx = mp.get_context("fork")
    workers = []
    for w in range(cores):
        parent, child = ctx.Pipe()
        p = ctx.Process(target=_ref_worker, args=(child, list(range(w, N_SEQS, cores)), lens0, SEED + 100 + w), daemon=True)
        p.start()
        workers.append((p, parent))
    for _, c in workers:
        assert c.recv() == "ready"

    def one_step(i):
        for _, c in workers:
            c.send(SEED + 1000 + i)
        return sum(c.recv() for _, c in workers)

    # bounded: at most ~3 minutes in total whatever K and W are
    t_probe = time.perf_counter()
    one_step(-1)
    per_step = time.perf_counter() - t_probe
    K = max(1, min(args.steps, int(150.0 / max(per_step, 1e-3))))
    W = max(0, min(args.warmup, int(20.0 / max(per_step, 1e-3))))
    for i in range(W):
        one_step(i)
    t0 = time.perf_counter()
    tokens = 0
    for i in range(K):
        tokens += one_step(W + i)
    dt = time.perf_counter() - t0
    for p, c in workers:
        c.send(None)
        p.join(timeout=5)
    value = tokens / dt
    return {
        "impl": "reference", "metric": "paged GQA decode tokens/s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": K, "warmup": W, "ms_per_step": dt / K * 1e3, "higher_is_better": True,
        # same workload at every N (the CPU arm does not shard): the label follows the GPU arm's
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "n_seqs": N_SEQS, "context": [CTX_LO, CTX_HI], "q_heads": HQ, "kv_heads": HKV,
                   "head_dim": D, "page_size": P, "rope_theta": THETA, "layers": 1},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"full workload step (64 sequences x 1 token) x {K} steps; NumPy restatement of the "
                                   f"reference path, one process per core (requested steps {args.steps})"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def main():
    global N_SEQS
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps; default by workload: decode 128, prefill 30, decoder 256, longctx 64 (the configurations' own counts)")
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--gather", choices=["fused", "nccl"], default="fused",
                    help="N > 1: how the per-rank attention outputs are gathered")
    ap.add_argument("--emulate-shard", type=int, default=1, help=argparse.SUPPRESS)
    ap.add_argument("--workload", choices=["decode", "prefill", "decoder", "longctx", "glue"], default="decode",
                    help="decode: the headline paged-decode workload; prefill: the 4096-token chunked-GQA op (1 GPU)")
    ap.add_argument("--kv", choices=["dense", "paged"], default="dense",
                    help="prefill workload: K/V as dense tensors or as scattered 16-token pages of a pool")
    ap.add_argument("--seqs", type=int, default=N_SEQS,
                    help="number of sequences (default: the workload's 64; smaller values are for profiler captures)")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"decode": 128, "prefill": 30, "decoder": 256, "longctx": 64, "glue": 30}[args.workload]
    N_SEQS = args.seqs
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        result = run_reference(args)
    elif args.workload == "prefill":
        result = run_prefill(args)
    elif args.workload == "decoder":
        result = run_decoder(args)
    elif args.workload == "longctx":
        result = run_longctx(args)
    elif args.workload == "glue":
        result = run_glue(args)
    else:
        result = run_ours(args)
    if result is not None:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
