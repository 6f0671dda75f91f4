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

def e2e_block(world):
    """End-to-end leg: steps travel in blocks of this many (every step has its own upload and read-back; an event sits
    between two steps on the compute stream only at block boundaries).  Short steps gain from it (8 GPUs: 0.055 ->
    0.041 ms per step), longer ones lose the pipeline's fill and drain (4 GPUs: 0.062 -> 0.065 ms, 1 GPU: 0.198 -> 0.204)."""
    return 4 if world >= 8 else 1
TOL_E2E = 2e-2      # end-to-end result against the device-resident step (bf16; the two are expected to agree to the bit)

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
SEQ_BLOCK = 64            # tokens per round-robin block of the sequence sharding (four pages)


def base_config(n_gpus, parallelism):
    """The `config` object both arms print (same keys, same values for the same workload)."""
    return {"workload": WORKLOAD, "n_seqs": N_SEQS, "context": [CTX_LO, CTX_HI], "q_heads": HQ, "kv_heads": HKV,
            "head_dim": D, "page_size": P, "rope_theta": THETA, "layers": 1, "parallelism": parallelism,
            "l2": "inputs larger than L2 (KV working set per step >= 1 GB / n_gpus)"}


def parallelism_label(world, shard, gather):
    if world == 1:
        return "single"
    if shard == "seq":
        return f"sequence_shard{world} (round-robin blocks of {SEQ_BLOCK} tokens), cross-rank merge fused into the merge kernel (peer stores)"
    return f"kv_head_shard{world}, output gather " + ("fused into the merge kernel (peer stores)" if gather == "fused" else "NCCL all-gather")


def rank_geometry(r, world, shard_kind):
    """(kv heads, q heads, per-sequence stored lengths) of rank r."""
    from lokahi_b200.sharding import InterleavedShard
    lens0 = workload_lengths()
    if shard_kind == "seq" and world > 1:
        sh = InterleavedShard(r, world, SEQ_BLOCK, P)
        return HKV, HQ, np.array([sh.local_count(int(t)) for t in lens0], dtype=np.int64), sh
    return HKV // world, HQ // world, lens0, None


def rank_tables(r, world, shard_kind, total_steps):
    """Page-table geometry of rank r's pool: the same on whichever rank computes it."""
    hkv, hq, lens_local, sh = rank_geometry(r, world, shard_kind)
    cap = lens_local + total_steps + 2 * P
    pages_each = (-(-cap // P)).astype(np.int64)
    n_pages = int(pages_each.sum()) + 16
    perm = np.random.default_rng(SEED + 1 + 101 * r).permutation(n_pages)   # page table = random permutation of the pool
    starts = np.concatenate([[0], np.cumsum(pages_each)])
    return hkv, hq, lens_local, sh, int(pages_each.max()), n_pages, [perm[starts[s]:starts[s + 1]] for s in range(N_SEQS)]


def rank_data(r, world, shard_kind, total_steps, dev):
    """K/V pool contents and per-step inputs of rank r, from a generator seeded by r alone, so that rank 0 can
    rebuild every rank's data for the parity check."""
    import torch
    hkv, hq, _, _, _, n_pages, _ = rank_tables(r, world, shard_kind, total_steps)
    gen = torch.Generator(device=dev).manual_seed(SEED + 17 * r)
    kp = torch.empty((n_pages, hkv, P, D), device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    vp = torch.empty((n_pages, hkv, P, D), device=dev, dtype=torch.bfloat16).normal_(generator=gen)
    # under sequence sharding every rank sees the same q, k, v rows (all heads): seeded alike
    gen_in = torch.Generator(device=dev).manual_seed(SEED + 5 + (0 if shard_kind == "seq" else 17 * r))
    mk = lambda h: torch.randn((total_steps, N_SEQS, h, D), generator=gen_in, device=dev, dtype=torch.float32).to(torch.bfloat16)
    return kp, vp, mk(hq), mk(hkv), mk(hkv)


def build_pool(L, torch, r, world, shard_kind, total_steps, dev, local_rank):
    hkv, hq, lens_local, sh, pages_per_seq, n_pages, tables = rank_tables(r, world, shard_kind, total_steps)
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=hkv, head_dim=D, num_pages=n_pages, max_seqs=N_SEQS,
                                       max_pages_per_seq=pages_per_seq, page_size=P, dtype=torch.bfloat16,
                                       device=local_rank, rope_theta=THETA))
    for s in range(N_SEQS):
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, tables[s].tolist(), int(lens_local[s]))
    return pool


def parity_check(L, torch, dist, args, world, rank, dev, local_rank, total_steps, pool, data, run_step):
    """One step, outside every timed region, whose result is compared (on rank 0) with the same step on ONE pool
    that holds all heads and all tokens, and with the NumPy oracle on sampled sequences.  Returns the `parity`
    object of the JSON line; a mismatch ends the run with a non-zero exit code."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    from parity import TOL_BF16, parity_errors, to_np
    from oracle import attention as oattn
    from oracle import paged as opaged
    kp, vp, q_all, k_all, v_all = data
    lens0 = workload_lengths()
    q0 = q_all[0].clone()
    got_local = run_step(q0, k_all[0], v_all[0], False).clone()     # [world, n, hq, D] / [n, HQ, D] / [n, hq, D]
    torch.cuda.synchronize()
    if world > 1 and args.shard == "head":
        got_local = got_local.movedim(0, 1).reshape(N_SEQS, HQ, D)
    result = None
    if rank == 0:
        # the unsharded pool: all heads, all tokens, filled from every rank's regenerated data
        if world == 1:
            full, q_full, out_full = pool, q0, got_local
        else:
            full = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=HKV, head_dim=D, max_seqs=N_SEQS,
                                               num_pages=int(sum(-(-(int(t) + 2 * P) // P) for t in lens0)) + 16,
                                               max_pages_per_seq=int(-(-(lens0.max() + 2 * P) // P)), page_size=P,
                                               dtype=torch.bfloat16, device=local_rank, rope_theta=THETA))
            for s in range(N_SEQS):
                assert full.alloc_sequence() == s
                full.reserve(s, int(lens0[s]) + 1)
            if args.shard == "head":
                hkv = HKV // world
                hist = None
                qs, ks, vs = [], [], []
                for r in range(world):
                    kp_r, vp_r, q_r, k_r, v_r = data if r == 0 else rank_data(r, world, "head", total_steps, dev)
                    tables = rank_tables(r, world, "head", total_steps)[6]
                    qs.append(q_r[0]); ks.append(k_r[0]); vs.append(v_r[0])
                    for s in range(N_SEQS):                # the rank's heads of sequence s, in token order
                        T = int(lens0[s])
                        pg = torch.as_tensor(tables[s][: -(-T // P)] if T else tables[s][:0], device=dev, dtype=torch.long)
                        kk = kp_r[pg].permute(1, 0, 2, 3).reshape(hkv, -1, D)[:, :T]
                        vv = vp_r[pg].permute(1, 0, 2, 3).reshape(hkv, -1, D)[:, :T]
                        if hist is None:
                            hist = [[torch.empty((HKV, int(t), D), device=dev, dtype=torch.bfloat16) for t in lens0] for _ in range(2)]
                        hist[0][s][r * hkv:(r + 1) * hkv] = kk
                        hist[1][s][r * hkv:(r + 1) * hkv] = vv
                    del kp_r, vp_r
                q_full = torch.cat(qs, dim=1).contiguous()
                k_new, v_new = torch.cat(ks, dim=1).contiguous(), torch.cat(vs, dim=1).contiguous()
            else:
                from lokahi_b200.sharding import InterleavedShard
                hist = [[torch.empty((HKV, int(t), D), device=dev, dtype=torch.bfloat16) for t in lens0] for _ in range(2)]
                for r in range(world):
                    kp_r, vp_r, q_r, k_r, v_r = data if r == 0 else rank_data(r, world, "seq", total_steps, dev)
                    tables = rank_tables(r, world, "seq", total_steps)[6]
                    sh = InterleavedShard(r, world, SEQ_BLOCK, P)
                    for s in range(N_SEQS):
                        idx = sh.global_positions(int(lens0[s]))
                        if not idx:
                            continue
                        pg = torch.as_tensor(tables[s][: -(-len(idx) // P)], device=dev, dtype=torch.long)
                        ix = torch.as_tensor(idx, device=dev, dtype=torch.long)
                        hist[0][s][:, ix] = kp_r[pg].permute(1, 0, 2, 3).reshape(HKV, -1, D)[:, :len(idx)]
                        hist[1][s][:, ix] = vp_r[pg].permute(1, 0, 2, 3).reshape(HKV, -1, D)[:, :len(idx)]
                    del kp_r, vp_r
                q_full, k_new, v_new = q_all[0].clone(), k_all[0], v_all[0]
            for s in range(N_SEQS):
                if int(lens0[s]):
                    full.append(0, hist[0][s][None], hist[1][s][None], seq_ids=[s], start_pos=[0])
            del hist
            out_full = full.decode_step(0, q_full, k_new, v_new)
            torch.cuda.synchronize()
        err_unsharded = parity_errors(got_local, to_np(out_full))[0] if world > 1 else 0.0
        # the oracle on the logical history of sampled sequences: shortest, longest, two drawn at random
        pick = sorted({int(np.argmin(lens0)), int(np.argmax(lens0)), *np.random.default_rng(SEED + 9).choice(N_SEQS, 2, replace=False).tolist()})
        err_oracle = 0.0
        for s in pick:
            T = int(lens0[s]) + 1
            kd, vd = full.gather(0, seq_ids=[s], max_len=T)
            ref = oattn.chunked_grouped_attention(to_np(q_full[s])[None, :, None, :], to_np(kd), to_np(vd),
                                                  query_positions=np.array([T - 1], dtype=np.int32))
            err_oracle = max(err_oracle, parity_errors(got_local[s], ref[0, :, 0, :])[0])
            qr = opaged.rope_rows(to_np(q_all[0][s] if world == 1 or args.shard == "seq" else torch.cat([x[s] for x in qs], 0))[None], np.array([T - 1]), THETA)[0]
            import ml_dtypes
            qr = qr.astype(ml_dtypes.bfloat16).astype(np.float32)      # one bf16 step of slack: sincosf vs NumPy cos/sin
            if not np.all(np.abs(to_np(q_full[s]) - qr) <= np.abs(qr) * 2.0 ** -7 + 1e-30):
                raise SystemExit(f"parity: rotated q of sequence {s} differs from the oracle's RoPE")
        result = {"checked": True, "tolerance": TOL_BF16, "vs_oracle_max_norm_err": err_oracle, "sequences": pick,
                  "vs_unsharded_pool_max_norm_err": err_unsharded if world > 1 else None,
                  "vs_unsharded_pool_sequences": N_SEQS if world > 1 else 0}
        if not (err_oracle <= TOL_BF16 and err_unsharded <= TOL_BF16):
            print(json.dumps({"parity": result, "error": "parity check failed"}), flush=True)
            raise SystemExit(3)
    # every rank goes back to the workload's starting lengths (the token written above is overwritten by the first step)
    _, _, lens_local, _ = rank_geometry(rank, world, args.shard)
    for s in range(N_SEQS):
        if pool.length(0, s) != int(lens_local[s]):
            pool.truncate(0, int(lens_local[s]), seq_ids=[s])
    torch.cuda.synchronize()
    if world > 1:
        ok = torch.tensor([1 if (rank != 0 or result is not None) else 0], device=dev, dtype=torch.int32)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    return result


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
    if args.shard == "head":
        shard = HeadShard(rank, world, HQ, HKV)        # raises when the KV heads do not divide over the ranks
    K, W, R = args.steps, args.warmup, max(1, args.repeats)
    K2 = min(K, 32)
    total_steps = W + K + 4                                # every timed repeat re-runs the same K steps
    hkv, hq, lens_local, seq_sh = rank_geometry(rank, world, args.shard)
    lens0 = workload_lengths()
    pool = build_pool(L, torch, rank, world, args.shard, total_steps, dev, local_rank)
    data = rank_data(rank, world, args.shard, total_steps, dev)
    kp, vp = pool.layer_views(0)
    kp.copy_(data[0]); vp.copy_(data[1])
    data = (kp, vp) + data[2:]
    _, _, q_all, k_all, v_all = data
    out_buf = torch.empty((N_SEQS, hq, D), device=dev, dtype=torch.bfloat16)
    gathered = torch.empty((world, N_SEQS, hq, D), device=dev, dtype=torch.bfloat16) if world > 1 else None
    mode = "plain" if world == 1 else ("seq" if args.shard == "seq" else args.gather)
    peer = None
    if mode in ("fused", "seq"):
        # peer-mapped buffers need torch symmetric memory on every rank; without it KV-head sharding falls back to
        # the NCCL all-gather on all ranks together (sequence sharding has no such fallback here)
        try:
            peer = (L.PeerGather(shard, N_SEQS, D, torch.bfloat16, dev, n_results=2 * e2e_block(world)) if mode == "fused"
                    else L.PeerSeqMerge(rank, world, N_SEQS, HQ, D, torch.bfloat16, dev, n_results=2 * e2e_block(world)))
            ok_local = 1
        except Exception as exc:   # noqa: BLE001 - any failure means "no peer mapping here"
            sys.stderr.write(f"[bench] rank {rank}: peer exchange unavailable ({exc})\n")
            ok_local = 0
        flag = torch.tensor([ok_local], device=dev, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            if mode == "seq":
                raise SystemExit("sequence sharding needs peer-mapped buffers (torch symmetric memory)")
            mode, peer = "nccl", None
    state = {"view": out_buf, "step": 0}

    def positions_for(step_index):
        cur = [int(t) + step_index for t in lens0]
        return cur, [seq_sh.owner(p) == rank for p in cur]

    def step_call(q, k, v, consecutive, step_index=None, out=None):
        """The library call of one decode step: RoPE of q and of the new K row, the append and the attention in the
        split-K kernel, then the merge kernel (under sharding: with the exchange between the GPUs inside it)."""
        if mode == "fused":
            state["view"] = pool.decode_step(0, q, k, v, exchange=peer, consecutive=consecutive)
        elif mode == "seq":
            cur, store = positions_for(state["step"] if step_index is None else step_index)
            state["view"] = pool.decode_step(0, q, k, v, exchange=peer, positions=cur, store=store, consecutive=consecutive)
        else:
            state["view"] = out_buf if out is None else out
            pool.decode_step(0, q, k, v, out=state["view"], consecutive=consecutive and mode != "nccl")
        return state["view"]

    def step(q, k, v, consecutive=True, step_index=None, out=None, gathered_out=None):
        view = step_call(q, k, v, consecutive, step_index, out)
        if mode == "nccl":
            state["view"] = gathered if gathered_out is None else gathered_out
            dist.all_gather_into_tensor(state["view"], view)
            view = state["view"]
        return view

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def rewind(n_steps_done):
        """Back to the state after `n_steps_done` steps from the workload's start (lengths only: the pages keep the
        appended rows, which the next run overwrites with the same bytes)."""
        for s in range(N_SEQS):
            want = int(lens0[s]) + n_steps_done if seq_sh is None else seq_sh.local_count(int(lens0[s]) + n_steps_done)
            if pool.length(0, s) != want:
                pool.truncate(0, want, seq_ids=[s])
        state["step"] = n_steps_done

    # ---- parity: one step against an unsharded pool and the oracle, outside every timed region ----------------
    parity = None
    if not args.no_parity:
        parity = parity_check(L, torch, dist, args, world, rank, dev, local_rank, total_steps, pool, data,
                              lambda q, k, v, c: step(q, k, v, c, 0))
    rewind(0)

    # ---- device-resident leg ---------------------------------------------------------------------------------
    # The inputs of step j are tensors of their own, so the calls are bound once (tensor checks and argument
    # marshalling happen here, not in the loop): bound[j](layer, stream) is one library call.
    bound = None
    if mode != "nccl":
        bound = []
        for j in range(W + K):
            kw = {"consecutive": True}
            if mode == "seq":
                kw["positions"], kw["store"] = positions_for(j)
            if mode in ("fused", "seq"):
                bound.append(pool.decode_step_binder(q_all[j], k_all[j], v_all[j], exchange=peer, **kw))
            else:
                bound.append(pool.decode_step_binder(q_all[j], k_all[j], v_all[j], out_buf, **kw))

    def run_steps(first, count, consecutive=True):
        if bound is not None:
            stream = torch.cuda.current_stream().cuda_stream
            for j in range(first, first + count):
                state["view"] = bound[j](0, stream)
            state["step"] = first + count
            return
        for i in range(count):
            j = first + i
            state["step"] = j
            step(q_all[j], k_all[j], v_all[j], consecutive, j)

    run_steps(0, W)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms_repeats, launches = [], 0
    host_us = []
    for r in range(R):
        rewind(W)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        launches0 = L._lib.lib.skv_launch_count()
        ev0.record()
        t_host = time.perf_counter()
        run_steps(W, K)
        host_us.append((time.perf_counter() - t_host) / K * 1e6)      # host time to enqueue a step (no sync inside)
        ev1.record()
        barrier()
        launches = L._lib.lib.skv_launch_count() - launches0
        ms_repeats.append(ev0.elapsed_time(ev1))
    clocks = sampler.stop() if rank == 0 else None

    # instrumented pass (not part of `value`): the same steps with CUDA events around the library call only
    # (split-K kernel + merge kernel, under sharding with the exchange inside it), for the roofline
    rewind(W)
    attn_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K2)]
    barrier()
    l_inst0 = L._lib.lib.skv_launch_count()
    for i in range(K2):
        j = W + i
        state["step"] = j
        attn_ev[i][0].record()
        step_call(q_all[j], k_all[j], v_all[j], False, j)
        attn_ev[i][1].record()
        if mode == "nccl":
            dist.all_gather_into_tensor(gathered, out_buf)
    launches_per_call = (L._lib.lib.skv_launch_count() - l_inst0) // K2
    barrier()
    attn_ms = np.array([a.elapsed_time(b) for a, b in attn_ev])
    if K2 > 4:
        attn_ms = attn_ms[2:]                             # the first launches after a barrier absorb rank skew
    # kernel-only pass under sharding: this rank's share of the step with no exchange at all (what one GPU needs for
    # its own heads / tokens), so that step time splits into kernels and exchange + skew
    kernel_only_ms = None
    if world > 1:
        rewind(W)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(K):
            j = W + i
            if mode == "seq":
                cur, store = positions_for(j)
                pool.decode_step(0, q_all[j], k_all[j], v_all[j], positions=cur, store=store, out=out_buf, consecutive=True)
            else:
                pool.decode_step(0, q_all[j], k_all[j], v_all[j], out=out_buf, consecutive=True)
        e1.record()
        barrier()
        kernel_only_ms = e0.elapsed_time(e1) / K
    if pool.check_device_status() != 0:
        raise SystemExit("device status flag set during the timed region")
    steps_timed = W + np.arange(K2)[K2 - len(attn_ms):]
    if seq_sh is None:
        algo_bytes = float(np.mean([algorithmic_bytes(lens0 + j + 1, hq, hkv) for j in steps_timed]))
    else:
        algo_bytes = float(np.mean([algorithmic_bytes(np.array([seq_sh.local_count(int(t) + j + 1) for t in lens0]), hq, hkv)
                                    for j in steps_timed]))

    # ---- end-to-end leg: every step's inputs come from pinned host memory, every step's result goes back ------------
    # `HostStepPipeline` (the package's host side of the decode step): two device staging buffers, the upload of step
    # s + 1 on a copy stream while step s computes, the result of step s read back on a third stream while step s + 1
    # computes, in blocks of E2E_BLOCK steps; the host waits for the results of block j - 2 before it enqueues block j, and
    # for the last results before the clock stops.  With the NCCL gather (the baseline) the same choreography runs from torch calls.
    Ke = K
    rewind(W)
    nq, nk = N_SEQS * hq * D, N_SEQS * hkv * D
    qkv_h = torch.cat([q_all[W:W + Ke].reshape(Ke, nq), k_all[W:W + Ke].reshape(Ke, nk), v_all[W:W + Ke].reshape(Ke, nk)], dim=1).cpu().pin_memory()
    res_shape = tuple(state["view"].shape) if mode != "nccl" else tuple(gathered.shape)
    # Under sharding every rank holds the whole result after a step.  Rank 0 reads all of it back (one host process has
    # the step's complete result, as with one GPU); the other ranks read back their own share of it (head sharding: the
    # rows of their heads; sequence sharding: a 1/N block of the rows), so the result does not cross the host link N times.
    readback = None
    if world > 1 and rank > 0 and mode != "nccl":
        share = int(np.prod(res_shape)) // world
        readback = (rank * share, share)
        res_shape = (share,)
    E2E_BLOCK = e2e_block(world)
    out_rows = 2 * E2E_BLOCK if mode != "nccl" else 2
    out_h = torch.empty((out_rows,) + res_shape, dtype=torch.bfloat16).pin_memory()
    if mode != "nccl":
        pipe = L.HostStepPipeline(pool, 0, N_SEQS, hq, exchange=peer, readback=readback, block=E2E_BLOCK,
                                  step_args=(lambda i: dict(zip(("positions", "store"), positions_for(W + i)))) if mode == "seq" else None,
                                  n_steps=Ke if mode == "seq" else None)

        def e2e_run(count):
            pipe.run(qkv_h[:count], out_h)
    else:
        qkv_d = [torch.empty((nq + 2 * nk,), device=dev, dtype=torch.bfloat16) for _ in range(2)]
        views = [(b[:nq].view(N_SEQS, hq, D), b[nq:nq + nk].view(N_SEQS, hkv, D), b[nq + nk:].view(N_SEQS, hkv, D)) for b in qkv_d]
        out_d = [torch.empty_like(out_buf) for _ in range(2)]
        gat_d = [torch.empty_like(gathered) for _ in range(2)]
        up, down, main = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev), torch.cuda.current_stream()
        ev_up, ev_step, ev_done = ([torch.cuda.Event() for _ in range(2)] for _ in range(3))

        def e2e_run(count):
            with torch.cuda.stream(up):
                qkv_d[0].copy_(qkv_h[0], non_blocking=True)
                ev_up[0].record(up)
            for i in range(count):
                b = i & 1
                if i + 1 < count:
                    with torch.cuda.stream(up):
                        if i >= 1:
                            up.wait_event(ev_step[1 - b])
                        qkv_d[1 - b].copy_(qkv_h[i + 1], non_blocking=True)
                        ev_up[1 - b].record(up)
                main.wait_event(ev_up[b])
                if i >= 2:
                    main.wait_event(ev_done[b])
                view = step(*views[b], False, W + i, out_d[b], gat_d[b])
                ev_step[b].record(main)
                with torch.cuda.stream(down):
                    down.wait_event(ev_step[b])
                    out_h[b].copy_(view, non_blocking=True)
                    ev_done[b].record(down)
                if i >= 1:
                    ev_done[1 - b].synchronize()
            ev_done[(count - 1) & 1].synchronize()

    e2e_run(min(max(W, 3), Ke))
    rewind(W)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    t0 = time.perf_counter()
    e2e_run(Ke)
    e1.record()
    wall_e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    ms_e2e = max(e0.elapsed_time(e1), wall_e2e_ms)      # the host has every result when the wall clock stops
    if pool.check_device_status() != 0:
        raise SystemExit("device status flag set during the end-to-end leg")
    # the last result the host received against the same step made again from device-resident inputs, on its own
    # (the pages hold the rows of the steps before it either way; q is taken from the host copy because a step
    # rotates q in place)
    rewind(W + Ke - 1)
    last = qkv_h[Ke - 1].to(dev)
    chk = step(last[:nq].view(N_SEQS, hq, D).clone(), last[nq:nq + nk].view(N_SEQS, hkv, D).clone(),
               last[nq + nk:].view(N_SEQS, hkv, D).clone(), False, W + Ke - 1)
    torch.cuda.synchronize()
    chk = chk.float().cpu()
    if readback is not None:
        chk = chk.reshape(-1)[readback[0]:readback[0] + readback[1]]
    e2e_diff = float((chk - out_h[(Ke - 1) % out_rows].float()).abs().max() / chk.abs().max().clamp_min(1e-30))
    if not e2e_diff <= TOL_E2E:
        print(f"end-to-end result differs from the device-resident step: normalised max error {e2e_diff:.3e}", file=sys.stderr)
        raise SystemExit(3)

    # ---- max over ranks ------------------------------------------------------------------------------------------
    stats = torch.tensor(ms_repeats + [ms_e2e, float(attn_ms.mean()), kernel_only_ms or 0.0, float(np.median(host_us)), e2e_diff],
                         device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    stats = [float(x) for x in stats.tolist()]
    ms_repeats, (ms_e2e, attn_mean_ms, kernel_only_ms, host_us_per_call, e2e_diff) = stats[:R], stats[R:]
    ms_total = float(np.median(ms_repeats))

    result = None
    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        achieved = algo_bytes / (attn_mean_ms * 1e-3) / 1e9
        tokens = N_SEQS * K
        step_desc = {2: "decode step call: split-K kernel with RoPE and the append folded in + merge kernel"
                        + (" (exchange between the GPUs and its wait inside the merge kernel)" if mode in ("fused", "seq") else ""),
                     3: "decode step call: append kernel + split-K kernel + merge kernel"}.get(
                         launches_per_call, f"decode step call: {launches_per_call} launches")
        result = {
            "metric": "paged GQA decode tokens/s", "value": tokens / (ms_total * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_total / K, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": base_config(world, parallelism_label(world, args.shard, mode)),
            "repeats": R, "ms_per_step_repeats": [m / K for m in ms_repeats],
            "timing": "median over `repeats` timed regions of K steps each (every region bracketed by a barrier and a device "
                      "synchronisation, max over ranks per region); steps are enqueued back to back and a step's split-K "
                      "kernel overlaps the previous step's merge kernel",
            "e2e": {"value": N_SEQS * Ke / (ms_e2e * 1e-3), "unit": "tokens/s", "ms_per_step": ms_e2e / Ke,
                    "h2d_bytes_per_step": int(nq + 2 * nk) * 2, "d2h_bytes_per_step": int(np.prod(res_shape)) * 2,
                    "bytes_are": "per rank; d2h is rank 0's, which reads back the whole result" +
                                 (f", the other ranks read back their 1/{world} share of it ({int(np.prod(res_shape)) * 2 // world} bytes)"
                                  if world > 1 and mode != "nccl" else ""),
                    "pipeline": ("HostStepPipeline" if mode != "nccl" else "torch calls") +
                                ": upload of step s+1 and read-back of step s-1 overlap step s (three "
                                "streams); every result is awaited on the host" +
                                (f"; steps travel in blocks of {E2E_BLOCK} (one upload and one read-back per step, one "
                                 "event wait and record per block), the host two blocks ahead of the last results it holds"
                                 if mode != "nccl" else ""),
                    "host_wall_ms_per_step": wall_e2e_ms / Ke,
                    "last_result_vs_device_resident_step": e2e_diff},
            "gpu_launches": int(launches),
            "host_us_per_call": host_us_per_call,
            "kernel_only_ms": kernel_only_ms if world > 1 else None,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / 8000.0,
                         "kernel": step_desc, "launches_per_call": int(launches_per_call),
                         "algorithmic_bytes_per_launch": algo_bytes, "launch_ms": attn_mean_ms,
                         "launch_ms_min": float(attn_ms.min()), "launch_ms_median": float(np.median(attn_ms)),
                         "launch_ms_p95": float(np.percentile(attn_ms, 95)), "traffic": algo_bytes * TRAFFIC_RATIO,
                         "traffic_source": "ncu dram bytes of a 16-sequence capture, scaled by the algorithmic bytes",
                         "pipelined_frac": algo_bytes / (ms_total / K * 1e-3) / 1e9 / peak},
            "parity": parity,
            "clocks": clocks,
        }
        if world == 1:
            result["prefill"] = prefill_block(L, torch, dev)
        if world == 1 and not args.no_cpu_baseline:
            result["cpu_baseline"] = cpu_baseline_sample(pool, kp, vp, np.array([pool.length(0, s) for s in range(N_SEQS)]), hq, hkv)
    if peer is not None:
        peer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return result


def prefill_block(L, torch, dev, calls=30, warmup=5):
    """The 4096-token chunked causal GQA op (32 query heads, 8 KV heads, head_dim 128, bf16, absolute positions
    0..4095): mean CUDA-event time over `calls` launches with L2 flushed between them, causal-useful flops
    4*Hq*D*S(S+1)/2 against the measured cuBLAS bf16 burst peak.  A short side block of the default line."""
    S = 4096
    gen = torch.Generator(device=dev).manual_seed(SEED)
    q = torch.randn((1, HQ, S, D), generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn((1, HKV, S, D), generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn((1, HKV, S, D), generator=gen, device=dev).to(torch.bfloat16)
    pos = torch.arange(S, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    call = lambda: L.chunked_grouped_attention(q, k, v, query_positions=pos, causal=True, q_block_size=512, k_block_size=512)
    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(calls)]
    for a, b in evs:
        flush.zero_()
        a.record()
        call()
        b.record()
    torch.cuda.synchronize()
    L.check_dense_attention_status(dev)
    ms = np.array([a.elapsed_time(b) for a, b in evs])
    flops = 4.0 * HQ * D * (S * (S + 1) / 2)
    peak, kind = 1590.0, "fallback"
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak, kind = float(json.load(f)["bf16_tflops"]), "measured"
    tf = flops / (ms.mean() * 1e-3) / 1e12
    return {"workload": "chunked_gqa_prefill_4096", "kernel": "prefill_tc_kernel (tcgen05 + TMEM + TMA)", "calls": calls,
            "ms": float(ms.mean()), "ms_min": float(ms.min()), "tflops": tf, "frac": tf / peak, "peak": peak,
            "peak_kind": f"of {kind} (burst)", "flops_counted": "causal-useful 4*Hq*D*S(S+1)/2", "bound": "tensor",
            "l2": "flushed between calls (256 MB write)"}


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
    """Secondary workload "long_context_llama3_8b_kv": the KV path of a Llama-3-8B at 96k context sharded one KV head
    per GPU: 32 layers, 1 KV head with its 4 query heads per rank, head_dim 128, bf16, 4 sequences of 98304 tokens of
    N(0,1) K/V.  `--gpus N` runs N of the 8 shards (8 = the whole configuration); with N > 1 every layer's output rows
    are gathered by the merge kernel.  Every decode step parks the oldest 25 % of each sequence's pages in pinned host
    memory and brings them back, appends one token and attends in all 32 layers.  Two schedules are timed:
      serial    park and fetch all four sequences, wait, then attend all four;
      pingpong  two half-batches: while one half's pages travel, the other half is attended (its pages are all
                resident), then the halves swap -- every sequence is parked, fetched and attended once per step.
    Two rooflines: HBM for the attention bytes (timed with nothing travelling), the host link for the parked bytes."""
    import torch
    import torch.distributed as dist

    import lokahi_b200 as L
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    layers, n_seq, hkv, hq, T0 = 32, 4, 1, 4, args.context
    K, W = max(1, min(args.steps, 64)), max(1, min(args.warmup, 3))
    room = 3 * (K + W) + 16
    pages_per_seq = -(-(T0 + room) // P)
    park = (T0 // P) // 4
    pool = L.PagedPool(L.PagedKVConfig(num_layers=layers, num_kv_heads=hkv, head_dim=D, num_pages=n_seq * pages_per_seq + 8,
                                       max_seqs=n_seq, max_pages_per_seq=pages_per_seq, page_size=P, dtype=torch.bfloat16,
                                       device=local_rank, host_pages=n_seq * park + 8, rope_theta=THETA))
    for s_ in range(n_seq):
        assert pool.alloc_sequence() == s_
        pool.reserve(s_, T0 + room)
    gen = torch.Generator(device=dev).manual_seed(SEED + 17 * rank)
    pool_set_lengths(pool, layers, n_seq, T0)        # declares the history (writes zeros) ...
    for layer in range(layers):                      # ... which is then filled with N(0,1) K/V in place
        kp, vp = pool.layer_views(layer)
        kp.normal_(generator=gen)
        vp.normal_(generator=gen)
    # one q per layer: the step rotates it in place, which keeps its norm, so the buffers are simply reused
    q = torch.randn((layers, n_seq, hq, D), generator=gen, device=dev).to(torch.bfloat16)
    kn = torch.randn((n_seq, hkv, D), generator=gen, device=dev).to(torch.bfloat16)
    vn = torch.randn((n_seq, hkv, D), generator=gen, device=dev).to(torch.bfloat16)
    halves = ([0, 1], [2, 3])
    peers = {}
    if world > 1:
        shard = L.HeadShard(rank, world, hq * world, hkv * world)
        for n in (n_seq, 2):
            peers[n] = L.PeerGather(shard, n, D, torch.bfloat16, dev)
    outs = {n_seq: torch.empty((n_seq, hq, D), device=dev, dtype=torch.bfloat16), 2: torch.empty((2, hq, D), device=dev, dtype=torch.bfloat16)}

    def bind(rows):
        n = len(rows)
        sel = slice(rows[0], rows[-1] + 1)
        ids = None if n == n_seq else rows
        if world > 1:
            return [pool.decode_step_binder(q[layer, sel], kn[sel], vn[sel], exchange=peers[n], seq_ids=ids, consecutive=True)
                    for layer in range(layers)]
        return [pool.decode_step_binder(q[layer, sel], kn[sel], vn[sel], outs[n], seq_ids=ids, consecutive=True)
                for layer in range(layers)]

    calls = {"all": bind(list(range(n_seq))), 0: bind(halves[0]), 1: bind(halves[1])}

    def attend(which):
        stream = torch.cuda.current_stream().cuda_stream
        for layer, call in enumerate(calls[which]):
            call(layer, stream)                      # RoPE + append + attention (+ gather): one library call per layer

    def move(rows):
        for s_ in rows:
            pool.evict(s_, 0, park)
        for s_ in rows:
            pool.prefetch(s_, 0, park)

    def step_serial():
        move(range(n_seq))
        pool.sync_transfers()
        attend("all")

    def step_pingpong():
        for h in (0, 1):
            move(halves[h])                          # this half's pages travel ...
            attend(1 - h)                            # ... while the other half, all resident, is attended
            pool.sync_transfers()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, count):
        for _ in range(W):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0 = pool.counters()
        l0 = L._lib.lib.skv_launch_count()
        e0.record()
        for _ in range(count):
            fn()
        e1.record()
        barrier()
        c1 = pool.counters()
        ms = e0.elapsed_time(e1) / count
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, (c1["bytes_d2h"] - c0["bytes_d2h"]) / count, (c1["bytes_h2d"] - c0["bytes_h2d"]) / count, L._lib.lib.skv_launch_count() - l0

    attn_ms, _, _, _ = timed(lambda: attend("all"), K)               # nothing travels: the HBM roofline of the attention
    copy_ms, d2h, h2d, _ = timed(lambda: (move(range(n_seq)), pool.sync_transfers()), max(2, K // 8))
    serial_ms, _, _, _ = timed(step_serial, K)
    ping_ms, d2h_p, h2d_p, launches = timed(step_pingpong, K)
    if pool.check_device_status() != 0:
        raise SystemExit("device status flag set")
    tokens_now = pool.length(0, 0)
    attn_bytes = float(layers * n_seq * (tokens_now - K // 2) * hkv * D * 2 * 2)
    peak, kind = measured_peak_gbs()
    # ---- parity, after the timed regions: one more step of the last layer (all pages have travelled to the host and
    # back several times by now) against the NumPy oracle on one sequence's logical history, on every rank for its own
    # head; under sharding every slot of the gathered view against what its rank computed (NCCL all-gather) ----------
    parity = None
    if not args.no_parity:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        from parity import TOL_BF16, parity_errors, to_np
        from oracle import attention as oattn
        from oracle import paged as opaged
        pool.sync_transfers()
        lc, sc = layers - 1, n_seq - 1
        T = pool.length(lc, sc)
        qc = torch.randn((n_seq, hq, D), generator=gen, device=dev).to(torch.bfloat16)
        q_in = to_np(qc[sc:sc + 1])
        if world > 1:
            view = pool.decode_step(lc, qc, kn, vn, exchange=peers[n_seq])
            local = view[rank]
        else:
            view = local = pool.decode_step(lc, qc, kn, vn, out=outs[n_seq])
        torch.cuda.synchronize()
        kd, vd = pool.gather(lc, seq_ids=[sc])
        ref = oattn.chunked_grouped_attention(to_np(qc[sc])[None, :, None, :], to_np(kd[:, :, :T + 1]), to_np(vd[:, :, :T + 1]),
                                              query_positions=np.array([T], dtype=np.int32))
        err = float(parity_errors(local[sc], ref[0, :, 0, :])[0])
        q_ref = opaged.rope_rows(q_in, np.array([T]), THETA)
        q_err = float(np.max(np.abs(to_np(qc[sc:sc + 1]) - q_ref)) / np.max(np.abs(q_ref)))
        exchange_equal = True
        if world > 1:
            every = [torch.empty_like(local) for _ in range(world)]
            dist.all_gather(every, local.contiguous())
            exchange_equal = all(bool(torch.equal(view[r_], every[r_])) for r_ in range(world))
        worst = torch.tensor([err, q_err, 0.0 if exchange_equal else 1.0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        err, q_err, bad = (float(x) for x in worst.tolist())
        parity = {"checked": True, "tolerance": TOL_BF16, "layer": lc, "sequence": sc, "tokens": int(T + 1),
                  "vs_oracle_max_norm_err_max_over_ranks": err, "rotated_q_max_norm_err": q_err,
                  "gathered_slots_equal_their_ranks_rows": bad == 0.0}
        if not (err <= TOL_BF16 and q_err <= 2.0 ** -7 and bad == 0.0):
            if rank == 0:
                print(json.dumps({"parity": parity, "error": "parity check failed"}), flush=True)
            raise SystemExit(3)
    for pe in peers.values():
        pe.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return None
    return {
        "metric": "long-context decode tokens/s (4 sequences x 96k, one KV head per GPU)", "value": n_seq / (ping_ms * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ping_ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "long_context_llama3_8b_kv", "layers": layers, "sequences": n_seq, "context": T0, "kv_heads_local": hkv,
                   "q_heads_local": hq, "head_dim": D, "page_size": P, "parked_fraction": 0.25, "shards_running": world, "shards_total": 8,
                   "schedule": "pingpong (two half-batches: one travels while the other is attended)"},
        "schedules": {"serial_ms_per_step": serial_ms, "pingpong_ms_per_step": ping_ms, "attention_only_ms": attn_ms, "copies_only_ms": copy_ms,
                      "overlap_hidden_ms": serial_ms - ping_ms},
        "attention": {"ms_per_step": attn_ms, "algorithmic_bytes_per_gpu": attn_bytes,
                      "achieved_gbs_per_gpu": attn_bytes / (attn_ms * 1e-3) / 1e9,
                      "frac_of_hbm_peak": attn_bytes / (attn_ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}",
                      "us_per_layer_step": attn_ms / layers * 1e3},
        "transfers": {"ms_per_step": copy_ms, "d2h_bytes_per_step_per_gpu": d2h, "h2d_bytes_per_step_per_gpu": h2d,
                      "gbs_each_way_per_gpu": (d2h + h2d) / 2 / (copy_ms * 1e-3 / 2) / 1e9,
                      "gbs_each_way_all_gpus": world * (d2h + h2d) / 2 / (copy_ms * 1e-3 / 2) / 1e9,
                      "note": "evict then fetch of the same pages on one copy stream; the two directions do not overlap through mapped host memory"},
        "gpu_launches": int(launches),
        "parity": parity,
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


# ncu dram__bytes_read.sum + dram__bytes_write.sum per decode launch: measured on a 16-sequence capture of the
# same kernel (296.56 MB of traffic for 287.04 MB algorithmic) and scaled to this workload by the algorithmic
# bytes, which is what the traffic grows with.
TRAFFIC_RATIO = 296.56 / 287.04


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
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": base_config(args.gpus, parallelism_label(args.gpus, args.shard, args.gather)),
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
    ap.add_argument("--shard", choices=["head", "seq"], default="head",
                    help="N > 1: shard by KV head (output gather) or by sequence (round-robin token blocks, cross-rank merge)")
    ap.add_argument("--repeats", type=int, default=10, help="decode workload: timed regions of K steps; the median is reported")
    ap.add_argument("--no-parity", action="store_true", help="skip the parity step (one unsharded pool + the oracle on rank 0)")
    ap.add_argument("--workload", choices=["decode", "prefill", "decoder", "longctx", "glue"], default="decode",
                    help="decode: the headline paged-decode workload; prefill: the 4096-token chunked-GQA op (1 GPU)")
    ap.add_argument("--kv", choices=["dense", "paged"], default="dense",
                    help="prefill workload: K/V as dense tensors or as scattered 16-token pages of a pool")
    ap.add_argument("--context", type=int, default=98304, help="longctx workload: tokens per sequence (96k = 98304)")
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
