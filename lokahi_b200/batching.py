"""Batched-request decode loop: prompts arrive and finish at different times, and every step re-forms a
one-token decode batch from the sequences that are ready.

The reference has a single-request greedy loop (``greedy_generate_mx``, src/ollm/generation.py:7-50) and describes
the target above it in docs/STRATA_ENGINE_ARCHITECTURE.md:620-694: a prefill queue feeding token-budgeted prefill
batches, a decode-ready set, a one-token decode batch re-formed after every iteration because sequences end at
different times, exclusion of cancelled sequences before dispatch, wait-time aging, and KV reservations that are
honoured before a sequence is admitted (:696-723 sketches the block pool those reservations live in).  This module is
that loop for the paged pool:

* a request owns one sequence of the pool; its page-table row is reserved for ``prompt + max_new_tokens`` tokens
  when it is admitted (all or nothing: a request that does not fit stays queued, nothing is changed);
* prompts are prefilled in chunks of at most ``prefill_token_budget`` tokens per scheduling quantum
  (RoPE-on-write append + paged attention over the cached prefix, bottom-right aligned);
* the decode batch is the ``max_batch`` longest-waiting ready sequences; its rows are ragged -- every sequence sits
  at its own length -- and one layer costs one library call (``skv_decode_step_ex`` with the sequence list): RoPE at
  each row's own position, the append and the attention;  q, k and v are slices of one fused projection output;
* finished (end-of-sequence token, output bound) and cancelled sequences are freed before the next batch forms;
* with a ``KVPagePrefetcher`` the pages of the batch are pinned while it runs and the pages of the sequences that
  will form the next batch are requested first, so their copy back from host memory overlaps this batch.

Greedy argmax is the sampling contract (docs/STRATA_ENGINE_ARCHITECTURE.md:617-620); logits stay on the device and
one token id per sequence comes back to the host.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

from ._lib import OutOfPagesError


@dataclass
class DecodeRequest:
    request_id: int
    prompt: List[int]
    max_new_tokens: int
    eos_token_id: Optional[int] = None
    seq: Optional[int] = None              # sequence id in the pool once admitted
    prefilled: int = 0                     # prompt tokens already in the cache
    generated: List[int] = field(default_factory=list)
    finished: Optional[str] = None         # "eos", "length", "cancelled"
    ready_since: int = 0                   # quantum at which it last produced a token (aging)
    logits: List[torch.Tensor] = field(default_factory=list)   # kept only with record_logits=True


class BatchedDecodeLoop:
    def __init__(self, model: Any, pool: Any, *, max_batch: int = 64, prefill_token_budget: int = 2048,
                 prefetcher: Optional[Any] = None, record_logits: bool = False):
        if max_batch <= 0 or prefill_token_budget <= 0:
            raise ValueError("max_batch and prefill_token_budget must be positive")
        c = pool.cfg
        if (c.num_layers, c.num_kv_heads, c.head_dim) != (model.config.num_hidden_layers, model.Hkv, model.D):
            raise ValueError("pool geometry does not match the model")
        self.model, self.pool = model, pool
        self.max_batch, self.prefill_token_budget = int(max_batch), int(prefill_token_budget)
        self.prefetcher = prefetcher
        self.record_logits = record_logits
        self.requests: Dict[int, DecodeRequest] = {}
        self.prefill_queue: Deque[int] = deque()
        self.ready: List[int] = []
        self.quantum = 0
        self._next_id = 0
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "decode_batches": 0, "admission_deferrals": 0}
        pool.set_rope(model.inv_freq_np, model.rope_scale)
        w, n_layers = model.w, model.config.num_hidden_layers
        # one projection weight per layer, [ (Hq + 2 Hkv) * D, hidden ]: q, k, v of a step are slices of its output
        self._w_qkv = [torch.cat([w[f"model.layers.{i}.self_attn.q_proj.weight"], w[f"model.layers.{i}.self_attn.k_proj.weight"],
                                  w[f"model.layers.{i}.self_attn.v_proj.weight"]], dim=0).contiguous() for i in range(n_layers)]
        self._head = w.get("lm_head.weight")
        if self._head is None:
            self._head = w["model.embed_tokens.weight"]

    # -- the caller's side -------------------------------------------------------------------------------------
    def submit(self, prompt: List[int], max_new_tokens: int, eos_token_id: Optional[int] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("input_ids must be a non-empty rank-2 tensor")      # generation.py:17-20
        if max_new_tokens < 0:
            raise ValueError("max_new_tokens must be non-negative")              # generation.py:13-14
        rid = self._next_id
        self._next_id += 1
        req = DecodeRequest(rid, prompt, int(max_new_tokens), eos_token_id)
        self.requests[rid] = req
        if max_new_tokens == 0:
            req.finished = "length"                                              # returns the input unchanged (:21-22)
        else:
            self.prefill_queue.append(rid)
        return rid

    def cancel(self, request_id: int) -> None:
        """Takes effect before the next batch is formed; the sequence's pages go back to the pool then."""
        req = self.requests[request_id]
        if req.finished is None:
            req.finished = "cancelled"

    def pending(self) -> bool:
        return bool(self.prefill_queue) or bool(self.ready)

    def run(self, max_quanta: int = 1 << 30) -> Dict[int, List[int]]:
        """Step until every request has finished; returns the generated tokens per request id."""
        while self.pending() and max_quanta > 0:
            self.step()
            max_quanta -= 1
        return {rid: list(r.generated) for rid, r in self.requests.items()}

    # -- one scheduling quantum ----------------------------------------------------------------------------------
    def step(self) -> List[Tuple[int, int]]:
        """Retire what has finished, prefill up to the token budget, run one decode batch.  Returns the
        (request id, token) pairs produced in this quantum."""
        self.quantum += 1
        emitted: List[Tuple[int, int]] = []
        self._retire()
        budget = self.prefill_token_budget
        while self.prefill_queue and budget > 0:
            req = self.requests[self.prefill_queue[0]]
            if req.finished is not None:                      # cancelled while queued
                self.prefill_queue.popleft()
                self._free(req)
                continue
            if req.seq is None and not self._admit(req):
                self.stats["admission_deferrals"] += 1
                break                                         # the head of the queue keeps its place (no starvation)
            n = min(budget, len(req.prompt) - req.prefilled)
            logits = self._prefill_chunk(req, n)
            budget -= n
            if req.prefilled == len(req.prompt):
                self.prefill_queue.popleft()
                self._accept(req, int(logits.argmax(-1)), logits, emitted)
                if req.finished is None:
                    self.ready.append(req.request_id)
                else:                                         # one token was all it asked for (or it was the end token)
                    self._free(req)
        self._retire()
        batch = self._form_batch()
        if batch:
            self._decode_batch(batch, emitted)
        self._retire()
        return emitted

    # -- admission and retirement ------------------------------------------------------------------------------
    def _admit(self, req: DecodeRequest) -> bool:
        """A sequence id plus pages for the whole request, or nothing."""
        try:
            seq = self.pool.alloc_sequence()
        except OutOfPagesError:
            return False
        try:
            self.pool.reserve(seq, len(req.prompt) + req.max_new_tokens)
        except OutOfPagesError:
            self.pool.free_sequence(seq)
            return False
        req.seq = seq
        if self.prefetcher is not None:
            self.prefetcher.residency.track(seq)
        return True

    def _free(self, req: DecodeRequest) -> None:
        if req.seq is not None:
            if self.prefetcher is not None:
                self.prefetcher.residency.forget(req.seq)
            self.pool.free_sequence(req.seq)
            req.seq = None

    def _retire(self) -> None:
        keep = []
        for rid in self.ready:
            req = self.requests[rid]
            if req.finished is None:
                keep.append(rid)
            else:
                self._free(req)
        self.ready = keep

    def _accept(self, req: DecodeRequest, token: int, logits: torch.Tensor, emitted: List[Tuple[int, int]]) -> None:
        req.generated.append(token)
        req.ready_since = self.quantum
        if self.record_logits:
            req.logits.append(logits.detach().float().cpu())
        emitted.append((req.request_id, token))
        if req.eos_token_id is not None and token == req.eos_token_id:
            req.finished = "eos"
        elif len(req.generated) >= req.max_new_tokens:
            req.finished = "length"

    def _form_batch(self) -> List[DecodeRequest]:
        live = [self.requests[r] for r in self.ready if self.requests[r].finished is None]
        live.sort(key=lambda r: (r.ready_since, r.request_id))            # longest-waiting first
        return live[: self.max_batch]

    # -- residency ---------------------------------------------------------------------------------------------------
    def _groups(self, req: DecodeRequest) -> range:
        gp = self.prefetcher.residency.group_pages
        return range(-(-len(self.pool.page_table(req.seq)) // gp))

    def _pin(self, batch: List[DecodeRequest]):
        if self.prefetcher is None:
            return []
        # the sequences that will form the NEXT batch (those left out now, longest-waiting first) are requested
        # before this batch runs, so that their pages travel while it computes
        in_batch = {r.request_id for r in batch}
        waiting = [self.requests[r] for r in self.ready if r not in in_batch and self.requests[r].finished is None]
        waiting.sort(key=lambda r: (r.ready_since, r.request_id))
        leases = [self.prefetcher.acquire(r.seq, g) for r in batch for g in self._groups(r)]
        for r in waiting[: self.max_batch]:
            for g in self._groups(r):
                self.prefetcher.prefetch(r.seq, g)
        return leases

    # -- model ------------------------------------------------------------------------------------------------------------
    def _prefill_chunk(self, req: DecodeRequest, n: int) -> torch.Tensor:
        """``n`` more prompt tokens of one request through every layer; returns the last position's logits."""
        m, pool = self.model, self.pool
        start = req.prefilled
        ids = torch.tensor([req.prompt[start:start + n]], dtype=torch.long, device=m.device)
        hidden = m.w["model.embed_tokens.weight"][ids]                            # [1, n, H]
        n_layers = m.config.num_hidden_layers
        leases = [self.prefetcher.acquire(req.seq, g) for g in self._groups(req)] if self.prefetcher is not None else []
        x = m._rms_norm(hidden, m.w["model.layers.0.input_layernorm.weight"])
        for i in range(n_layers):
            b = f"model.layers.{i}"
            qkv = F.linear(x, self._w_qkv[i]).view(1, n, m.Hq + 2 * m.Hkv, m.D).transpose(1, 2)    # [1, heads, n, D]
            q = qkv[:, :m.Hq].contiguous()
            k, v = qkv[:, m.Hq:m.Hq + m.Hkv], qkv[:, m.Hq + m.Hkv:]
            pool.append(i, k, v, seq_ids=[req.seq], start_pos=[start], rope_k=True, q=q)
            out = pool.prefill_attention(i, q, seq_ids=[req.seq])                   # positions: start .. start + n - 1
            delta = F.linear(out.transpose(1, 2).reshape(1, n, -1), m.w[f"{b}.self_attn.o_proj.weight"])
            hidden, x = m._add_norm(hidden, delta, m.w[f"{b}.post_attention_layernorm.weight"])
            nxt = m.w[f"model.layers.{i + 1}.input_layernorm.weight"] if i + 1 < n_layers else m.w["model.norm.weight"]
            hidden, x = m._add_norm(hidden, m._mlp(x, b), nxt)
        for lease in leases:
            lease.release()
        req.prefilled += n
        self.stats["prefill_tokens"] += n
        return F.linear(x[0, -1], self._head)

    def _decode_batch(self, batch: List[DecodeRequest], emitted: List[Tuple[int, int]]) -> None:
        """One token for every request of the batch: rows are ragged, one library call per layer."""
        m, pool = self.model, self.pool
        n = len(batch)
        ids = [r.seq for r in batch]
        tokens = torch.tensor([r.generated[-1] for r in batch], dtype=torch.long, device=m.device)
        hidden = m.w["model.embed_tokens.weight"][tokens]                         # [n, H]
        n_layers = m.config.num_hidden_layers
        leases = self._pin(batch)
        attn = torch.empty((n, m.Hq, m.D), dtype=m.dtype, device=m.device)
        qd, kd = m.Hq * m.D, m.Hkv * m.D
        x = m._rms_norm(hidden, m.w["model.layers.0.input_layernorm.weight"])
        for i in range(n_layers):
            b = f"model.layers.{i}"
            qkv = F.linear(x, self._w_qkv[i])                                      # [n, (Hq + 2 Hkv) * D]
            q = qkv[:, :qd].view(n, m.Hq, m.D)
            k = qkv[:, qd:qd + kd].view(n, m.Hkv, m.D)
            v = qkv[:, qd + kd:].view(n, m.Hkv, m.D)
            pool.decode_step(i, q, k, v, out=attn, seq_ids=ids)                    # RoPE + append + attention, strided rows
            delta = F.linear(attn.view(n, -1), m.w[f"{b}.self_attn.o_proj.weight"])
            hidden, x = m._add_norm(hidden, delta, m.w[f"{b}.post_attention_layernorm.weight"])
            nxt = m.w[f"model.layers.{i + 1}.input_layernorm.weight"] if i + 1 < n_layers else m.w["model.norm.weight"]
            hidden, x = m._add_norm(hidden, m._mlp(x, b), nxt)
        for lease in leases:
            lease.release()
        logits = F.linear(x, self._head)                                          # [n, vocab], stays on the device
        picked = logits.argmax(-1).tolist()                                       # one token id per sequence comes back
        self.stats["decode_tokens"] += n
        self.stats["decode_batches"] += 1
        for row, req in enumerate(batch):
            self._accept(req, int(picked[row]), logits[row], emitted)
