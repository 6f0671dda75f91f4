"""Llama / DeepSeek-style decoder around the B200 hot path.

The linear layers are torch (cuBLAS); RMSNorm (with the residual add before it) and the SiLU-gate product
are single launches of the library (``glue.py``): they are the callers of the hot path, not part of it.  What matters here is the call sequence around the cache, which
follows the reference exactly (MLXLlamaAttention.__call__, src/ollm/llama_mlx.py:220-342;
MLXLlamaModel.__call__, :740-833; MLXLlamaForCausalLM.__call__, :863-912; DeepSeek twin
src/ollm/deepseek_mlx.py:72-169, 426-549):

    past = cache.get_seq_length(); cache_position = arange(past, past + L); position_ids = [1, L]
    q, k, v = projections -> [B, H, L, D]
    RoPE(q, k) -> cache.update(k, v, layer, {"cache_position"}) -> attention(q, K, V,
        query_positions=position_ids, causal=True, q_block_size=32768,
        k_block_size=1024 if L > 128 else 1000000) -> o_proj

With ``fused_rope=True`` (default) RoPE and the append are one launch (``update_with_rope``), and a cached
decode step (L == 1) is ONE library call covering RoPE, update and attention (``decode_step_with_rope``); with
``False`` RoPE runs first and ``cache.update`` receives rotated K, as in the reference.
``use_cache=False`` never touches the cache (llama_mlx.py:762).
"""
from __future__ import annotations

import os
import time
import weakref
from typing import Any, Dict, Optional

import torch
import torch.nn.functional as F

from .attention import PagedView, chunked_grouped_attention
from .glue import add_rms_norm, rms_norm, swiglu
from .generation import greedy_generate
from .pool import rope_inv_freq, rope_rows


def rope_scaling_factor(config: Any) -> float:
    """Linear position scaling factor of a config (1.0 when absent).  The reference reads only
    ``rope_theta`` (llama_mlx.py:698-702); the factor follows the Hugging Face "linear" convention."""
    f = getattr(config, "rope_scaling_factor", None)
    if f:
        return float(f)
    rs = getattr(config, "rope_scaling", None)
    if isinstance(rs, dict) and rs.get("type", rs.get("rope_type")) == "linear":
        return float(rs.get("factor", 1.0))
    return 1.0


class _DecodeGraphs:
    """CUDA graphs of a cached decode step for one batch size.  The hot-path call of each layer stays an ordinary
    library call (it does host-side bookkeeping: lengths, page growth, the split-K plan), so the step is cut at
    those calls: ``pre`` = embedding, first norm and the first layer's q/k/v projections; ``post[i]`` = layer i's
    output projection, residual add + norm, MLP, residual add + next norm and the next layer's q/k/v projections
    (for the last layer: the final norm and the logits).  All tensors are static buffers of the graphs' shared
    memory pool; the hot path reads q/k/v from them and writes the attention output into ``attn``."""

    def __init__(self):
        self.ids = None
        self.attn = None
        self.qkv = []          # per layer (q, k, v), each [B, H, 1, D]
        self.pre = None
        self.post = []
        self.logits = None
        self.bound = {}        # id(cache) -> (pool, per-layer bound hot-path calls)


class PagedDecoder:
    def __init__(self, config: Any, weights: Dict[str, torch.Tensor], *, tracer: Optional[Any] = None,
                 fused_rope: bool = True, fused_glue: Optional[bool] = None, decode_graphs: Optional[bool] = None):
        self.config = config
        self.w = weights
        self.tracer = tracer
        self.fused_rope = fused_rope
        # RMSNorm (+ residual add) and SwiGLU as single launches; False (or SKV_FUSED_GLUE=0): plain torch ops
        self.fused_glue = (os.environ.get("SKV_FUSED_GLUE", "1") != "0") if fused_glue is None else bool(fused_glue)
        # Cached decode steps replay CUDA graphs for everything between two hot-path calls (see _DecodeGraphs);
        # False (or SKV_DECODE_GRAPHS=0): every op is launched from Python.  Weights must not be replaced after the
        # first graphed step.
        self.decode_graphs = (os.environ.get("SKV_DECODE_GRAPHS", "1") != "0") if decode_graphs is None else bool(decode_graphs)
        self._graphs: Dict[int, "_DecodeGraphs"] = {}
        self._eager_decodes: Dict[int, int] = {}
        self.H = config.hidden_size
        self.Hq = config.num_attention_heads
        # deepseek_mlx.py:235: KV heads default to the attention-head count (MHA)
        self.Hkv = getattr(config, "num_key_value_heads", None) or self.Hq
        self.D = self.H // self.Hq
        self.eps = getattr(config, "rms_norm_eps", 1e-6)
        self.theta = float(getattr(config, "rope_theta", 10000.0))
        self.rope_scale = rope_scaling_factor(config)
        any_w = next(iter(weights.values()))
        self.device, self.dtype = any_w.device, any_w.dtype
        if not any_w.is_cuda:
            raise RuntimeError("PagedDecoder needs CUDA weights; there is no CPU path")
        self.inv_freq_np = rope_inv_freq(self.D, self.theta)
        self.inv_freq = torch.from_numpy(self.inv_freq_np).to(self.device)
        # when set to a list, (start, end) CUDA events around the hot path (RoPE + cache update + attention)
        # of every layer call are appended to it
        self.hot_path_events = None
        # One projection for q, k and v and one for gate and up (the reference projects them separately,
        # llama_mlx.py:257-281, 398-406): the weights are concatenated once, q / k / v and gate / up are strided
        # slices of the one GEMM output, and the hot path and the SwiGLU launch read them in place.
        self.fused_proj = os.environ.get("SKV_FUSED_PROJ", "1") != "0"
        self._w_qkv: Dict[int, torch.Tensor] = {}
        self._w_gate_up: Dict[int, torch.Tensor] = {}

    # -- glue (llama_mlx.py:53-92, 345-408) ------------------------------------------------------------
    def _rms_norm(self, x, weight):
        if self.fused_glue:
            return rms_norm(x.contiguous(), weight, self.eps)             # one launch
        x32 = x.float()
        var = x32.pow(2).mean(-1, keepdim=True)
        return (weight.float() * (x32 * torch.rsqrt(var + self.eps))).to(x.dtype)

    def _add_norm(self, hidden, delta, weight):
        """hidden + delta, and the RMSNorm of that sum (the residual add and the norm that follows it)."""
        if self.fused_glue:
            return add_rms_norm(hidden.contiguous(), delta.contiguous(), weight, self.eps)   # one launch, sum in place
        hidden = hidden + delta
        return hidden, self._rms_norm(hidden, weight)

    def _qkv_weight(self, layer: int) -> torch.Tensor:
        w = self._w_qkv.get(layer)
        if w is None:
            b = f"model.layers.{layer}.self_attn"
            w = self._w_qkv[layer] = torch.cat([self.w[f"{b}.q_proj.weight"], self.w[f"{b}.k_proj.weight"],
                                                self.w[f"{b}.v_proj.weight"]], dim=0).contiguous()
        return w

    def _qkv(self, layer: int, hidden: torch.Tensor):
        """q, k, v as ``[B, heads, L, D]`` views of one projection output ``[B, L, (Hq + 2 Hkv) * D]``."""
        B, L, _ = hidden.shape
        if not self.fused_proj:
            b = f"model.layers.{layer}.self_attn"
            return (F.linear(hidden, self.w[f"{b}.q_proj.weight"]).view(B, L, self.Hq, self.D).transpose(1, 2).contiguous(),
                    F.linear(hidden, self.w[f"{b}.k_proj.weight"]).view(B, L, self.Hkv, self.D).transpose(1, 2).contiguous(),
                    F.linear(hidden, self.w[f"{b}.v_proj.weight"]).view(B, L, self.Hkv, self.D).transpose(1, 2).contiguous())
        qkv = F.linear(hidden, self._qkv_weight(layer)).view(B, L, self.Hq + 2 * self.Hkv, self.D).transpose(1, 2)
        return qkv[:, :self.Hq], qkv[:, self.Hq:self.Hq + self.Hkv], qkv[:, self.Hq + self.Hkv:]

    def _mlp(self, x, b):
        if self.fused_proj and self.fused_glue:
            w = self._w_gate_up.get(b)
            if w is None:
                w = self._w_gate_up[b] = torch.cat([self.w[f"{b}.mlp.gate_proj.weight"], self.w[f"{b}.mlp.up_proj.weight"]],
                                                   dim=0).contiguous()
            gu = F.linear(x, w)
            inter = gu.shape[-1] // 2
            return F.linear(swiglu(gu[..., :inter], gu[..., inter:]), self.w[f"{b}.mlp.down_proj.weight"])
        gate = F.linear(x, self.w[f"{b}.mlp.gate_proj.weight"])
        up = F.linear(x, self.w[f"{b}.mlp.up_proj.weight"])
        act = swiglu(gate, up) if self.fused_glue else F.silu(gate) * up
        return F.linear(act, self.w[f"{b}.mlp.down_proj.weight"])

    def _rope_inplace(self, x: torch.Tensor, positions: torch.Tensor):
        """x [B, H, L, D] contiguous, one position per token shared by the batch (llama_mlx.py:777)."""
        B, H, L, D = x.shape
        view = x.view(B * H, L, D).transpose(0, 1)          # [L, B*H, D] with strides (D, L*D, 1)
        rope_rows(view, positions, self.inv_freq, self.rope_scale, out=view)
        return x

    # -- attention layer (llama_mlx.py:220-342) -----------------------------------------------------------
    def _attention(self, layer, hidden, position_ids, cache, cache_position):
        B, L, _ = hidden.shape
        b = f"model.layers.{layer}.self_attn"
        past_length = cache.get_seq_length(layer) if cache is not None else 0
        phase = "decode" if past_length > 0 else ("prefill" if cache is not None else "forward")
        started = time.perf_counter()
        q, k, v = self._qkv(layer, hidden)         # strided views of one projection output when fused_proj is on
        kwargs = {"cache_position": cache_position}
        if self.hot_path_events is not None:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        out = None
        if cache is not None and self.fused_rope and L == 1 and past_length > 0 and hasattr(cache, "decode_step_with_rope"):
            # RoPE, cache update and attention of a cached decode step in one library call (two launches)
            out = cache.decode_step_with_rope(q, k, v, layer, kwargs, inv_freq=self.inv_freq_np,
                                              scaling_factor=self.rope_scale)
        if out is None:
            q = q.contiguous()                     # rotated in place below and read by the dense / paged prefill kernels
            if cache is None or not (self.fused_rope and hasattr(cache, "update_with_rope")):
                k, v = k.contiguous(), v.contiguous()
            if cache is not None and self.fused_rope and hasattr(cache, "update_with_rope"):
                k_hist, v_hist = cache.update_with_rope(q, k, v, layer, kwargs, inv_freq=self.inv_freq_np,
                                                        scaling_factor=self.rope_scale)
            else:
                pos_dev = torch.as_tensor(cache_position, dtype=torch.int32, device=self.device)
                self._rope_inplace(q, pos_dev)
                self._rope_inplace(k, pos_dev)
                k_hist, v_hist = (k, v) if cache is None else cache.update(k, v, layer, kwargs)
            out = chunked_grouped_attention(q, k_hist, v_hist, query_positions=position_ids, causal=True,
                                            q_block_size=32768, k_block_size=(1024 if L > 128 else 1000000))
        if self.hot_path_events is not None:
            ev[1].record()
            self.hot_path_events.append(ev)
        out = out.transpose(1, 2).reshape(B, L, -1)
        out = F.linear(out, self.w[f"{b}.o_proj.weight"])
        if self.tracer is not None:
            torch.cuda.synchronize(self.device)
            # the reference records the query, the full key / value history and the layer output (llama_mlx.py:318-340)
            self.tracer.record_tensor("query", q, phase=phase, layer=layer)
            if cache is not None:
                k_seen, v_seen = PagedView(cache, layer, "key"), PagedView(cache, layer, "value")
            else:
                k_seen, v_seen = k, v
            self.tracer.record_tensor("key", k_seen, phase=phase, layer=layer)
            self.tracer.record_tensor("value", v_seen, phase=phase, layer=layer)
            self.tracer.record_tensor("attention_output", out, phase=phase, layer=layer)
            self.tracer.record_operation("attention", (time.perf_counter() - started) * 1000.0, phase=phase, layer=layer,
                                         active_memory_bytes=torch.cuda.memory_allocated(self.device),
                                         peak_memory_bytes=torch.cuda.max_memory_allocated(self.device))
        return out

    # -- graphed decode step ---------------------------------------------------------------------------------
    def _project_qkv(self, layer: int, x: torch.Tensor):
        return self._qkv(layer, x)

    def _capture_decode_graphs(self, B: int) -> _DecodeGraphs:
        g = _DecodeGraphs()
        n_layers = self.config.num_hidden_layers
        g.ids = torch.zeros((B, 1), dtype=torch.long, device=self.device)
        g.attn = torch.zeros((B, self.Hq, 1, self.D), dtype=self.dtype, device=self.device)
        head = self.w.get("lm_head.weight")
        if head is None:
            head = self.w["model.embed_tokens.weight"]
        mem = torch.cuda.graph_pool_handle()
        torch.cuda.synchronize(self.device)
        g.pre = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g.pre, pool=mem):
            hidden = self.w["model.embed_tokens.weight"][g.ids]
            x = self._rms_norm(hidden, self.w["model.layers.0.input_layernorm.weight"])
            g.qkv.append(self._project_qkv(0, x))
        for i in range(n_layers):
            b = f"model.layers.{i}"
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=mem):
                delta = F.linear(g.attn.transpose(1, 2).reshape(B, 1, -1), self.w[f"{b}.self_attn.o_proj.weight"])
                hidden, x = self._add_norm(hidden, delta, self.w[f"{b}.post_attention_layernorm.weight"])
                next_w = self.w[f"model.layers.{i + 1}.input_layernorm.weight"] if i + 1 < n_layers else self.w["model.norm.weight"]
                hidden, x = self._add_norm(hidden, self._mlp(x, b), next_w)
                if i + 1 < n_layers:
                    g.qkv.append(self._project_qkv(i + 1, x))
                else:
                    g.logits = F.linear(x, head)
            g.post.append(graph)
        return g

    def _graphed_decode(self, input_ids: torch.Tensor, cache: Any, past: int) -> torch.Tensor:
        B = input_ids.shape[0]
        g = self._graphs.get(B)
        if g is None:
            g = self._graphs[B] = self._capture_decode_graphs(B)
        # the hot-path calls on the graphs' static buffers, bound once per (cache, pool): one ctypes call per layer
        bound = g.bound.get(id(cache))
        ids_now = tuple(cache.seq_ids or ())
        if bound is None or bound[0]() is not cache or bound[1] is not cache.pool or bound[2] != ids_now:
            steps = [cache.bind_decode_step(q, k, v, g.attn, inv_freq=self.inv_freq_np, scaling_factor=self.rope_scale)
                     if hasattr(cache, "bind_decode_step") else None for q, k, v in g.qkv]
            bound = g.bound[id(cache)] = (weakref.ref(cache), cache.pool, ids_now, None if any(s is None for s in steps) else steps)
            if len(g.bound) > 8:                    # caches come and go: keep the table small
                g.bound.pop(next(iter(g.bound)))
        steps = bound[3]
        kwargs = {"cache_position": [past]}
        stream = torch.cuda.current_stream(self.device).cuda_stream
        g.ids.copy_(input_ids)
        g.pre.replay()
        for i, (q, k, v) in enumerate(g.qkv):
            if self.hot_path_events is not None:
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
            if steps is not None:
                steps[i](i, past, stream)
            elif cache.decode_step_with_rope(q, k, v, i, kwargs, inv_freq=self.inv_freq_np, scaling_factor=self.rope_scale,
                                             out=g.attn) is None:
                raise RuntimeError("the cache refused the one-call decode step inside a graphed decode")
            if self.hot_path_events is not None:
                ev[1].record()
                self.hot_path_events.append(ev)
            g.post[i].replay()
        return g.logits.clone()

    def _can_graph_decode(self, L: int, cache: Any, past: int) -> bool:
        return (self.decode_graphs and self.fused_rope and self.fused_glue and self.tracer is None and L == 1 and past > 0
                and cache is not None and hasattr(cache, "decode_step_with_rope") and self.config.num_hidden_layers > 0
                and all(cache.get_seq_length(i) == past for i in range(self.config.num_hidden_layers)))

    # -- model (llama_mlx.py:740-833, 863-912) ---------------------------------------------------------------
    def __call__(self, input_ids: torch.Tensor, past_key_values: Optional[Any] = None, use_cache: bool = False) -> torch.Tensor:
        input_ids = input_ids.to(self.device)
        B, L = input_ids.shape
        hidden = self.w["model.embed_tokens.weight"][input_ids]
        cache = past_key_values if use_cache else None
        past = cache.get_seq_length() if cache is not None else 0
        if self._can_graph_decode(L, cache, past):
            # the first cached steps of a batch size run from Python (library and cuBLAS set-up must not happen
            # inside a capture); from the third on the step replays graphs
            seen = self._eager_decodes.get(B, 0)
            if seen >= 2:
                return self._graphed_decode(input_ids, cache, past)
            self._eager_decodes[B] = seen + 1
        cache_position = list(range(past, past + L))            # host values: no device sync to validate them
        position_ids = torch.tensor([cache_position], dtype=torch.int32)
        # Same block as the reference (norm -> attention -> add -> norm -> MLP -> add, llama_mlx.py:608-658), with
        # every residual add folded into the norm that follows it.
        n_layers = self.config.num_hidden_layers
        x = self._rms_norm(hidden, self.w["model.layers.0.input_layernorm.weight"]) if n_layers else None
        for i in range(n_layers):
            b = f"model.layers.{i}"
            hidden, x = self._add_norm(hidden, self._attention(i, x, position_ids, cache, cache_position),
                                       self.w[f"{b}.post_attention_layernorm.weight"])
            next_w = self.w[f"model.layers.{i + 1}.input_layernorm.weight"] if i + 1 < n_layers else self.w["model.norm.weight"]
            hidden, x = self._add_norm(hidden, self._mlp(x, b), next_w)
        hidden = x if n_layers else self._rms_norm(hidden, self.w["model.norm.weight"])
        head = self.w.get("lm_head.weight")
        if head is None:                                          # tied-embedding fallback (llama_mlx.py:886-890)
            head = self.w["model.embed_tokens.weight"]
        return F.linear(hidden, head)

    def generate(self, input_ids, max_new_tokens: int = 100, temperature: float = 1.0, top_p: float = 1.0,
                 past_key_values: Optional[Any] = None):
        del top_p   # greedy, as in the reference (llama_mlx.py:934)
        return greedy_generate(self, input_ids, max_new_tokens=max_new_tokens, temperature=temperature,
                               past_key_values=past_key_values)
