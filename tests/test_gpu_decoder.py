"""Model-level parity: the two-layer float32 fixture (prefill 32 + 16 cached decode steps against a full
causal forward) and a truncated DeepSeek-1.3B-shaped bf16 decoder, both against the NumPy decoder oracle;
plus the reference's model tests (tests/test_mlx_generation.py:140-156, 249-257, 282-323)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import lokahi_b200 as L
from oracle import decoder as od
from oracle.kvcache import ConcatKVCache
from parity import TOL_BF16, TOL_F32, assert_parity, assert_parity_logits, bf16_round, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _to_torch(weights, dtype):
    return {k: torch.from_numpy(v).to(DEV).to(dtype) for k, v in weights.items()}


def tiny_config(**kw):
    return od.make_config(vocab_size=17, hidden_size=8, intermediate_size=12, num_hidden_layers=2,
                          num_attention_heads=2, num_key_value_heads=1, max_position_embeddings=32, **kw)


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("mha", [False, True])
def test_tiny_cached_decode_matches_full_causal_forward(fused, mha):
    cfg = tiny_config()
    if mha:
        cfg.num_key_value_heads = None
    w = od.random_weights(cfg, seed=7, std=0.15)
    model = L.PagedDecoder(cfg, _to_torch(w, torch.float32), fused_rope=fused)
    oracle = od.DecoderOracle(cfg, w)
    ids = torch.tensor([[2, 5, 3, 11]], dtype=torch.int64)
    full = model(ids, use_cache=False)
    cache = L.PagedKVCache(cfg, cache_dir=None)
    model(ids[:, :3], past_key_values=cache, use_cache=True)
    dec = model(ids[:, 3:], past_key_values=cache, use_cache=True)
    assert cache.get_seq_length() == 4
    assert np.allclose(to_np(full[:, -1, :]), to_np(dec[:, -1, :]), atol=1e-5, rtol=1e-5)
    assert np.allclose(to_np(full), oracle(ids.numpy(), use_cache=False), atol=1e-5, rtol=1e-5)


def test_cache_is_not_mutated_when_use_cache_is_false():
    cfg = tiny_config()
    model = L.PagedDecoder(cfg, _to_torch(od.random_weights(cfg, seed=7, std=0.15), torch.float32))
    cache = L.PagedKVCache(cfg, cache_dir=None)
    model(torch.tensor([[2, 5, 3]]), past_key_values=cache, use_cache=False)
    assert cache.get_seq_length() == 0


def test_generation_prefills_once_then_decodes_one_token_at_a_time():
    class RecordingModel:
        def __init__(self):
            self.config = SimpleNamespace(num_hidden_layers=1, max_position_embeddings=32)
            self.input_lengths, self.cache_lengths = [], []

        def __call__(self, input_ids, past_key_values=None, use_cache=False):
            self.input_lengths.append(input_ids.shape[1])
            self.cache_lengths.append(past_key_values.get_seq_length())
            B, Lq = input_ids.shape
            st = input_ids[:, None, :, None].float().expand(B, 1, Lq, 2).contiguous().to(DEV)
            start = past_key_values.get_seq_length()
            past_key_values.update(st, st, 0, {"cache_position": torch.arange(start, start + Lq)})
            return torch.tensor([0.0, 0.0, 0.0, 1.0, 0.0]).expand(B, Lq, 5)

    m = RecordingModel()
    out = L.greedy_generate(m, torch.tensor([[1, 2, 4, 2]]), max_new_tokens=3, temperature=1.0)
    assert m.input_lengths == [4, 1, 1] and m.cache_lengths == [0, 4, 5]
    assert tuple(out.shape) == (1, 7) and out[:, -3:].tolist() == [[3, 3, 3]]
    with pytest.raises(ValueError, match="non-negative"):
        L.greedy_generate(m, torch.tensor([[1]]), max_new_tokens=-1, temperature=1.0)
    with pytest.raises(ValueError, match="temperature must be positive"):
        L.greedy_generate(m, torch.tensor([[1]]), max_new_tokens=1, temperature=0.0)
    with pytest.raises(ValueError, match="shape"):
        L.greedy_generate(m, torch.tensor([1]), max_new_tokens=1, temperature=1.0)


def test_two_layer_fp32_fixture_prefill_then_16_decode_steps():
    """hidden 256, 4 query heads, 2 KV heads, head_dim 64, MLP 512, vocab 1024, theta 10000, weights N(0, 0.02),
    32-token prompt, 16 cached decode steps; every cached step must match the last row of a full causal
    forward over the same prefix and the oracle, 1e-4 relative."""
    cfg = od.make_config(vocab_size=1024, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                         num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128, rope_theta=10000.0)
    w = od.random_weights(cfg, seed=3)
    oracle = od.DecoderOracle(cfg, w)
    model = L.PagedDecoder(cfg, _to_torch(w, torch.float32))
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, 1024, size=(1, 32))
    tokens = od.greedy_generate(oracle, prompt, max_new_tokens=16, temperature=1.0)   # oracle's greedy tokens feed both sides
    cache = L.PagedKVCache(cfg, cache_dir=None)
    ocache = ConcatKVCache(cfg, cache_dir=None)
    logits = model(torch.from_numpy(prompt), past_key_values=cache, use_cache=True)
    ologits = oracle(prompt, past_key_values=ocache, use_cache=True)
    assert_parity(logits, ologits, TOL_F32, "prefill logits")
    for step in range(16):
        nxt = tokens[:, 32 + step: 33 + step]
        logits = model(torch.from_numpy(nxt), past_key_values=cache, use_cache=True)
        ologits = oracle(nxt, past_key_values=ocache, use_cache=True)
        full = oracle(tokens[:, : 33 + step], use_cache=False)[:, -1:, :]
        assert_parity(logits, ologits, TOL_F32, f"decode step {step} vs cached oracle")
        assert_parity(logits, full, TOL_F32, f"decode step {step} vs full causal forward")
    assert cache.get_seq_length() == 48
    for layer in range(2):   # the projections come from cuBLAS vs NumPy, so the stored K/V agree to rounding only
        assert_parity(cache[layer]["value"], ocache[layer]["value"], TOL_F32, "stored values")
        assert_parity(cache[layer]["key"], ocache[layer]["key"], TOL_F32, "rotated keys")
    out = model.generate(torch.from_numpy(prompt), max_new_tokens=16)
    assert np.array_equal(to_np(out), tokens)


def test_deepseek_shaped_bf16_decoder_truncated():
    """DeepSeek-coder-1.3B geometry (hidden 2048, 16 MHA heads of 128, MLP 5504, vocab 32256, theta 100000 with
    linear scaling 4) cut to 2 layers, batch 2, 96-token prompt and 4 decode steps, bf16, KV held in pages."""
    cfg = od.make_config(vocab_size=32256, hidden_size=2048, intermediate_size=5504, num_hidden_layers=2,
                         num_attention_heads=16, num_key_value_heads=None, max_position_embeddings=512,
                         rope_theta=100000.0, rope_scaling_factor=4.0)
    w = od.random_weights(cfg, seed=11)
    import ml_dtypes
    w16 = {k: v.astype(ml_dtypes.bfloat16).astype(np.float32) for k, v in w.items()}
    oracle = od.DecoderOracle(cfg, w16, round_dtype=ml_dtypes.bfloat16, round_glue=True)
    model = L.PagedDecoder(cfg, _to_torch(w16, torch.bfloat16))
    rng = np.random.default_rng(12)
    prompt = rng.integers(0, 32256, size=(2, 96))
    cache = L.PagedKVCache(cfg, cache_dir=None)
    ocache = ConcatKVCache(cfg, cache_dir=None)
    logits = model(torch.from_numpy(prompt), past_key_values=cache, use_cache=True)
    ologits = oracle(prompt, past_key_values=ocache, use_cache=True)
    assert_parity_logits(logits, ologits, TOL_BF16, "bf16 prefill logits")
    nxt = np.argmax(ologits[:, -1, :], axis=-1)[:, None]
    for step in range(4):
        logits = model(torch.from_numpy(nxt), past_key_values=cache, use_cache=True)
        ologits = oracle(nxt, past_key_values=ocache, use_cache=True)
        assert_parity_logits(logits, ologits, TOL_BF16, f"bf16 decode step {step}")
        nxt = np.argmax(ologits[:, -1, :], axis=-1)[:, None]
    assert cache.get_seq_length() == 100 and cache.pool.cfg.num_kv_heads == 16
    assert cache.pool.check_device_status() == 0


def test_tracer_hook_records_attention_phases():
    class Tracer:
        def __init__(self):
            self.events = []

        def record_tensor(self, name, tensor, *, phase, layer=None):
            self.events.append(("tensor", name, phase, layer, tuple(tensor.shape)))

        def record_operation(self, name, duration_ms, *, phase, layer=None, **kw):
            self.events.append(("operation", name, phase, layer, duration_ms))

    cfg = tiny_config()
    tr = Tracer()
    model = L.PagedDecoder(cfg, _to_torch(od.random_weights(cfg, seed=7, std=0.15), torch.float32), tracer=tr)
    cache = L.PagedKVCache(cfg, cache_dir=None)
    model(torch.tensor([[2, 5, 3]]), past_key_values=cache, use_cache=True)
    model(torch.tensor([[11]]), past_key_values=cache, use_cache=True)
    phases = {e[2] for e in tr.events if e[0] == "operation" and e[1] == "attention"}
    assert phases == {"prefill", "decode"}


@pytest.mark.parametrize("dtype,tol", [(torch.float32, TOL_F32), (torch.bfloat16, TOL_BF16)])
def test_glue_kernels_match_the_oracle(dtype, tol):
    """RMSNorm (alone and fused with the residual add before it) and SwiGLU against the oracle's float32
    restatement of the reference layers, at a hidden size that takes the 16-byte path and one that does not."""
    from oracle import decoder as odec
    rng = np.random.default_rng(5)
    rnd = bf16_round if dtype == torch.bfloat16 else (lambda a: a)
    for rows, hidden in ((7, 2048), (5, 100), (3, 257)):
        x = rnd(rng.standard_normal((rows, hidden), dtype=np.float32) * 3)
        d = rnd(rng.standard_normal((rows, hidden), dtype=np.float32))
        w = rnd(1.0 + 0.1 * rng.standard_normal(hidden, dtype=np.float32))
        xt, dt, wt = (torch.from_numpy(a).to(DEV).to(dtype) for a in (x, d, w))
        assert_parity(L.rms_norm(xt, wt, 1e-6), odec.rms_norm(x, w, 1e-6), tol, f"rmsnorm {rows}x{hidden}")
        h = xt.clone()
        summed, normed = L.add_rms_norm(h, dt, wt, 1e-6)
        s_ref = rnd(x + d)
        assert summed.data_ptr() == h.data_ptr()
        assert np.array_equal(to_np(summed), s_ref), "the residual sum is rounded once, like a stored tensor"
        assert_parity(normed, odec.rms_norm(s_ref, w, 1e-6), tol, f"add+rmsnorm {rows}x{hidden}")
        g = rnd(rng.standard_normal((rows, hidden), dtype=np.float32) * 4)
        gt = torch.from_numpy(g).to(DEV).to(dtype)
        assert_parity(L.swiglu(gt, dt), odec.silu(g) * d, tol, f"swiglu {rows}x{hidden}")
    with pytest.raises(ValueError, match="same shape"):
        L.swiglu(gt, dt[:1])
    with pytest.raises(RuntimeError, match="no CPU path"):
        L.rms_norm(torch.zeros(2, 8), torch.ones(8))


def test_fused_glue_decoder_agrees_with_the_torch_glue_decoder():
    """The same bf16 decoder with RMSNorm/SwiGLU as library launches and as plain torch ops: logits agree within the
    bf16 tolerance over a prefill and a few cached steps, and the caches end at the same length."""
    from oracle import decoder as odec
    cfg = odec.make_config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, intermediate_size=1024,
                           vocab_size=512, num_hidden_layers=2, rope_theta=10000.0)
    w = {k: torch.from_numpy(v).to(DEV).to(torch.bfloat16) for k, v in odec.random_weights(cfg, seed=3, std=0.05).items()}
    ids = torch.from_numpy(np.random.default_rng(4).integers(0, 512, size=(2, 40))).to(DEV)
    outs = []
    for fused in (True, False):
        model = L.PagedDecoder(cfg, w, fused_glue=fused)
        cache = L.PagedKVCache(cfg)
        logits = [model(ids, past_key_values=cache, use_cache=True)[:, -1]]
        nxt = ids[:, -1:]
        for _ in range(3):
            logits.append(model(nxt, past_key_values=cache, use_cache=True)[:, -1])
        outs.append((torch.stack(logits), cache.get_seq_length()))
    from parity import assert_parity_logits
    assert outs[0][1] == outs[1][1] == 43
    assert_parity_logits(outs[0][0], to_np(outs[1][0]), TOL_BF16, "fused glue vs torch glue")


def test_reference_style_tracer_sees_query_key_value_and_output_per_layer():
    """With the library's own ``TensorTracer`` (the reference's record, src/ollm/tracing.py): per layer and call the
    events query, key, value, attention_output and the timed operation "attention", as the reference's attention
    layer records them (llama_mlx.py:318-340); key and value describe the whole cached history."""
    cfg = tiny_config()
    tr = L.TensorTracer()
    model = L.PagedDecoder(cfg, _to_torch(od.random_weights(cfg, seed=7, std=0.15), torch.float32), tracer=tr)
    cache = L.PagedKVCache(cfg, cache_dir=None)
    model(torch.tensor([[2, 5, 3]]), past_key_values=cache, use_cache=True)
    model(torch.tensor([[11]]), past_key_values=cache, use_cache=True)
    per_call = [e for e in tr.events if e.layer == 0]
    assert [e.name for e in per_call] == ["query", "key", "value", "attention_output", "attention"] * 2
    assert [e.phase for e in per_call[:5]] == ["prefill"] * 5 and [e.phase for e in per_call[5:]] == ["decode"] * 5
    D = cfg.hidden_size // cfg.num_attention_heads
    key_decode = per_call[6]
    assert key_decode.kind == "tensor" and key_decode.shape == (1, cfg.num_key_value_heads, 4, D)
    assert key_decode.byte_size == cfg.num_key_value_heads * 4 * D * 4 and "float32" in key_decode.dtype
    op = per_call[9]
    assert op.kind == "operation" and op.duration_ms > 0 and op.active_memory_bytes is not None
    assert {e.layer for e in tr.events} == set(range(cfg.num_hidden_layers))


def test_graphed_decode_steps_equal_the_eager_ones():
    """Cached decode steps with everything between two hot-path calls replayed from CUDA graphs against the same
    steps launched op by op: identical logits (the kernels and their inputs are the same), identical cache
    lengths, for two batch sizes on one model and across the eager-to-graph switch."""
    cfg = od.make_config(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, intermediate_size=1024,
                         vocab_size=512, num_hidden_layers=3, rope_theta=10000.0)
    w = {k: torch.from_numpy(v).to(DEV).to(torch.bfloat16) for k, v in od.random_weights(cfg, seed=9, std=0.05).items()}
    rng = np.random.default_rng(10)
    runs = {}
    for graphs in (False, True):
        model = L.PagedDecoder(cfg, w, decode_graphs=graphs)
        outs = []
        for B in (2, 3):
            ids = torch.from_numpy(np.random.default_rng(11 + B).integers(0, 512, size=(B, 21))).to(DEV)
            cache = L.PagedKVCache(cfg)
            logits = model(ids, past_key_values=cache, use_cache=True)
            nxt = logits[:, -1].argmax(-1, keepdim=True)
            for _ in range(6):                      # steps 1-2 run eagerly, 3-6 replay graphs when enabled
                logits = model(nxt, past_key_values=cache, use_cache=True)
                outs.append(logits.clone())
                nxt = logits[:, -1].argmax(-1, keepdim=True)
            assert cache.get_seq_length() == 27
        runs[graphs] = outs
        if graphs:
            assert sorted(model._graphs) == [2, 3] and len(model._graphs[2].post) == 3
    for a, b in zip(runs[False], runs[True]):
        assert torch.equal(a, b)
    del rng


def test_deepseek_shaped_bf16_decoder_four_layers_2048_token_prompt():
    """The same geometry at the prompt length of the configuration: 4 of the 24 layers, one sequence, a 2048-token
    prompt (the paged tensor-core prefill inside the decoder at full length) and 4 cached decode steps, against the
    NumPy decoder oracle.  The oracle at this size is tens of seconds of CPU, which is what bounds the sample."""
    cfg = od.make_config(vocab_size=32256, hidden_size=2048, intermediate_size=5504, num_hidden_layers=4,
                         num_attention_heads=16, num_key_value_heads=None, max_position_embeddings=4096,
                         rope_theta=100000.0, rope_scaling_factor=4.0)
    w = od.random_weights(cfg, seed=13)
    import ml_dtypes
    w16 = {k: v.astype(ml_dtypes.bfloat16).astype(np.float32) for k, v in w.items()}
    oracle = od.DecoderOracle(cfg, w16, round_dtype=ml_dtypes.bfloat16, round_glue=True)
    model = L.PagedDecoder(cfg, _to_torch(w16, torch.bfloat16))
    rng = np.random.default_rng(14)
    prompt = rng.integers(0, 32256, size=(1, 2048))
    cache = L.PagedKVCache(cfg, cache_dir=None)
    ocache = ConcatKVCache(cfg, cache_dir=None)
    logits = model(torch.from_numpy(prompt), past_key_values=cache, use_cache=True)
    ologits = oracle(prompt, past_key_values=ocache, use_cache=True)
    # Every GEMM output is rounded to bf16 on both sides, after sums taken in a different order, so now and then a
    # hidden element lands one bf16 step apart (2^-8 relative).  A logit sums 2048 of them: about 0.2 % of the
    # logits' rms per rounding point, and four layers have some twenty-four such points, i.e. a spread near 1 % of
    # the rms -- the element-wise criterion (2 % of the rms) is then a two-sigma event.  The normalised maximum
    # error keeps the 2e-2 bound; the share of elements outside the element-wise criterion may reach 10 %.
    for r0 in (0, 1000, 2047):                                  # rows sampled over the prompt, the last one included
        assert_parity_logits(logits[:, r0:r0 + 1], ologits[:, r0:r0 + 1], TOL_BF16, f"prefill logits, row {r0}",
                             max_outlier_fraction=0.10)
    nxt = np.argmax(ologits[:, -1, :], axis=-1)[:, None]
    for step in range(4):
        logits = model(torch.from_numpy(nxt), past_key_values=cache, use_cache=True)
        ologits = oracle(nxt, past_key_values=ocache, use_cache=True)
        assert_parity_logits(logits, ologits, TOL_BF16, f"decode step {step} after a 2048-token prompt", max_outlier_fraction=0.10)
        nxt = np.argmax(ologits[:, -1, :], axis=-1)[:, None]
    assert cache.get_seq_length() == 2052 and cache.pool.check_device_status() == 0
