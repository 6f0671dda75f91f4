"""Regenerate the golden fixtures in this folder from the reference checkout.

Run once, in a container that holds the reference source tree:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's own NumPy code (nothing from this repository):
  * ``grouped_attention_reference``  -- tests/test_mlx_attention.py:17-40, applied
    to the seeded inputs of the reference's attention tests (:53-130);
  * ``CPUReferenceExecutor`` linear / RMSNorm / SiLU arithmetic --
    src/ollm/backends/cpu_reference.py:230-369.
The RoPE fixture uses the inline float formula of the reference's RoPE test
(tests/test_mlx_generation.py:259-280) with float64 cos/sin tables.

The fixtures are small ``.npz`` files holding inputs and expected outputs, so
the tests need neither the reference nor this script at run time.
"""
from __future__ import annotations

import os
import sys
from types import SimpleNamespace

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def attention_cases(ref):
    cases = {}
    # each reference test builds a fresh default_rng(0) in setUp (:45-46)
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 4, 7, 6), dtype=np.float32)
    k = rng.standard_normal((1, 2, 9, 6), dtype=np.float32)
    v = rng.standard_normal((1, 2, 9, 6), dtype=np.float32)
    cases["unmasked"] = dict(q=q, k=k, v=v, out=ref(q, k, v), q_block=3, k_block=4, causal=0)

    rng = np.random.default_rng(0)
    q = rng.standard_normal((2, 4, 7, 6), dtype=np.float32)
    k = rng.standard_normal((2, 2, 7, 6), dtype=np.float32)
    v = rng.standard_normal((2, 2, 7, 6), dtype=np.float32)
    pos = np.broadcast_to(np.arange(7), (2, 7)).astype(np.int32)
    cases["causal_prefill"] = dict(q=q, k=k, v=v, positions=pos, out=ref(q, k, v, pos),
                                   q_block=3, k_block=2, causal=1)

    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 4, 1, 6), dtype=np.float32)
    k = rng.standard_normal((1, 2, 6, 6), dtype=np.float32)
    v = rng.standard_normal((1, 2, 6, 6), dtype=np.float32)
    pos = np.array([[5]], dtype=np.int32)
    cases["decode_abs_position"] = dict(q=q, k=k, v=v, positions=pos, out=ref(q, k, v, pos),
                                        q_block=1, k_block=2, causal=1)

    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, 2, 5, 4), dtype=np.float32)
    k = rng.standard_normal((1, 1, 5, 4), dtype=np.float32)
    v = rng.standard_normal((1, 1, 5, 4), dtype=np.float32)
    v2 = v.copy()
    v2[:, :, 3:] += 1000.0
    pos = np.arange(5, dtype=np.int32)[None]
    cases["future_values"] = dict(q=q, k=k, v=v, v_changed=v2, positions=pos,
                                  out=ref(q, k, v, pos), out_changed=ref(q, k, v2, pos),
                                  q_block=32768, k_block=2, causal=1)

    # A larger seeded case at the head geometry of the benchmark workload,
    # still small enough for a CPU test.
    rng = np.random.default_rng(1234)
    q = rng.standard_normal((2, 8, 12, 128), dtype=np.float32)
    k = rng.standard_normal((2, 2, 40, 128), dtype=np.float32)
    v = rng.standard_normal((2, 2, 40, 128), dtype=np.float32)
    pos = np.stack([np.arange(28, 40), np.arange(10, 22)]).astype(np.int32)
    cases["gqa_d128_offsets"] = dict(q=q, k=k, v=v, positions=pos, out=ref(q, k, v, pos),
                                     q_block=5, k_block=16, causal=1)
    return cases


def rope_case():
    rng = np.random.default_rng(11)
    q = rng.normal(size=(1, 2, 3, 4)).astype(np.float32)
    k = rng.normal(size=(1, 1, 3, 4)).astype(np.float32)
    positions = np.array([[0, 2, 5]], dtype=np.int32)
    dim, base = 4, 10000.0
    inv = 1.0 / (base ** (np.arange(0, dim, 2, dtype=np.float64) / dim))
    freqs = np.outer(positions.reshape(-1).astype(np.float64), inv)
    emb = np.concatenate([freqs, freqs], axis=-1)
    cos = np.cos(emb).reshape(1, 3, dim)[:, None]
    sin = np.sin(emb).reshape(1, 3, dim)[:, None]

    def rotate_half(x):
        a, b = np.split(x, 2, axis=-1)
        return np.concatenate([-b, a], axis=-1)

    return dict(q=q, k=k, positions=positions, dim=dim, base=base,
                q_out=(q * cos + rotate_half(q) * sin).astype(np.float32),
                k_out=(k * cos + rotate_half(k) * sin).astype(np.float32))


def glue_case(executor_cls):
    ex = executor_cls()
    rng = np.random.default_rng(5)
    x = rng.normal(size=(2, 5, 16)).astype(np.float32)
    w = rng.normal(0.0, 0.2, size=(24, 16)).astype(np.float32)
    scale = rng.normal(1.0, 0.1, size=(16,)).astype(np.float32)
    op = lambda **attrs: SimpleNamespace(operation_id="golden", attributes=attrs)
    return dict(
        x=x, w=w, scale=scale, eps=1e-6,
        linear=ex._linear(op(weight_layout="out_in"), (x, w)).astype(np.float32),
        rms=ex._rms_norm(op(epsilon=1e-6), (x, scale)).astype(np.float32),
        silu=ex._silu(op(), (x,)).astype(np.float32),
    )


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path to the reference checkout>")
    ref_root = sys.argv[1]
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from test_mlx_attention import grouped_attention_reference  # the reference's own oracle
    from ollm.backends.cpu_reference import CPUReferenceExecutor

    for name, case in attention_cases(grouped_attention_reference).items():
        np.savez_compressed(os.path.join(HERE, f"attention_{name}.npz"), **case)
    np.savez_compressed(os.path.join(HERE, "rope_half_rotation.npz"), **rope_case())
    np.savez_compressed(os.path.join(HERE, "decoder_glue.npz"), **glue_case(CPUReferenceExecutor))
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
