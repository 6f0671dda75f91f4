"""Decode attention for hosts that cannot allocate device memory.

Some users of the library run where cudaMalloc is off limits: all device memory was handed out at
start-up, or they live inside another program's arena.  For them skv_decode_attn_static keeps the
split-K partials in a fixed 16 MiB array inside the library, so the caller brings only q and out.
This test drives that entry point through the C ABI, twice in a row on the same inputs and then on
a changed batch (the array is shared between calls and keeps old contents, so the second and third
calls prove that stale partials are never read), and compares each result with what the ordinary
entry point (caller-provided workspace) returns.  It also checks that a request too large for the
array is refused with a clear error instead of being launched.

This file is collected last so that a failure here cannot hide the result of any other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import lokahi_b200 as L
from lokahi_b200 import _lib
from parity import TOL_BF16, assert_parity, to_np

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _pool(lens, n_pages_extra=4, hkv=8, max_pages_per_seq=None):
    rng = np.random.default_rng(99)
    P, D = 16, 128
    per = max_pages_per_seq or max(1, max(-(-(t + 1) // P) for t in lens))
    n_pages = len(lens) * min(per, max(1, max(-(-(t + 1) // P) for t in lens))) + n_pages_extra
    pool = L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=hkv, head_dim=D, num_pages=n_pages, max_seqs=len(lens),
                                       max_pages_per_seq=per, page_size=P, dtype=torch.bfloat16))
    perm = rng.permutation(n_pages)
    at = 0
    for s, t in enumerate(lens):
        n = max(1, -(-(t + 1) // P))
        assert pool.alloc_sequence() == s
        pool.set_page_table(s, perm[at:at + n].tolist(), t)
        at += n
    kp, vp = pool.layer_views(0)
    gen = torch.Generator(device=DEV).manual_seed(5)
    kp.normal_(generator=gen)
    vp.normal_(generator=gen)
    return pool, gen


def _call_static(pool, q, out, seq_ids=None, q_pos=None):
    """Straight through the C ABI: no tensor is created here."""
    st = _lib.lib.skv_decode_attn_static(pool._h, 0, _lib.i32_array(seq_ids), q.shape[0], q.data_ptr(), out.data_ptr(),
                                         _lib.i32_array(q_pos), q.shape[1], 1e-12,
                                         torch.cuda.current_stream().cuda_stream)
    _lib.raise_for_status(st, pool._h)


def test_static_scratch_decode_matches_workspace_decode_on_consecutive_calls():
    lens = [1, 16, 17, 250, 1023, 2048, 3000, 4097]
    pool, gen = _pool(lens)
    q = torch.randn((len(lens), 32, 128), generator=gen, device=DEV).to(torch.bfloat16)
    ids, qpos = [6, 0, 3], [2999, 0, 100]
    q3 = q[:3].contiguous()
    expect = pool.decode_attention(0, q)                      # ordinary entry point, caller workspace
    expect2 = pool.decode_attention(0, q3, seq_ids=ids, q_pos=qpos)
    out = torch.full_like(q, float("nan"))
    first = torch.empty_like(q)
    out2 = torch.full_like(q3, float("nan"))
    # a warm-up call first: module loading, the kernel's shared-memory attribute and the lookup of the array's address
    # happen once per device, on the first call
    _call_static(pool, q, out)
    out.fill_(float("nan"))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]                # the driver's view: sees a cudaMalloc that torch's counter would miss
    _call_static(pool, q, out)
    first.copy_(out)
    out.fill_(float("nan"))
    _call_static(pool, q, out)                                # second call reuses the array as the first left it
    # a different batch over the same array: fewer sequences, other order, explicit positions
    _call_static(pool, q3, out2, seq_ids=ids, q_pos=qpos)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before, "the static-scratch entry point must not allocate device memory"
    assert torch.cuda.mem_get_info()[0] == free_before, "free device memory changed across the static-scratch calls"
    assert_parity(first, to_np(expect), TOL_BF16, "static scratch, first call")
    assert_parity(out, to_np(expect), TOL_BF16, "static scratch, second call")
    assert torch.equal(first, expect) and torch.equal(out, expect)   # same kernels, same plan: identical bits
    assert_parity(out2, to_np(expect2), TOL_BF16, "static scratch, changed batch")
    # the Python wrapper reaches the same entry point
    assert torch.equal(pool.decode_attention_static(0, q), expect)
    assert pool.check_device_status() == 0


def test_static_scratch_rejects_requests_beyond_its_size():
    # 256 sequences x 32 query heads whose page-table rows hold 9600 tokens need 5 partials each: > 16 MiB
    lens = [8] * 256
    pool, gen = _pool(lens, max_pages_per_seq=600)
    q = torch.randn((256, 32, 128), generator=gen, device=DEV).to(torch.bfloat16)
    need = _lib.lib.skv_decode_workspace_bytes(pool._h, 256, 32)
    assert need > _lib.STATIC_SCRATCH_BYTES
    out = torch.empty_like(q)
    with pytest.raises(NotImplementedError, match="built-in scratch array holds"):
        _call_static(pool, q, out)
    # the ordinary entry point still serves the same request
    pool.decode_attention(0, q, out=out)
    torch.cuda.synchronize()
    assert np.isfinite(to_np(out)).all()
