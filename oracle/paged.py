"""Python model of the paged KV pool: allocator policy, page tables, logical view.

Test infrastructure only (see ``oracle/__init__.py``).

The reference has no page tables (its cache concatenates whole tensors,
src/ollm/mlx_kvcache.py:107-118), so this part of the oracle is *defined* here
("parity unpinned"): a page table denotes, per sequence, the logical
``[Hkv, T, D]`` K and V that the reference would hold after the same appends,
and attention over pages must equal the restated reference function applied to
that logical view, one sequence at a time.

Allocator policy (mirrored bit-for-bit by the C++ pool):
  * device pages form a LIFO stack initialised so that pops yield 0, 1, 2, ...;
  * sequence ids likewise;
  * releasing a run of pages pushes them in reverse slot order, so the next pops
    return them in their old slot order;
  * a request that cannot be met changes nothing and reports out-of-pages;
  * page-table entries: ``>= 0`` device page, ``-1`` unassigned,
    ``-2 - s`` parked in host slot ``s``.
"""
from __future__ import annotations

from typing import List

import numpy as np

from . import attention as _attn
from . import rope as _rope

UNASSIGNED = -1


class OutOfPages(RuntimeError):
    pass


class PagePoolModel:
    def __init__(self, num_layers: int, num_pages: int, page_size: int, max_seqs: int,
                 max_pages_per_seq: int, host_pages: int = 0):
        self.num_layers = num_layers
        self.num_pages = num_pages
        self.page_size = page_size
        self.max_seqs = max_seqs
        self.max_pages_per_seq = max_pages_per_seq
        self.free_pages: List[int] = list(range(num_pages - 1, -1, -1))   # pop() -> 0,1,2..
        self.free_seqs: List[int] = list(range(max_seqs - 1, -1, -1))
        self.free_host: List[int] = list(range(host_pages - 1, -1, -1))
        self.page_table = np.full((max_seqs, max_pages_per_seq), UNASSIGNED, dtype=np.int32)
        self.num_seq_pages = np.zeros(max_seqs, dtype=np.int32)
        self.lengths = np.zeros((num_layers, max_seqs), dtype=np.int32)
        self.live = np.zeros(max_seqs, dtype=bool)

    def alloc_sequence(self) -> int:
        if not self.free_seqs:
            raise OutOfPages("no free sequence id")
        s = self.free_seqs.pop()
        self.live[s] = True
        return s

    def free_sequence(self, seq: int):
        n = int(self.num_seq_pages[seq])
        for slot in range(n - 1, -1, -1):
            e = int(self.page_table[seq, slot])
            if e >= 0:
                self.free_pages.append(e)
            elif e <= -2:
                self.free_host.append(-2 - e)
        self.page_table[seq, :] = UNASSIGNED
        self.num_seq_pages[seq] = 0
        self.lengths[:, seq] = 0
        self.live[seq] = False
        self.free_seqs.append(seq)

    def reserve(self, seq: int, total_tokens: int):
        need = -(-total_tokens // self.page_size)
        have = int(self.num_seq_pages[seq])
        if need <= have:
            return
        if need > self.max_pages_per_seq or need - have > len(self.free_pages):
            raise OutOfPages(f"need {need - have} pages, {len(self.free_pages)} free")
        for slot in range(have, need):
            self.page_table[seq, slot] = self.free_pages.pop()
        self.num_seq_pages[seq] = need

    def append(self, layer: int, seq: int, start: int, count: int):
        """Length bookkeeping of one append; ``start`` must equal the current length."""
        cur = int(self.lengths[layer, seq])
        if start != cur:
            raise ValueError(
                "cache_position must append exactly after the cached sequence; "
                f"expected start {cur}, got {start}"
            )
        self.reserve(seq, cur + count)
        self.lengths[layer, seq] = cur + count

    def evict(self, seq: int, first_slot: int, count: int):
        if count > len(self.free_host):
            raise OutOfPages("no free host slot")
        moved = []
        for slot in range(first_slot, first_slot + count):
            e = int(self.page_table[seq, slot])
            if e < 0:
                continue
            h = self.free_host.pop()
            self.page_table[seq, slot] = -2 - h
            moved.append((slot, e, h))
        for slot, e, h in reversed(moved):
            self.free_pages.append(e)
        return moved

    def prefetch(self, seq: int, first_slot: int, count: int):
        slots = [s for s in range(first_slot, first_slot + count) if int(self.page_table[seq, s]) <= -2]
        if len(slots) > len(self.free_pages):
            raise OutOfPages("no free device page")
        moved = []
        for slot in slots:
            h = -2 - int(self.page_table[seq, slot])
            p = self.free_pages.pop()
            self.page_table[seq, slot] = p
            moved.append((slot, p, h))
        for slot, p, h in reversed(moved):
            self.free_host.append(h)
        return moved


def logical_kv(pool: np.ndarray, page_table_row: np.ndarray, length: int) -> np.ndarray:
    """``[Hkv, length, D]`` view that a page-table row denotes.

    ``pool`` has layout ``[page][Hkv][page_size][D]``.
    """
    P = pool.shape[2]
    n_pages = -(-length // P)
    pages = np.asarray(page_table_row[:n_pages], dtype=np.int64)
    if n_pages and pages.min() < 0:
        raise ValueError("page not resident")
    gathered = pool[pages]                      # [n_pages, Hkv, P, D]
    gathered = np.transpose(gathered, (1, 0, 2, 3)).reshape(pool.shape[1], n_pages * P, pool.shape[3])
    return gathered[:, :length]


def paged_decode_attention(q, k_pool, v_pool, page_table, lengths, q_positions=None,
                           seq_ids=None, k_block_size: int = 1000000, out_dtype=None):
    """One query token per sequence against its paged history.

    ``q`` is ``[num_seqs, Hq, D]``.  Applies the restated reference attention
    (``k_block_size`` 1000000 is what the reference's decode call uses,
    llama_mlx.py:307) to each sequence separately with ``B = 1, Lq = 1`` and the
    absolute position ``q_positions[i]`` (default: ``lengths[i] - 1``).
    """
    n = q.shape[0]
    seq_ids = np.arange(n) if seq_ids is None else np.asarray(seq_ids)
    out_dtype = q.dtype if out_dtype is None else out_dtype
    out = np.zeros(q.shape, dtype=out_dtype)
    for i, s in enumerate(seq_ids):
        T = int(lengths[s])
        pos = T - 1 if q_positions is None else int(q_positions[i])
        if T == 0:
            continue
        kk = logical_kv(k_pool, page_table[s], T)[None]
        vv = logical_kv(v_pool, page_table[s], T)[None]
        o = _attn.chunked_grouped_attention(
            q[i][None, :, None, :], kk, vv,
            query_positions=np.array([[pos]], dtype=np.int32), causal=True,
            q_block_size=32768, k_block_size=k_block_size, out_dtype=np.float32,
        )
        out[i] = o[0, :, 0, :].astype(out_dtype)
    return out


def write_tokens(pool: np.ndarray, page_table_row: np.ndarray, start: int, rows: np.ndarray):
    """Scatter ``rows`` (``[Hkv, n, D]``) into ``pool`` at token positions ``start..start+n``."""
    P = pool.shape[2]
    for j in range(rows.shape[1]):
        t = start + j
        pool[int(page_table_row[t // P]), :, t % P, :] = rows[:, j, :]


def rope_rows(x: np.ndarray, positions: np.ndarray, base: float, scaling_factor: float = 1.0) -> np.ndarray:
    """RoPE for ``x`` of shape ``[n, H, D]`` with one absolute position per row; float32 result."""
    cos, sin = _rope.cos_sin(np.asarray(positions).reshape(1, -1), x.shape[-1], base, scaling_factor)
    xb = np.transpose(np.asarray(x, dtype=np.float32), (1, 0, 2))[None]   # [1, H, n, D]
    y = _rope.apply(xb, cos, sin)[0]
    return np.transpose(y, (1, 0, 2))
