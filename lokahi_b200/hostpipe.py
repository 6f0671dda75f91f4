"""Decode steps fed from pinned host memory: upload, step and read-back as a three-stream pipeline.

A caller whose per-step inputs live in host memory (the q, k, v rows of a step arrive from another process, a
network card, a CPU stage) pays one host-to-device copy and one device-to-host copy per step.  Issued one after
the other on one stream they add to the step; here the upload of step s + 1 runs on a copy stream while step s
computes, the result of step s is read back on a third stream while step s + 1 computes, and the host waits for
result s - ``lookahead`` before it enqueues step s + 1 (and for the last results before ``run`` returns).  With
``lookahead`` 1 the chain "step done, read-back, host wakes, next enqueue" has to fit into one step, which it does not
when a step is short; the default 2 gives it two.
Steps can also travel in blocks of ``block``: the block's uploads, its steps and its read-backs are each enqueued
together, with one event wait before the block's first step and one event record after its last.  Every step still
gets its own upload and its own read-back; what changes is how often an event sits between two steps on the compute
stream.  An event record or wait between two steps keeps the second from starting beside the first (the library's
back-to-back mode), and on eight GPUs a step that starts on its own takes 54 us against 29 us beside its predecessor.
``2 * block`` device staging buffers and as many result buffers rotate.  The per-step choreography (copies, event records and waits) goes
straight to the CUDA runtime through ctypes, and the step itself is a bound library call
(``PagedPool.decode_step_binder``), so a step costs the host a few microseconds beside the two launches.

The reference has no counterpart (its arrays live in unified memory); this is the host side of the decode step
for a discrete GPU.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import torch

_H2D, _D2H = 1, 2


def _cudart():
    """The CUDA runtime torch itself uses (already loaded in the process)."""
    for name in ("libcudart.so.12", "libcudart.so"):
        try:
            lib = C.CDLL(name)
            lib.cudaMemcpyAsync.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
            lib.cudaEventRecord.argtypes = [C.c_void_p, C.c_void_p]
            lib.cudaStreamWaitEvent.argtypes = [C.c_void_p, C.c_void_p, C.c_uint]
            lib.cudaEventSynchronize.argtypes = [C.c_void_p]
            return lib
        except OSError:
            continue
    raise RuntimeError("the CUDA runtime library is not loadable; HostStepPipeline needs it")


class HostStepPipeline:
    """Runs ``decode_step`` for a fixed batch shape with inputs from, and results to, pinned host tensors.

    ``exchange`` (a ``sharding.PeerGather`` / ``PeerSeqMerge`` built with ``n_results = 2 * block``) makes the step the
    sharded one; ``step_args`` is called with the step index and returns the per-step keyword arguments of
    ``decode_step_binder`` that vary (``positions`` / ``store`` under sequence sharding), or is None.  ``consecutive``
    passes the library's back-to-back promise: between two steps the compute stream holds at most event records and
    waits (the wait for a block's uploads comes before its first step, so the inputs are complete when a kernel
    starts, however early that is).  ``readback`` = (first element, element count) reads back only that contiguous part
    of a step's flattened result (under sharding every rank holds the whole gathered result; a rank that only needs
    its own rows on the host does not pay for N copies of it); ``outputs`` is then ``[rows, count]``."""

    def __init__(self, pool, layer: int, n_seqs: int, n_q_heads: int, *, exchange=None, step_args=None, n_steps: Optional[int] = None,
                 consecutive: bool = True, lookahead: int = 2, block: int = 1, readback: Optional[Tuple[int, int]] = None):
        c = pool.cfg
        self.pool, self.layer = pool, layer
        dev = pool.torch_device
        D, hkv = c.head_dim, c.num_kv_heads
        if lookahead not in (1, 2):
            raise ValueError("lookahead is 1 or 2 (blocks)")
        if not 1 <= block <= 16:
            raise ValueError("block is 1 to 16 steps")
        self.lookahead, self.block = lookahead, block
        self.n_slots = slots = 2 * block
        if exchange is not None and exchange.n_results != slots:
            raise ValueError(f"the exchange rotates {exchange.n_results} result buffers, blocks of {block} need {slots}")
        self.nq, self.nk = n_seqs * n_q_heads * D, n_seqs * hkv * D
        self.in_elems = self.nq + 2 * self.nk
        self.stage = [torch.empty((self.in_elems,), device=dev, dtype=c.dtype) for _ in range(slots)]
        self.views = [(b[:self.nq].view(n_seqs, n_q_heads, D), b[self.nq:self.nq + self.nk].view(n_seqs, hkv, D),
                       b[self.nq + self.nk:].view(n_seqs, hkv, D)) for b in self.stage]
        self.exchange = exchange
        self.consecutive = bool(consecutive)
        self.results = None if exchange is not None else [torch.empty((n_seqs, n_q_heads, D), device=dev, dtype=c.dtype) for _ in range(slots)]
        self.result_shape = tuple(exchange.out_shape) if exchange is not None else (n_seqs, n_q_heads, D)
        self.readback = None
        if readback is not None:
            first, count = int(readback[0]), int(readback[1])
            total = 1
            for d_ in self.result_shape:
                total *= d_
            if first < 0 or count <= 0 or first + count > total:
                raise ValueError("readback lies outside the result")
            self.readback = (first, count)
            self.result_shape = (count,)
        self.esize = self.stage[0].element_size()
        self.rt = _cudart()
        self.up, self.down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.main = torch.cuda.current_stream(dev)
        mk = lambda: [torch.cuda.Event() for _ in range(2)]      # by block parity
        self.ev_up, self.ev_step, self.ev_done = mk(), mk(), mk()
        for group, stream in ((self.ev_up, self.up), (self.ev_step, self.main), (self.ev_done, self.down)):
            for e in group:
                e.record(stream)                       # creates the CUDA event behind the torch object
        torch.cuda.synchronize(dev)
        # the step calls, bound once: one per slot (staging buffer s and result buffer s; with an exchange the result
        # buffer is the exchange's own rotation of as many buffers), or one per step when arguments vary by step
        self._calls: List = []
        if step_args is None:
            for slot in range(slots):
                self._calls.append(self._bind(slot, {}))
        else:
            if n_steps is None:
                raise ValueError("n_steps is needed with step_args")
            for i in range(n_steps):
                self._calls.append(self._bind(self._slot(i), step_args(i)))
        self._per_step = step_args is not None

    def _slot(self, i: int) -> int:
        """Staging / result slot of step i: block parity times the block length, plus the step's place in its block."""
        return ((i // self.block) & 1) * self.block + i % self.block

    def _bind(self, slot: int, kw: dict):
        q, k, v = self.views[slot]
        kw = dict(kw, consecutive=self.consecutive)
        if self.exchange is not None:
            return self.pool.decode_step_binder(q, k, v, exchange=self.exchange, **kw)
        return self.pool.decode_step_binder(q, k, v, self.results[slot], **kw)

    def run(self, inputs: torch.Tensor, outputs: torch.Tensor) -> None:
        """``inputs`` pinned ``[n_steps, in_elems]`` (row = q | k | v of a step, flattened), ``outputs`` pinned
        ``[rows, *result_shape]`` with ``rows >= 2 * block``: the result of step i lands in row ``i % rows`` (a ring when
        there are fewer rows than steps; a consumer that needs time with a row gives more rows).
        Runs the steps in order and returns when the last result is in ``outputs``."""
        if not (inputs.is_pinned() and outputs.is_pinned()):
            raise ValueError("inputs and outputs must be pinned host tensors")
        n = inputs.shape[0]
        rows_out = outputs.shape[0]
        if inputs.shape[1] != self.in_elems or tuple(outputs.shape[1:]) != self.result_shape or rows_out < min(n, self.n_slots):
            raise ValueError("inputs / outputs do not match the pipeline's shapes")
        if self._per_step and n > len(self._calls):
            raise ValueError("more steps than were bound")
        rt, esize = self.rt, self.esize
        up, down, main = self.up.cuda_stream, self.down.cuda_stream, self.main.cuda_stream
        e_up = [e.cuda_event for e in self.ev_up]
        e_step = [e.cuda_event for e in self.ev_step]
        e_done = [e.cuda_event for e in self.ev_done]
        stage = [t.data_ptr() for t in self.stage]
        in_ptr, in_row = inputs.data_ptr(), inputs.stride(0) * esize
        out_ptr, out_row = outputs.data_ptr(), outputs.stride(0) * outputs.element_size()
        in_bytes, out_bytes = self.in_elems * esize, outputs[0].numel() * outputs.element_size()
        src_off = self.readback[0] * outputs.element_size() if self.readback is not None else 0
        layer, calls, per_step, look, B = self.layer, self._calls, self._per_step, self.lookahead, self.block
        memcpy, record, wait, sync = rt.cudaMemcpyAsync, rt.cudaEventRecord, rt.cudaStreamWaitEvent, rt.cudaEventSynchronize
        wait(up, e_step[0], 0)                                     # whatever ran before has finished with the staging buffers
        wait(up, e_step[1], 0)
        for t in range(min(B, n)):
            memcpy(stage[t], in_ptr + t * in_row, in_bytes, _H2D, up)
        record(e_up[0], up)
        for j in range((n + B - 1) // B):                          # block j: steps first .. first + count - 1
            b, first = j & 1, j * B
            count = min(B, n - first)
            if look == 2 and j >= 2:
                sync(e_done[b])                                    # the host consumes the results of block j - 2 here
            wait(main, e_up[b], 0)
            if look == 1 and j >= 2:
                wait(main, e_done[b], 0)                           # the result buffers of this parity have been read back
            views = [calls[first + t if per_step else b * B + t](layer, main) for t in range(count)]   # the steps, back to back
            record(e_step[b], main)
            wait(down, e_step[b], 0)
            for t in range(count):
                memcpy(out_ptr + ((first + t) % rows_out) * out_row, views[t].data_ptr() + src_off, out_bytes, _D2H, down)
            record(e_done[b], down)
            nxt = first + count
            if nxt < n:                                            # the next block's inputs, while this block computes
                if j >= 1:
                    wait(up, e_step[1 - b], 0)                     # block j - 1 has finished reading those staging buffers
                for t in range(min(B, n - nxt)):
                    memcpy(stage[(1 - b) * B + t], in_ptr + (nxt + t) * in_row, in_bytes, _H2D, up)
                record(e_up[1 - b], up)
            if look == 1 and j >= 1:
                sync(e_done[1 - b])                                # the host consumes the results of block j - 1 here
        sync(e_done[0])
        sync(e_done[1])
