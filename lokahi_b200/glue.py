"""RMSNorm and SwiGLU of the decoder block as single launches (C ABI ``skv_rmsnorm`` / ``skv_swiglu``).

Same arithmetic as the reference's layers (MLXRMSNorm, src/ollm/llama_mlx.py:77-92; the SiLU-gate product of
MLXLlamaMLP, :345-408) and the same fusion its optimised layer applies (optimized_rmsnorm,
optimized_rmsnorm_residual, optimized_swiglu, src/ollm/metal_optimizations.py:75-157): float32 inside, one
rounding per output element.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import lib, raise_for_status


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    if t.dtype == torch.float32:
        return _lib.F32
    raise ValueError("tensors must be float32 or bfloat16")


def _check(*tensors: torch.Tensor) -> None:
    first = tensors[0]
    for t in tensors:
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError("needs CUDA tensors; there is no CPU path")
        if t.dtype != first.dtype or t.device != first.device:
            raise ValueError("tensors must share dtype and device")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``weight * (x * rsqrt(mean(x^2, -1) + eps))`` over the last dimension."""
    _check(x, weight)
    hidden = x.shape[-1]
    if weight.shape != (hidden,):
        raise ValueError("weight must have shape [hidden]")
    out = torch.empty_like(x)
    rows = x.numel() // hidden if hidden else 0
    raise_for_status(lib.skv_rmsnorm(x.data_ptr(), None, None, weight.data_ptr(), out.data_ptr(), rows, hidden, float(eps),
                                     _code(x), torch.cuda.current_stream(x.device).cuda_stream))
    return out


def add_rms_norm(hidden_states: torch.Tensor, delta: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6
                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """The residual add and the norm that follows it in one launch: returns ``(hidden_states + delta, norm of that
    sum)``.  The sum is written in place into ``hidden_states``."""
    _check(hidden_states, delta, weight)
    if hidden_states.shape != delta.shape:
        raise ValueError("hidden_states and delta must have the same shape")
    hidden = hidden_states.shape[-1]
    if weight.shape != (hidden,):
        raise ValueError("weight must have shape [hidden]")
    out = torch.empty_like(hidden_states)
    rows = hidden_states.numel() // hidden if hidden else 0
    raise_for_status(lib.skv_rmsnorm(hidden_states.data_ptr(), delta.data_ptr(), hidden_states.data_ptr(), weight.data_ptr(),
                                     out.data_ptr(), rows, hidden, float(eps), _code(hidden_states),
                                     torch.cuda.current_stream(hidden_states.device).cuda_stream))
    return hidden_states, out


def _row_stride(t: torch.Tensor) -> Optional[int]:
    """Row stride of ``t`` seen as [rows, cols] (last dimension packed, leading dimensions collapsible), else None."""
    if t.dim() < 2 or t.stride(-1) != 1:
        return None
    stride = t.stride(-2)
    for d in range(t.dim() - 2, 0, -1):
        if t.stride(d - 1) != t.stride(d) * t.shape[d]:
            return None
    return stride


def swiglu(gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``silu(gate) * up`` element-wise.  ``gate`` and ``up`` may be strided row slices of one fused projection output
    (last dimension packed); the result is packed."""
    if not (gate.is_contiguous() and up.is_contiguous()):
        gs, us = _row_stride(gate), _row_stride(up)
        if gs is None or us is None or gate.shape != up.shape or not gate.is_cuda or gate.dtype != up.dtype:
            raise ValueError("gate and up must be contiguous, or row slices with a packed last dimension")
        if out is None:
            out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
        cols = gate.shape[-1]
        raise_for_status(lib.skv_swiglu_rows(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel() // cols, cols, gs, us,
                                             cols, _code(gate), torch.cuda.current_stream(gate.device).cuda_stream))
        return out
    _check(gate, up)
    if gate.shape != up.shape:
        raise ValueError("gate and up must have the same shape")
    if out is None:
        out = torch.empty_like(gate)
    raise_for_status(lib.skv_swiglu(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _code(gate),
                                    torch.cuda.current_stream(gate.device).cuda_stream))
    return out
