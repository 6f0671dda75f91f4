"""B200 backend: the reference's ``Backend`` plugin surface for this hot path.

Duck-typed to the seven members of ``ollm.backends.base.Backend`` (src/ollm/backends/base.py:14-40)
and shaped like ``MLXBackend`` (src/ollm/backends/mlx_backend.py:15-96): ``create_kv_cache`` returns
the paged KV cache, ``attention_kernel`` returns the chunked-GQA callable.  When the reference
package is importable, ``register()`` adds it to the reference registry under the name "b200" so
that ``select_backend("b200")`` / ``"b200:1"`` resolve to it (base.py:70-105); the reference pins
its built-in registry contents, so registration happens from here, not by editing its package.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple

import torch

try:  # the reference package is optional
    from ollm.backends.base import Backend as _Base, BackendError  # type: ignore
except Exception:  # pragma: no cover - depends on the environment
    class BackendError(RuntimeError):
        """Raised when a backend is unavailable or misconfigured."""

    class _Base:  # minimal stand-in with the reference's member names
        name = "base"


@dataclass(frozen=True)
class B200Capabilities:
    """Field names follow ``RuntimeCapabilities`` (src/ollm/core/capabilities.py:107-125)."""

    compute_units: Tuple[str, ...] = ("gpu",)
    supported_phases: Tuple[str, ...] = ("prefill", "decode")
    supported_operations: Tuple[str, ...] = ("attention", "rope", "kv_cache")
    supported_dtypes: Tuple[str, ...] = ("float32", "bfloat16")
    supports_weight_paging: bool = False
    supports_async_prefetch: bool = True       # KV pages: pinned-host tier with async prefetch
    supports_external_kv_cache: bool = True
    supports_quantized_weights: bool = False
    supports_graph_capture: bool = False
    supports_memory_counters: bool = True
    supports_dynamic_shapes: bool = True
    supports_concurrent_dispatch: bool = True
    requires_private_api: bool = False


class B200Backend(_Base):
    name = "b200"

    def is_available(self) -> bool:
        if not torch.cuda.is_available():
            return False
        try:
            from . import _lib  # noqa: F401
        except Exception:
            return False
        return torch.cuda.get_device_capability(0)[0] >= 10

    def resolve_device(self, device_request: Optional[str]) -> Any:
        if not torch.cuda.is_available():
            raise BackendError("B200 backend is not available (no CUDA device)")
        if device_request in (None, "", "auto", "gpu", "cuda"):
            return torch.device("cuda", torch.cuda.current_device())
        req = device_request.lower()
        for prefix in ("cuda:", "gpu:"):
            if req.startswith(prefix):
                req = req[len(prefix):]
        if req.isdigit() and int(req) < torch.cuda.device_count():
            return torch.device("cuda", int(req))
        raise BackendError(f"Unsupported B200 device specification: {device_request}")

    def move_model_to_device(self, model: Any, device: Any) -> Any:
        to = getattr(model, "to", None)
        return to(device) if callable(to) else model

    def create_kv_cache(self, cache_dir: str, stats: Optional[Any], config: Optional[Any] = None,
                        model_id: Optional[str] = None, **kw):
        if not torch.cuda.is_available():
            raise BackendError("B200 backend is not available (no CUDA device)")
        if config is None:
            raise BackendError("config is required to create the paged KV cache")
        from .kvcache import create_paged_kv_cache
        return create_paged_kv_cache(model_id=model_id or "default", config=config, cache_dir=cache_dir, stats=stats, **kw)

    def attention_kernel(self):
        from .attention import chunked_grouped_attention
        return chunked_grouped_attention

    def capabilities(self):
        return B200Capabilities()


def register() -> bool:
    """Add the backend to the reference registry when ``ollm`` is importable; returns whether it did."""
    try:
        from ollm.backends.base import register_backend, _REGISTRY  # type: ignore
    except Exception:
        return False
    if B200Backend.name not in _REGISTRY:
        register_backend(B200Backend())
    return True
