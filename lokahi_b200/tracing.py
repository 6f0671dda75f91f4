"""Trace records with the reference's event names and fields.

``TensorTracer`` of the reference (src/ollm/tracing.py:9-115) collects two kinds of events, "tensor" (name,
phase, layer, shape, dtype, byte size) and "operation" (name, phase, layer, duration, memory readings, group id,
cache status, bytes moved and bandwidth), and keeps only scalar metadata so that tracing never pins activations.
This is the same record and the same two calls for users without ``ollm`` installed; an ``ollm.tracing``
tracer can be passed wherever this one is accepted (``PagedDecoder(tracer=...)``, ``KVPagePrefetcher(tracer=...)``),
the keyword arguments are the reference's.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass
from threading import RLock
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TraceEvent:
    kind: str                                   # "tensor" or "operation"
    name: str
    phase: str
    layer: Optional[int] = None
    shape: Optional[Tuple[int, ...]] = None
    dtype: Optional[str] = None
    byte_size: Optional[int] = None
    duration_ms: Optional[float] = None
    active_memory_bytes: Optional[int] = None
    peak_memory_bytes: Optional[int] = None
    group_id: Optional[str] = None
    cache_status: Optional[str] = None
    bytes_transferred: Optional[int] = None
    bandwidth_bytes_per_second: Optional[float] = None


def _int_or_none(x):
    return None if x is None else int(x)


class TensorTracer:
    def __init__(self) -> None:
        self.events: List[TraceEvent] = []
        self._lock = RLock()

    def _add(self, event: TraceEvent) -> TraceEvent:
        with self._lock:
            self.events.append(event)
        return event

    def record_tensor(self, name: str, tensor: Any, *, phase: str, layer: Optional[int] = None) -> TraceEvent:
        """Metadata of a tensor-like object: anything with ``shape`` and ``dtype`` and either ``nbytes`` or
        ``size`` and ``itemsize`` (dense tensors and the cache's paged views both qualify)."""
        nbytes = getattr(tensor, "nbytes", None)
        if nbytes is None:
            size = getattr(tensor, "size", 0)
            size = size() if callable(size) else size
            try:
                size = int(size)
            except TypeError:                   # torch.Size
                n = 1
                for d in size:
                    n *= int(d)
                size = n
            nbytes = size * int(getattr(tensor, "itemsize", 0))
        return self._add(TraceEvent(kind="tensor", name=name, phase=phase, layer=layer,
                                    shape=tuple(int(d) for d in tensor.shape), dtype=str(tensor.dtype), byte_size=int(nbytes)))

    def record_operation(self, name: str, duration_ms: float, *, phase: str, layer: Optional[int] = None,
                         active_memory_bytes: Optional[int] = None, peak_memory_bytes: Optional[int] = None,
                         group_id: Optional[str] = None, cache_status: Optional[str] = None,
                         bytes_transferred: Optional[int] = None,
                         bandwidth_bytes_per_second: Optional[float] = None) -> TraceEvent:
        return self._add(TraceEvent(
            kind="operation", name=name, phase=phase, layer=layer, duration_ms=float(duration_ms),
            active_memory_bytes=_int_or_none(active_memory_bytes), peak_memory_bytes=_int_or_none(peak_memory_bytes),
            group_id=group_id, cache_status=cache_status, bytes_transferred=_int_or_none(bytes_transferred),
            bandwidth_bytes_per_second=None if bandwidth_bytes_per_second is None else float(bandwidth_bytes_per_second)))

    def clear(self) -> None:
        with self._lock:
            self.events.clear()

    def to_dicts(self) -> List[Dict[str, Any]]:
        with self._lock:
            return [asdict(e) for e in self.events]
