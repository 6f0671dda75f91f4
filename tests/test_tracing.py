"""The trace record: event kinds, names and fields of the reference's tracer (src/ollm/tracing.py:9-115)."""
from types import SimpleNamespace

import numpy as np

import lokahi_b200 as L


def test_tensor_and_operation_events_carry_the_reference_fields():
    tr = L.TensorTracer()
    x = np.zeros((2, 3, 4), dtype=np.float32)
    e1 = tr.record_tensor("query", x, phase="prefill", layer=1)
    e2 = tr.record_operation("attention", 1.5, phase="decode", layer=0, active_memory_bytes=10, peak_memory_bytes=20.0,
                             group_id="layer.0", cache_status="resident_hit", bytes_transferred=64, bandwidth_bytes_per_second=3)
    assert (e1.kind, e1.name, e1.phase, e1.layer, e1.shape, e1.dtype, e1.byte_size) == ("tensor", "query", "prefill", 1, (2, 3, 4), "float32", 96)
    assert e1.duration_ms is None and e2.shape is None
    assert (e2.kind, e2.duration_ms, e2.active_memory_bytes, e2.peak_memory_bytes) == ("operation", 1.5, 10, 20)
    assert (e2.group_id, e2.cache_status, e2.bytes_transferred, e2.bandwidth_bytes_per_second) == ("layer.0", "resident_hit", 64, 3.0)
    dicts = tr.to_dicts()
    assert [d["name"] for d in dicts] == ["query", "attention"]
    assert set(dicts[0]) == {"kind", "name", "phase", "layer", "shape", "dtype", "byte_size", "duration_ms", "active_memory_bytes",
                             "peak_memory_bytes", "group_id", "cache_status", "bytes_transferred", "bandwidth_bytes_per_second"}
    tr.clear()
    assert tr.events == []


def test_objects_without_nbytes_use_size_times_itemsize():
    view = SimpleNamespace(shape=(1, 2, 5, 8), dtype="bfloat16", size=80, itemsize=2)
    assert L.TensorTracer().record_tensor("key", view, phase="decode").byte_size == 160
