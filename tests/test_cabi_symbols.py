"""The C-ABI library loads on a machine without a GPU and exports exactly what include/*.h declares."""
import ctypes
import glob
import os
import re

from conftest import ROOT


def declared_symbols():
    names = set()
    for header in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = open(header).read()
        names |= set(re.findall(r"SKV_API\s+[\w\s\*]+?\b(skv_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    from lokahi_b200 import _lib
    decl = declared_symbols()
    assert len(decl) >= 28
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(decl):
        assert hasattr(raw, name), f"{name} declared in the header but not exported"
    assert decl == set(_lib.SIGNATURES), "ctypes binding and header disagree"
    assert _lib.lib.skv_abi_version() == _lib.ABI_VERSION


def test_status_strings_and_null_handling():
    from lokahi_b200 import _lib
    assert _lib.lib.skv_status_string(0) == b"ok"
    assert b"append" in _lib.lib.skv_status_string(_lib.ERR_REPLAY)
    assert _lib.lib.skv_create(None, None) == _lib.ERR_BAD_ARG
    assert _lib.lib.skv_destroy(None) == _lib.OK
    assert _lib.lib.skv_decode_workspace_bytes(None, 1, 1) == 0


def test_compute_entry_points_fail_loudly_without_cuda():
    import pytest
    import torch
    import lokahi_b200 as L
    if torch.cuda.is_available():
        pytest.skip("this check is for machines without a GPU")
    with pytest.raises(RuntimeError, match="no CPU path"):
        L.PagedPool(L.PagedKVConfig(num_layers=1, num_kv_heads=1, head_dim=8, num_pages=2, max_seqs=1, max_pages_per_seq=2))
    with pytest.raises(RuntimeError, match="no CPU path"):
        L.chunked_grouped_attention(torch.zeros(1, 1, 1, 8), torch.zeros(1, 1, 1, 8), torch.zeros(1, 1, 1, 8))
    assert L.B200Backend().is_available() is False
