"""The B200 backend inside the reference's own registry (src/ollm/backends/base.py:50-105), when the reference
package can be imported (it can in the build container; elsewhere the test is skipped).  Mirrors
tests/test_backends.py of the reference: selection by name and by ``name:device``, the unknown-name error, the
duplicate-registration error and the attention hook."""
import os
import sys

import pytest

# the reference checkout is looked for next to this repository (or where OLLM_SRC points)
REF_SRC = os.environ.get("OLLM_SRC") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference", "src"))


@pytest.fixture()
def ref_backends():
    if not os.path.isdir(os.path.join(REF_SRC, "ollm", "backends")):
        pytest.skip("reference package not present")
    sys.path.insert(0, REF_SRC)
    try:
        import ollm.backends as ob
        from ollm.backends import base
    except Exception as exc:        # optional dependencies of the reference missing
        pytest.skip(f"reference backends not importable: {exc}")
    saved = dict(base._REGISTRY)
    yield ob, base
    base._REGISTRY.clear()
    base._REGISTRY.update(saved)
    sys.path.remove(REF_SRC)
    for name in [m for m in sys.modules if m == "ollm" or m.startswith("ollm.")]:
        del sys.modules[name]
    import importlib
    import lokahi_b200.backend as lb
    importlib.reload(lb)            # back to the stand-in base class for the other tests


def test_registers_and_resolves_through_the_reference_registry(ref_backends):
    import importlib
    import torch
    import lokahi_b200.backend as lb
    ob, base = ref_backends
    lb = importlib.reload(lb)       # pick up the reference's Backend base class and BackendError
    assert issubclass(lb.B200Backend, base.Backend) and lb.BackendError is base.BackendError
    assert lb.register() is True and "b200" in ob.list_backends()
    assert ob.get_backend("b200").name == "b200"
    assert callable(ob.get_backend("b200").attention_kernel())
    with pytest.raises(base.BackendError):
        base.register_backend(lb.B200Backend())                  # duplicate name (base.py:54-55)
    with pytest.raises(base.BackendError):
        ob.select_backend("unknown:0")
    if torch.cuda.is_available():
        sel = ob.select_backend("b200:0")
        assert sel.backend.name == "b200" and sel.device_request == "0"
    else:                                                        # unavailable backends are refused at selection
        with pytest.raises(base.BackendError):
            ob.select_backend("b200:0")
    assert set(("ane", "metal", "mlx")) <= set(ob.list_backends())   # the built-ins are untouched
