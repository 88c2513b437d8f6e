"""The shared library loads on a host without a GPU and exports exactly the
entry points ``include/evg_b200.h`` declares (no compute is called here)."""

import ctypes
import re
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent
HEADER = REPO / "include" / "evg_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(evg_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from evograd_b200 import _cabi

    names = declared_functions()
    assert len(names) >= 20
    lib = ctypes.CDLL(str(_cabi.LIB_PATH))
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_binding_table_matches_header():
    from evograd_b200 import _cabi

    assert sorted(_cabi.SIGNATURES) == declared_functions()


def test_version_and_target():
    from evograd_b200 import _cabi

    assert _cabi.lib.evg_abi_version() == 2
    assert _cabi.lib.evg_built_for_sm() == 100


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected before anything is enqueued."""
    from evograd_b200 import _cabi

    lib = _cabi.lib
    assert lib.evg_softmax_fwd(None, None, 4, 4, 0, None) == -6
    assert "null" in _cabi.last_error()
    assert lib.evg_tune_set(b"no.such.knob", 1) == -8
    assert lib.evg_tune_set(b"rows.force_generic", 1) == 0
    assert lib.evg_tune_get(b"rows.force_generic") == 1
    assert lib.evg_tune_set(b"rows.force_generic", 0) == 0
    assert lib.evg_tune_get(b"rows.force_generic") == 0


def test_cpu_tensors_are_refused():
    import pytest
    import torch

    from evograd_b200 import ops

    with pytest.raises(RuntimeError, match="CUDA"):
        ops.softmax_fwd(torch.zeros(2, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.rmsnorm_fwd(torch.zeros(2, 8), torch.ones(8))
