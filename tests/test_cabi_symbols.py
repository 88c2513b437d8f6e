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

    import __graft_entry__ as entry

    assert _cabi.lib.evg_abi_version() == entry.header_abi_version() >= 2
    assert _cabi.lib.evg_built_for_sm() == 100


def test_build_entry_point_runs_clean():
    """``__graft_entry__.build()`` compiles (or finds up to date) the library,
    imports the package and checks version and target without raising."""
    import __graft_entry__ as entry

    entry.build()


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


def test_attention_scale_must_be_positive_and_finite():
    """The tensor-core kernels scale after taking the row maximum, so a scale that
    is zero, negative or not finite is refused before anything is enqueued."""
    import ctypes as C

    from evograd_b200 import _cabi

    buf = (C.c_char * 64)()
    p = C.cast(buf, C.c_void_p)
    for bad in (0.0, -0.125, float("inf"), float("nan")):
        rc = _cabi.lib.evg_causal_attention_fwd(p, p, p, p, p, 1, 1, 128, 128, bad, 2, None)
        assert rc == -8, (bad, rc)
        assert "scale" in _cabi.last_error()
        rc = _cabi.lib.evg_causal_gqa_attention_fwd(p, p, p, p, p, 1, 2, 1, 128, 128, bad, 2, None)
        assert rc == -8, (bad, rc)


def test_cpu_tensors_are_refused():
    import pytest
    import torch

    from evograd_b200 import ops

    with pytest.raises(RuntimeError, match="CUDA"):
        ops.softmax_fwd(torch.zeros(2, 8))
    with pytest.raises(RuntimeError, match="CUDA"):
        ops.rmsnorm_fwd(torch.zeros(2, 8), torch.ones(8))
