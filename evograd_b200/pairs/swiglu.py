"""SwiGLU autograd pair: c = silu(a)*b; nothing is saved beyond a and b. The
backward writes fresh da/db (set EVG_SWIGLU_IN_PLACE=1 to write them over a and
b, which the declaration allows).

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op swiglu <this file>``, ``evograd bench``, ``evograd suite``):
exports ``swiglu_forward_with_saved`` / ``swiglu_backward_from_saved`` with the
signatures the declaration derives (src/evograd/ops/level1/swiglu/__init__.py:61-97).
All arithmetic runs in the sm_100a kernels of ``libevg_b200.so``.
"""

import os
import sys

# evograd imports candidates by file path, so the package root may be absent
# from sys.path.
_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from evograd_b200 import ops  # noqa: E402

_IN_PLACE = os.environ.get("EVG_SWIGLU_IN_PLACE", "0") == "1"


# EVOLVE-BLOCK-START
def _forward_with_saved_impl(a, b):
    return ops.swiglu_fwd(a, b), (a, b)


def _backward_from_saved_impl(dc, saved_tensors):
    a, b = saved_tensors
    in_place = _IN_PLACE and a.is_contiguous() and b.is_contiguous()
    return ops.swiglu_bwd(dc, a, b, in_place=in_place)
# EVOLVE-BLOCK-END


def swiglu_forward_with_saved(a, b):
    return _forward_with_saved_impl(a, b)


def swiglu_backward_from_saved(dc, saved_tensors):
    return _backward_from_saved_impl(dc, saved_tensors)
