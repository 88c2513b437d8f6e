"""GeGLU autograd pair: c = gelu_tanh(a)*b; nothing is saved beyond a and b.

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op geglu <this file>``, ``evograd bench``, ``evograd suite``):
exports ``geglu_forward_with_saved`` / ``geglu_backward_from_saved`` with the
signatures the declaration derives (src/evograd/ops/level1/geglu/__init__.py:52-84).
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


# EVOLVE-BLOCK-START
def _forward_with_saved_impl(a, b):
    return ops.geglu_fwd(a, b), (a, b)


def _backward_from_saved_impl(dc, saved_tensors):
    a, b = saved_tensors
    return ops.geglu_bwd(dc, a, b)
# EVOLVE-BLOCK-END


def geglu_forward_with_saved(a, b):
    return _forward_with_saved_impl(a, b)


def geglu_backward_from_saved(dc, saved_tensors):
    return _backward_from_saved_impl(dc, saved_tensors)
