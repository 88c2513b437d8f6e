"""Row softmax autograd pair: the forward saves y only; dx = y*(dy - sum(dy*y)).

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op softmax <this file>``, ``evograd bench``, ``evograd suite``):
exports ``softmax_forward_with_saved`` / ``softmax_backward_from_saved`` with the
signatures the declaration derives (src/evograd/ops/level1/softmax/__init__.py:69-92).
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
def _forward_with_saved_impl(x):
    y = ops.softmax_fwd(x)
    return y, (y,)


def _backward_from_saved_impl(dy, saved_tensors):
    (y,) = saved_tensors
    return (ops.softmax_bwd(y, dy),)
# EVOLVE-BLOCK-END


def softmax_forward_with_saved(x):
    return _forward_with_saved_impl(x)


def softmax_backward_from_saved(dy, saved_tensors):
    return _backward_from_saved_impl(dy, saved_tensors)
