"""RMSNorm autograd pair: the forward adds only float32 rstd per row to the saved
state (x and weight are kept by reference); dweight uses a two-stage atomic-free
column reduction.

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op rmsnorm <this file>``, ``evograd bench``, ``evograd suite``):
exports ``rmsnorm_forward_with_saved`` / ``rmsnorm_backward_from_saved`` with the
signatures the declaration derives (src/evograd/ops/level1/rmsnorm/__init__.py:72-130).
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
def _forward_with_saved_impl(x, weight, eps=1e-5):
    y, rstd = ops.rmsnorm_fwd(x, weight, eps)
    return y, (x, weight, rstd)


def _backward_from_saved_impl(dy, saved_tensors, eps=1e-5):
    _ = eps  # rstd already contains it
    x, weight, rstd = saved_tensors
    return ops.rmsnorm_bwd(dy, x, weight, rstd)
# EVOLVE-BLOCK-END


def rmsnorm_forward_with_saved(x, weight, eps=1e-5):
    return _forward_with_saved_impl(x, weight, eps)


def rmsnorm_backward_from_saved(dy, saved_tensors, eps=1e-5):
    return _backward_from_saved_impl(dy, saved_tensors, eps)
