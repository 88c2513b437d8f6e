"""LayerNorm autograd pair: the forward adds only float32 mean/rstd per row to the
saved state (x and weight are kept by reference); dweight/dbias use a two-stage
atomic-free column reduction.

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op layernorm <this file>``, ``evograd bench``, ``evograd suite``):
exports ``layernorm_forward_with_saved`` / ``layernorm_backward_from_saved`` with the
signatures the declaration derives (src/evograd/ops/level1/layernorm/__init__.py:124-171).
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
def _forward_with_saved_impl(x, weight, bias, eps=1e-5):
    y, mean, rstd = ops.layernorm_fwd(x, weight, bias, eps)
    return y, (x, weight, mean, rstd)


def _backward_from_saved_impl(dy, saved_tensors, eps=1e-5):
    _ = eps  # the statistics already contain it
    x, weight, mean, rstd = saved_tensors
    return ops.layernorm_bwd(dy, x, weight, mean, rstd)
# EVOLVE-BLOCK-END


def layernorm_forward_with_saved(x, weight, bias, eps=1e-5):
    return _forward_with_saved_impl(x, weight, bias, eps)


def layernorm_backward_from_saved(dy, saved_tensors, eps=1e-5):
    return _backward_from_saved_impl(dy, saved_tensors, eps)
