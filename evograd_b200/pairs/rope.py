"""RoPE autograd pair (rotate-half convention, x laid out [batch, heads, tokens,
head_dim]): no activation is saved, the backward is the transposed rotation and
only needs the cos/sin tables.

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op rope <this file>``, ``evograd bench``, ``evograd suite``):
exports ``rope_forward_with_saved`` / ``rope_backward_from_saved`` with the
signatures the declaration derives (src/evograd/ops/level1/rope/__init__.py:98-162).
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
def _forward_with_saved_impl(x, cos, sin):
    return ops.rope_fwd(x, cos, sin, layout="bhtd"), (cos, sin)


def _backward_from_saved_impl(dy, saved_tensors):
    cos, sin = saved_tensors
    return (ops.rope_bwd(dy, cos, sin, layout="bhtd"),)
# EVOLVE-BLOCK-END


def rope_forward_with_saved(x, cos, sin):
    return _forward_with_saved_impl(x, cos, sin)


def rope_backward_from_saved(dy, saved_tensors):
    return _backward_from_saved_impl(dy, saved_tensors)
