"""EvoformerAttention autograd pair: softmax(scale*q k^T + pair_bias + res_mask) v
over [B, N_seq, N_res, Head, Dim] tensors; the forward saves the output and the
float32 log-sum-exp (inputs are kept by reference), d_pair_bias is reduced over
the MSA axis in a fixed order without atomics.

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op evoattention <this file>``): exports
``evoattention_forward_with_saved`` / ``evoattention_backward_from_saved`` with
the signatures the declaration derives
(src/evograd/ops/level1/evoattention/__init__.py:80-137).
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
def _forward_with_saved_impl(q, k, v, res_mask, pair_bias):
    o, lse = ops.evoattention_fwd(q, k, v, res_mask, pair_bias)
    return o, (q, k, v, res_mask, pair_bias, o, lse)


def _backward_from_saved_impl(do, saved_tensors):
    q, k, v, res_mask, pair_bias, o, lse = saved_tensors
    return ops.evoattention_bwd(do, q, k, v, res_mask, pair_bias, o, lse)
# EVOLVE-BLOCK-END


def evoattention_forward_with_saved(q, k, v, res_mask, pair_bias):
    return _forward_with_saved_impl(q, k, v, res_mask, pair_bias)


def evoattention_backward_from_saved(do, saved_tensors):
    return _backward_from_saved_impl(do, saved_tensors)
