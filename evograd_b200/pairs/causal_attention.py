"""Causal attention autograd pair for q, k, v of shape [B, H, S, D]: the forward
saves O and the float32 log-sum-exp per row (q, k, v by reference); the backward
recomputes the probabilities tile by tile on the tcgen05 tensor cores.

Candidate module for evograd's correctness gate and benchmarks
(``evograd verify --op causal_attention <this file>``, ``evograd bench``, ``evograd suite``):
exports ``causal_attention_forward_with_saved`` / ``causal_attention_backward_from_saved`` with the
signatures the declaration derives (the external declaration evograd_b200/decls/b200_decls.py:causal_attention).
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
def _forward_with_saved_impl(q, k, v):
    o, lse = ops.causal_attention_fwd(q, k, v)
    return o, (q, k, v, o, lse)


def _backward_from_saved_impl(do, saved_tensors):
    q, k, v, o, lse = saved_tensors
    return ops.causal_attention_bwd(do, q, k, v, o, lse)
# EVOLVE-BLOCK-END


def causal_attention_forward_with_saved(q, k, v):
    return _forward_with_saved_impl(q, k, v)


def causal_attention_backward_from_saved(do, saved_tensors):
    return _backward_from_saved_impl(do, saved_tensors)
