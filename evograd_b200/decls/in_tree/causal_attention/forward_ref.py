"""Trusted forward of the ``causal_attention`` operator (in-tree form).

The same call the reference's decoder block makes
(ops/level3/llama3_decoder_layer/forward_ref.py:107); with the declaration's
``reference_dtype="float32"`` the oracle runs it on float32 copies of q, k, v.
"""

import torch


def causal_attention_forward_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """softmax(scale * q k^T + causal mask) v over [B, H, S, D], scale = D**-0.5."""
    if q.ndim != 4:
        raise ValueError(f"expected 4D q [B, H, S, D], got {tuple(q.shape)}")
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)
