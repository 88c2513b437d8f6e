"""Llama-3 decoder layer autograd pair: the composition either side of the hot
path, built from this package's kernels (RMSNorm, RoPE, grouped-query causal
attention, SwiGLU) with the projections as plain library GEMMs (cuBLAS through
``torch``), residual adds folded into the GEMM epilogues (``addmm``).

    x -> RMSNorm -> Q/K/V proj -> RoPE -> causal GQA -> O proj -> +x
      -> RMSNorm -> SwiGLU MLP -> +residual
    (src/evograd/ops/level3/llama3_decoder_layer/forward_ref.py:53-117)

Saved state: the two float32 rstd vectors, the rotated q/k and v in the
attention layout, the attention output with its float32 log-sum-exp, the
post-attention residual stream and the gate/up activations. Both normalised
activations, the SwiGLU product and the head-major copies are recomputed in the
backward. RoPE reads the projection output through a transposed view and
writes the attention layout directly (and the reverse in the backward), so no
separate transpose pass exists for q and k; the attention kernels read v and the
upstream gradient of o and write o and dv token-major ([B, T, H, hd]), which
is how the projections around them produce and consume them: no transposing
copies at all.
dK/dV are summed over each query group inside the attention kernel.

Candidate module for evograd's gate and benchmarks (``evograd verify --op
llama3_decoder_layer <this file>``): exports
``llama3_decoder_layer_forward_with_saved`` / ``..._backward_from_saved`` with the
signatures the declaration derives (.../llama3_decoder_layer/__init__.py:137-222).
"""

import os
import sys

import torch

# evograd imports candidates by file path, so the package root may be absent
# from sys.path.
_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if _ROOT not in sys.path:
    sys.path.insert(0, _ROOT)

from evograd_b200 import ops  # noqa: E402


# EVOLVE-BLOCK-START
def _heads_first(t2d, B, T, H, hd):
    """[B*T, H*hd] projection output viewed as [B, H, T, hd] (strided, no copy)."""
    return t2d.view(B, T, H, hd).transpose(1, 2)


def _forward_with_saved_impl(x, input_norm_weight, q_weight, k_weight, v_weight, o_weight,
                             post_norm_weight, gate_weight, up_weight, down_weight, cos, sin,
                             eps=1e-5):
    B, T, hidden = x.shape
    hd = cos.shape[-1]
    Hq, Hkv = q_weight.shape[0] // hd, k_weight.shape[0] // hd
    if q_weight.shape[0] % hd or k_weight.shape[0] % hd or Hq % Hkv:
        raise ValueError("q_out and kv_out must be multiples of head_dim, and Hq of Hkv")
    x2 = x.reshape(B * T, hidden)
    h, rstd1 = ops.rmsnorm_fwd(x2, input_norm_weight, eps)
    q = torch.mm(h, q_weight.t())
    k = torch.mm(h, k_weight.t())
    v = torch.mm(h, v_weight.t())
    qr = ops.rope_fwd(_heads_first(q, B, T, Hq, hd), cos, sin, layout="bhtd")
    kr = ops.rope_fwd(_heads_first(k, B, T, Hkv, hd), cos, sin, layout="bhtd")
    vv = v.view(B, T, Hkv, hd)  # token-major, as the projection wrote it
    o, lse = ops.causal_gqa_attention_fwd_tm(qr, kr, vv)  # o is [B, T, Hq, hd] as well
    attn = o.view(B * T, Hq * hd)
    x1 = torch.addmm(x2, attn, o_weight.t())            # residual add in the GEMM epilogue
    h2, rstd2 = ops.rmsnorm_fwd(x1, post_norm_weight, eps)
    gate = torch.mm(h2, gate_weight.t())
    up = torch.mm(h2, up_weight.t())
    act = ops.swiglu_fwd(gate, up)
    out = torch.addmm(x1, act, down_weight.t())
    saved = (x2, input_norm_weight, q_weight, k_weight, v_weight, o_weight, post_norm_weight,
             gate_weight, up_weight, down_weight, cos, sin, rstd1, qr, kr, vv, o, lse, x1, rstd2,
             gate, up)
    return out.view(B, T, hidden), saved


def _backward_from_saved_impl(dout, saved_tensors, eps=1e-5):
    (x2, w_in, Wq, Wk, Wv, Wo, w_post, Wg, Wu, Wd, cos, sin, rstd1, qr, kr, vv, o, lse, x1, rstd2,
     gate, up) = saved_tensors
    B, Hq, T, hd = qr.shape
    Hkv = kr.shape[1]
    hidden = x2.shape[1]
    g = dout.reshape(B * T, hidden)

    # MLP
    act = ops.swiglu_fwd(gate, up)
    d_down = torch.mm(g.t(), act)
    d_act = torch.mm(g, Wd)
    d_gate, d_up = ops.swiglu_bwd(d_act, gate, up)
    h2, _ = ops.rmsnorm_fwd(x1, w_post, eps)
    d_gate_w = torch.mm(d_gate.t(), h2)
    d_up_w = torch.mm(d_up.t(), h2)
    d_h2 = torch.addmm(torch.mm(d_gate, Wg), d_up, Wu)
    d_x1n, d_w_post = ops.rmsnorm_bwd(d_h2, x1, w_post, rstd2)
    d_x1 = g + d_x1n

    # attention
    attn = o.view(B * T, Hq * hd)
    d_o_w = torch.mm(d_x1.t(), attn)
    d_attn = torch.mm(d_x1, Wo).view(B, T, Hq, hd)
    dq, dk, dv = ops.causal_gqa_attention_bwd_tm(d_attn, qr, kr, vv, o, lse)  # dv [B, T, Hkv, hd]
    dq2 = torch.empty(B, T, Hq, hd, device=dq.device, dtype=dq.dtype)
    dk2 = torch.empty(B, T, Hkv, hd, device=dk.device, dtype=dk.dtype)
    ops.rope_bwd(dq, cos, sin, layout="bhtd", out=dq2.transpose(1, 2))
    ops.rope_bwd(dk, cos, sin, layout="bhtd", out=dk2.transpose(1, 2))
    dq2 = dq2.view(B * T, Hq * hd)
    dk2 = dk2.view(B * T, Hkv * hd)
    dv2 = dv.view(B * T, Hkv * hd)
    h, _ = ops.rmsnorm_fwd(x2, w_in, eps)
    d_q_w = torch.mm(dq2.t(), h)
    d_k_w = torch.mm(dk2.t(), h)
    d_v_w = torch.mm(dv2.t(), h)
    d_h = torch.addmm(torch.addmm(torch.mm(dq2, Wq), dk2, Wk), dv2, Wv)
    d_xn, d_w_in = ops.rmsnorm_bwd(d_h, x2, w_in, rstd1)
    dx = (d_x1 + d_xn).view(B, T, hidden)
    return dx, d_w_in, d_q_w, d_k_w, d_v_w, d_o_w, d_w_post, d_gate_w, d_up_w, d_down
# EVOLVE-BLOCK-END


def llama3_decoder_layer_forward_with_saved(x, input_norm_weight, q_weight, k_weight, v_weight,
                                            o_weight, post_norm_weight, gate_weight, up_weight,
                                            down_weight, cos, sin, eps=1e-5):
    return _forward_with_saved_impl(x, input_norm_weight, q_weight, k_weight, v_weight, o_weight,
                                    post_norm_weight, gate_weight, up_weight, down_weight, cos,
                                    sin, eps)


def llama3_decoder_layer_backward_from_saved(dout, saved_tensors, eps=1e-5):
    return _backward_from_saved_impl(dout, saved_tensors, eps)
