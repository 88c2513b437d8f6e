"""External evograd declarations for the B200 build (needs ``evograd`` importable).

Load with ``--declaration evograd_b200/decls/b200_decls.py:<attribute>`` or the
``EVOGRAD_DECLARATION`` environment variable (src/evograd/ops/__init__.py:68-99;
the attribute's ``name`` must equal ``--op``).

Attributes
    causal_attention  a NEW operator: the reference declares no standalone causal
                      attention (only ``evoattention`` and SDPA inside its decoder
                      block). Layout [B, H, S, D], trusted forward =
                      ``F.scaled_dot_product_attention(..., is_causal=True)`` as
                      at ops/level3/llama3_decoder_layer/forward_ref.py:107,
                      float32 reference dtype.
    softmax, layernorm, rmsnorm, swiglu, rope, geglu, fused_add_rms_norm
                      the built-in declarations with one extra named benchmark
                      suite ``"b200"`` holding the baseline configuration's exact
                      shape/dtype (and, where the input recipe differs from the
                      built-in hook, its own ``make_inputs``). Everything else,
                      including the correctness gate, is the reference's.
"""

from __future__ import annotations

import dataclasses

from evograd.opdecl import Active, Provenance, Workload, declare_op
from evograd.ops import get_op

_FILE = __file__


# ------------------------------------------------------------ causal attention
def causal_attention_forward_ref(q, k, v):
    import torch

    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)


def _attention_inputs(torch, op, workload, device="cuda"):
    d = workload.dims
    B, H, S, D = d["B"], d["H"], d["S"], d["D"]
    dtype = getattr(torch, workload.dtype)
    # seed pattern of ops/level1/evoattention/__init__.py:17 with its MSA axis at 1
    torch.manual_seed((((B * 131 + 1) * 131 + H) * 131 + S) * 131 + D)
    std = 1.0 if workload.dims.get("S", 0) >= 8192 else 0.5
    mk = lambda: torch.randn((B, H, S, D), device=device, dtype=dtype) * std
    return {"q": mk(), "k": mk(), "v": mk(), "do": mk()}


def _attn(B, H, S, D, dtype, **kw):
    return Workload(dims=dict(B=B, H=H, S=S, D=D), dtype=dtype, **kw)


# A level-1 declaration must say where its timed shape comes from
# (opdecl/activity.py:395-410). The reference's model registry has no
# standalone-attention component, so the origin is recorded as hand-picked.
_ATTN_BENCH = (
    _attn(4, 32, 8192, 128, "bfloat16", provenance=Provenance(
        model="llama_3_8b", component="causal_attention", free={"batch": 4, "seq": 8192},
        source="handpicked",
        note="32 query heads of width 128 as in Llama-3-8B; batch 4 x 8192 tokens fills one B200",
    )),
)

causal_attention = declare_op(
    name="causal_attention",
    level=1,
    family="attention",
    forward=f"{_FILE}:causal_attention_forward_ref",
    declaration=f"{_FILE}:causal_attention",
    dims=("B", "H", "S", "D"),
    args=(
        Active("q", "[B, H, S, D]", dtype="float16|bfloat16"),
        Active("k", "[B, H, S, D]", dtype="float16|bfloat16"),
        Active("v", "[B, H, S, D]", dtype="float16|bfloat16"),
    ),
    output=Active("o", "[B, H, S, D]"),
    forward_semantics=(
        "o = softmax(scale * q @ k^T + causal_mask) @ v with scale = D**-0.5, scores and "
        "softmax in float32, key j visible to query i iff j <= i."
    ),
    backward_semantics=(
        "Return (dq, dk, dv) in the input dtype. With P the probabilities and "
        "delta = rowsum(do*o): dv = P^T do; dS = P*(do v^T - delta); dq = scale*dS k; dk = scale*dS^T q."
    ),
    reference_dtype="float32",
    correctness=(
        _attn(1, 2, 128, 128, "bfloat16"),
        _attn(1, 2, 129, 128, "bfloat16"),
        _attn(2, 3, 384, 128, "bfloat16"),
        _attn(1, 2, 77, 128, "float16"),
        _attn(2, 2, 333, 64, "bfloat16"),
        _attn(1, 2, 1000, 128, "bfloat16"),
    ),
    benchmark=_ATTN_BENCH,
    benchmark_suites={"b200": _ATTN_BENCH},
    # o within the 16-bit gate; the gradients within 2e-2 max-abs of the float32 reference
    tolerances={"float16": (1e-2, 1.6e-2), "bfloat16": (1e-2, 1.6e-2)},
    tolerance_multipliers={"dq": (2.0, 1e-3), "dk": (2.0, 1e-3), "dv": (2.0, 1e-3)},
    make_inputs=_attention_inputs,
)


# --------------------------------------------------- b200 suites for built-ins
def _with_b200(name, workloads, make_inputs=None):
    op = get_op(name)
    suites = dict(op.benchmark_suites)
    suites["b200"] = tuple(workloads)
    changes = {"benchmark_suites": suites, "declaration": f"{_FILE}:{name}"}
    if make_inputs is not None:
        builtin = op.make_inputs
        b200_dims = [dict(w.dims) for w in workloads]

        def hook(torch, op_, workload, device="cuda"):
            if dict(workload.dims) in b200_dims:
                return make_inputs(torch, op_, workload, device)
            return builtin(torch, op_, workload, device)

        changes["make_inputs"] = hook
    return dataclasses.replace(op, **changes)


def _layernorm_b200_inputs(torch, op, workload, device="cuda"):
    rows, hidden = workload.dims["rows"], workload.dims["hidden"]
    dtype = getattr(torch, workload.dtype)
    torch.manual_seed(rows * 100000 + hidden)
    x = torch.randn((rows, hidden), device=device, dtype=dtype)
    weight = (1.0 + 0.1 * torch.randn((hidden,), device=device, dtype=torch.float32)).to(dtype)
    bias = (0.1 * torch.randn((hidden,), device=device, dtype=torch.float32)).to(dtype)
    dy = torch.randn((rows, hidden), device=device, dtype=dtype)
    return {"x": x, "weight": weight, "bias": bias, "eps": 1e-5, "dy": dy}


def _rmsnorm_b200_inputs(torch, op, workload, device="cuda"):
    rows, hidden = workload.dims["rows"], workload.dims["hidden"]
    dtype = getattr(torch, workload.dtype)
    torch.manual_seed(rows * 100000 + hidden)
    x = torch.randn((rows, hidden), device=device, dtype=dtype)
    weight = (1.0 + 0.1 * torch.randn((hidden,), device=device, dtype=torch.float32)).to(dtype)
    dy = torch.randn((rows, hidden), device=device, dtype=dtype)
    return {"x": x, "weight": weight, "eps": 1e-6, "dy": dy}


softmax = _with_b200("softmax", [Workload(dims=dict(rows=4096, cols=1024), dtype="float32")])
layernorm = _with_b200(
    "layernorm", [Workload(dims=dict(rows=16384, hidden=4096), dtype="bfloat16")],
    _layernorm_b200_inputs,
)
rmsnorm = _with_b200(
    "rmsnorm", [Workload(dims=dict(rows=32768, hidden=4096), dtype="bfloat16")],
    _rmsnorm_b200_inputs,
)
swiglu = _with_b200("swiglu", [Workload(dims=dict(rows=32768, cols=14336), dtype="bfloat16")])
geglu = _with_b200("geglu", [Workload(dims=dict(rows=32768, cols=14336), dtype="bfloat16")])
fused_add_rms_norm = _with_b200(
    "fused_add_rms_norm", [Workload(dims=dict(rows=32768, cols=4096), dtype="bfloat16")]
)
# The reference layout is [B, heads, T, head_dim] with one tensor per call; the
# [B, S, H, D] q-and-k form of the baseline config is served by
# evograd_b200.ops.rope_qk_fwd / rope_qk_bwd and timed by bench.py.
rope = _with_b200(
    "rope", [Workload(dims=dict(B=8, n_heads=32, T=4096, head_dim=128), dtype="bfloat16")]
)
