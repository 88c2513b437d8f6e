"""Operator declaration: causal_attention (drop-in package for an evograd checkout).

Copy this directory to ``src/evograd/ops/level1/causal_attention/`` of an evograd
tree: ``evograd.ops._discover_ops`` (ops/__init__.py:29-65) then registers the
operator as a built-in (the package exposes the ``OpDecl`` as ``op`` and its name
equals the package name), so ``evograd verify`` / ``bench`` / ``suite`` find it
without ``--declaration``. Nothing here imports the B200 kernels: the declaration
is the contract, the candidate is ``evograd_b200/pairs/causal_attention.py``.

The same declaration in external form (``--declaration file.py:causal_attention``)
lives in ``evograd_b200/decls/b200_decls.py``.
"""

from evograd.opdecl import Active, Provenance, Workload, declare_op


def make_causal_attention_inputs(torch, op, workload, device="cuda"):
    d = workload.dims
    b, h, s, dim = d["B"], d["H"], d["S"], d["D"]
    dtype = getattr(torch, workload.dtype)
    # seed pattern of ops/level1/evoattention/__init__.py:17 with its MSA axis at 1
    torch.manual_seed((((b * 131 + 1) * 131 + h) * 131 + s) * 131 + dim)
    std = 1.0 if s >= 8192 else 0.5

    def draw():
        return torch.randn((b, h, s, dim), device=device, dtype=dtype) * std

    return {"q": draw(), "k": draw(), "v": draw(), "do": draw()}


def _case(b, h, s, d, dtype, **kw):
    return Workload(dims=dict(B=b, H=h, S=s, D=d), dtype=dtype, **kw)


# A level-1 declaration says where its timed shape comes from
# (opdecl/activity.py:395-410); the model registry has no standalone-attention
# component, so the origin is recorded as hand-picked.
_BENCHMARK = (
    _case(4, 32, 8192, 128, "bfloat16", provenance=Provenance(
        model="llama_3_8b", component="causal_attention", free={"batch": 4, "seq": 8192},
        source="handpicked",
        note="32 query heads of width 128 as in Llama-3-8B; batch 4 x 8192 tokens fills one B200",
    )),
)

op = declare_op(
    name="causal_attention",
    level=1,
    family="attention",
    forward="evograd.ops.level1.causal_attention.forward_ref:causal_attention_forward_ref",
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
        _case(1, 2, 128, 128, "bfloat16"),
        _case(1, 2, 129, 128, "bfloat16"),
        _case(2, 3, 384, 128, "bfloat16"),
        _case(1, 2, 77, 128, "float16"),
        _case(2, 2, 333, 64, "bfloat16"),
        _case(1, 2, 1000, 128, "bfloat16"),
    ),
    benchmark=_BENCHMARK,
    benchmark_suites={"b200": _BENCHMARK},
    # o within the 16-bit gate; the gradients within 2e-2 max-abs of the float32 reference
    tolerances={"float16": (1e-2, 1.6e-2), "bfloat16": (1e-2, 1.6e-2)},
    tolerance_multipliers={"dq": (2.0, 1e-3), "dk": (2.0, 1e-3), "dv": (2.0, 1e-3)},
    make_inputs=make_causal_attention_inputs,
)
