"""CPU restatement of evograd's parity oracle for the six hot-path operators.

TEST INFRASTRUCTURE, NOT PRODUCT: only ``tests/``, ``__graft_entry__.smoke()``
and the CPU-baseline legs of ``bench.py`` may import this module. The shipped
path (``evograd_b200``) never does, and it has no CPU fallback.

What evograd's oracle is (citations are paths inside akumdam2/evograd):
``evograd.opdecl.oracle.oracle`` (src/evograd/opdecl/oracle.py:44-111) clones
every ``Active`` argument as an autograd leaf, optionally widens floating inputs
to the declaration's ``reference_dtype``, runs the declaration's trusted forward
and takes ``torch.autograd.grad(y, leaves, grad_outputs=dout)`` (oracle.py:103);
results are cast back to the input dtypes. The arithmetic itself lives in
PyTorch (a dependency the reference leaves unpinned in pyproject.toml:12-16;
2.11.0 is installed where the golden vectors were generated), so this file
restates (a) the trusted forwards, (b) the seeded input recipes, (c) the oracle
procedure and (d) the gate ``torch.allclose(a.float(), e.float(), atol, rtol)``
plus shape/dtype equality (src/evograd/opdecl/verify.py:85-115).

Pinning: ``tests/golden/*.npz`` were produced by importing the reference itself
(``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks every
function here against them. Causal attention has no declaration in the
reference; its restatement follows the reference's primitive attention spelling
(ops/level1/evoattention/forward_ref.py:36-48) and is pinned against that
function run with a causal additive bias.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

# --------------------------------------------------------------------------
# (a) trusted forwards


def softmax_forward(x):
    """ops/level1/softmax/forward_ref.py:6-7 - float32 softmax, one cast back."""
    return torch.softmax(x.float(), dim=-1).to(x.dtype)


def layernorm_forward(x, weight, bias, eps=1e-5):
    """ops/level1/layernorm/forward_ref.py:20-23 - all float32, two-pass variance."""
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(dim=-1, keepdim=True)
    x_hat = (xf - mean) * torch.rsqrt(var + eps)
    return (x_hat * weight.float() + bias.float()).to(x.dtype)


def rmsnorm_forward(x, weight, eps=1e-5):
    """ops/level1/rmsnorm/forward_ref.py:19-21 - mean of squares in float32."""
    xf = x.float()
    ms = (xf * xf).mean(dim=-1, keepdim=True)
    x_hat = xf * torch.rsqrt(ms + eps)
    return (x_hat * weight.float()).to(x.dtype)


def swiglu_forward(a, b):
    """ops/level1/swiglu/forward_ref.py:6-9 - silu in float32, ROUNDED to the
    input dtype, then multiplied by b in the input dtype."""
    return torch.nn.functional.silu(a.float()).to(a.dtype) * b


def geglu_forward(a, b):
    """ops/level1/geglu/forward_ref.py:6-9 - tanh-approximate gelu in float32,
    ROUNDED to the input dtype, then multiplied by b in the input dtype."""
    return torch.nn.functional.gelu(a.float(), approximate="tanh").to(a.dtype) * b


def fused_add_rms_norm_forward(x, residual, weight, eps=1e-6):
    """ops/level2/fused_add_rms_norm/forward_ref.py:6-14 - the sum is taken in the
    input dtype; rstd is float32 but cast to the input dtype before it multiplies
    the sum; both products are taken in the input dtype."""
    summed = x + residual
    rstd = torch.rsqrt(summed.float().pow(2).mean(dim=-1, keepdim=True) + eps)
    return (summed * rstd.to(summed.dtype)) * weight


def rope_forward(x, cos, sin):
    """ops/level1/rope/forward_ref.py:28-47 - x is [batch, heads, tokens, head_dim];
    rotate_half(x) = cat(-x2, x1); float32 products and sum, one cast back."""
    half = x.shape[-1] // 2
    xf = x.float()
    rot = torch.cat((-xf[..., half:], xf[..., :half]), dim=-1)
    return (xf * cos[None, None].float() + rot * sin[None, None].float()).to(x.dtype)


def causal_attention_forward(q, k, v):
    """Primitive spelling of ops/level1/evoattention/forward_ref.py:36-48 with the
    additive bias replaced by the causal mask: q is scaled by D**-0.5 in the
    input dtype, scores and softmax are float32, probabilities are cast to the
    input dtype before the product with v. q, k, v are [B, H, S, D]."""
    S, D = q.shape[-2], q.shape[-1]
    scale = D ** -0.5
    scores = torch.matmul(q * scale, k.transpose(-1, -2))
    mask = torch.full((S, S), float("-inf"), dtype=torch.float32, device=q.device).triu(1)
    scores = scores + mask
    probs = torch.softmax(scores.float(), dim=-1).to(q.dtype)
    return torch.matmul(probs, v)


def causal_attention_forward_sdpa(q, k, v):
    """The fused spelling the reference uses inside its decoder block
    (ops/level3/llama3_decoder_layer/forward_ref.py:107); linear memory, so it is
    the one that can run at full sequence length on the host."""
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)


def evoattention_forward(q, k, v, res_mask, pair_bias):
    """ops/level1/evoattention/forward_ref.py:22-49. q, k, v are
    [B, N_seq, N_res, Head, Dim]; res_mask [B, N_seq, 1, 1, N_res] additive;
    pair_bias [B, 1, Head, N_res, N_res]. q is scaled by Dim**-0.5 in the input
    dtype, the scores get bias and mask, the softmax runs in float32 over the key
    residue axis and is cast to the input dtype before the product with v."""
    dtype = q.dtype
    scale = q.shape[-1] ** -0.5
    q_t, k_t, v_t = (t.transpose(-2, -3) for t in (q, k, v))
    scores = torch.matmul(q_t * scale, k_t.transpose(-1, -2))
    scores = scores + pair_bias + res_mask
    probs = torch.softmax(scores.float(), dim=-1).to(dtype)
    return torch.matmul(probs, v_t).transpose(-2, -3).contiguous()


def causal_gqa_attention_forward(q, k, v):
    """Grouped-query causal attention as the decoder block spells it
    (ops/level3/llama3_decoder_layer/forward_ref.py:100-107): each k/v head is
    repeated across its query group, then scaled_dot_product_attention.
    q is [B, Hq, S, D]; k, v are [B, Hkv, S, D]."""
    repeat = q.shape[1] // k.shape[1]
    if repeat > 1:
        k = k.repeat_interleave(repeat, dim=1)
        v = v.repeat_interleave(repeat, dim=1)
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True)


def llama3_decoder_layer_forward(x, input_norm_weight, q_weight, k_weight, v_weight, o_weight,
                                 post_norm_weight, gate_weight, up_weight, down_weight, cos, sin,
                                 eps=1e-5):
    """One Llama-3 decoder layer, ops/level3/llama3_decoder_layer/forward_ref.py:53-117:
    RMSNorm (float32 statistics, normalised value cast to the input dtype, then
    the gain) -> q/k/v projections (weights [out, in]) -> rotate-half RoPE in
    float32 -> grouped-query causal SDPA -> o projection + residual -> RMSNorm
    -> silu(gate.float()) * up.float() cast back -> down projection + residual.
    Head counts come from the weight shapes and cos.shape[-1]."""
    F = torch.nn.functional

    def rms_norm(t, w):  # forward_ref.py:33-37
        t32 = t.float()
        rrms = torch.rsqrt(t32.pow(2).mean(-1, keepdim=True) + eps)
        return (t32 * rrms).to(t.dtype) * w

    def rope(t):  # forward_ref.py:40-50
        half = t.shape[-1] // 2
        t32 = t.float()
        rot = torch.cat((-t32[..., half:], t32[..., :half]), dim=-1)
        return (t32 * cos[None, None].float() + rot * sin[None, None].float()).to(t.dtype)

    batch, tokens, _hidden = x.shape
    head_dim = cos.shape[-1]
    n_heads, n_kv = q_weight.shape[0] // head_dim, k_weight.shape[0] // head_dim
    h = rms_norm(x, input_norm_weight)
    q = F.linear(h, q_weight).view(batch, tokens, n_heads, head_dim).transpose(1, 2)
    k = F.linear(h, k_weight).view(batch, tokens, n_kv, head_dim).transpose(1, 2)
    v = F.linear(h, v_weight).view(batch, tokens, n_kv, head_dim).transpose(1, 2)
    attn = causal_gqa_attention_forward(rope(q), rope(k), v)
    attn = attn.transpose(1, 2).reshape(batch, tokens, n_heads * head_dim)
    x = x + F.linear(attn, o_weight)
    h = rms_norm(x, post_norm_weight)
    act = (F.silu(F.linear(h, gate_weight).float()) * F.linear(h, up_weight).float()).to(h.dtype)
    return x + F.linear(act, down_weight)


# --------------------------------------------------------------------------
# declarations (only what the oracle needs from opdecl/activity.py:179-337)

STANDARD_TOLERANCES = {  # ops/_common.py:13-17, (atol, rtol)
    "float32": (2e-5, 2e-5),
    "float16": (5e-2, 5e-2),
    "bfloat16": (8e-2, 8e-2),
}
# The tighter figures the build is held to: float32 exact-ish, 16-bit types
# against a float32-promoted oracle; attention gradients 2e-2 max-abs.
STRICT_TOLERANCES = {
    "float32": (1e-5, 1e-5),
    "float16": (1e-2, 1.6e-2),
    "bfloat16": (1e-2, 1.6e-2),
}


@dataclass(frozen=True)
class OpSpec:
    name: str
    forward: object
    args: tuple  # (name, active) in declaration order; scalars listed in `scalars`
    output: str
    scalars: dict = field(default_factory=dict)
    dims: tuple = ()
    tolerances: dict = field(default_factory=lambda: dict(STANDARD_TOLERANCES))
    row_scaled_grads: tuple = ()  # bf16 atol grows as sqrt(rows/8) for these
    tolerance_hook: object = None  # (dims, dtype, result, atol, rtol) -> (atol, rtol)
    # Results whose same-dtype reference value itself misses the strict figures
    # against the float32-promoted oracle (the trusted forward rounds inside the
    # reduction's inputs); they keep the declared tolerance in strict mode.
    strict_exempt: tuple = ()
    grad_overrides: dict = field(default_factory=dict)  # input name -> gradient name (Active(grad=...))

    def grad_name(self, arg: str) -> str:  # activity.py:43-45
        return self.grad_overrides.get(arg, "d" + arg)

    def strict_tolerance_for(self, dims: dict, dtype: str, result: str | None = None):
        if dtype != "float32" and result in self.strict_exempt:
            return self.tolerance_for(dims, dtype, result)
        return STRICT_TOLERANCES[dtype]

    @property
    def upstream(self) -> str:  # "d" + output name, activity.py:43-45
        return "d" + self.output

    def grad_names(self) -> tuple:
        return tuple(self.grad_name(n) for n, active in self.args if active)

    def tolerance_for(self, dims: dict, dtype: str, result: str | None = None):
        """(atol, rtol) as OpDecl.tolerance_for (activity.py:517-528) with the
        layernorm/rmsnorm hooks (layernorm/__init__.py:95-100, rmsnorm/__init__.py:39-49)."""
        atol, rtol = self.tolerances[dtype]
        if dtype == "bfloat16" and result in self.row_scaled_grads:
            atol = max(atol, atol * math.sqrt(max(1.0, dims["rows"] / 8.0)))
        if self.tolerance_hook is not None:
            atol, rtol = self.tolerance_hook(dims, dtype, result, atol, rtol)
        return float(atol), float(rtol)


def _fused_add_rms_norm_tolerance(dims, dtype, result, atol, rtol):
    """ops/level2/fused_add_rms_norm/__init__.py:42-52: dweight is a reduction
    over rows, its atol is 2e-3 / 2e-1 / 2e-1 (fp32 / fp16 / bf16) times
    sqrt(rows/64) once rows exceed 64."""
    if result == "dweight":
        base = {"float32": 2e-3, "float16": 2e-1, "bfloat16": 2e-1}.get(dtype, atol)
        atol = base * max(1.0, math.sqrt(dims["rows"] / 64.0))
    return atol, rtol


def _decoder_layer_tolerance(dims, dtype, result, atol, rtol):
    """ops/level3/llama3_decoder_layer/__init__.py:228-233: the three longest
    reductions get 1.5x the atol."""
    if result in ("dk_weight", "dv_weight", "ddown_weight"):
        atol = atol * 1.5
    return atol, rtol


OPS = {
    "softmax": OpSpec("softmax", softmax_forward, (("x", True),), "y", dims=("rows", "cols")),
    "layernorm": OpSpec(
        "layernorm", layernorm_forward, (("x", True), ("weight", True), ("bias", True)), "y",
        scalars={"eps": 1e-5}, dims=("rows", "hidden"), row_scaled_grads=("dweight", "dbias"),
    ),
    "rmsnorm": OpSpec(
        "rmsnorm", rmsnorm_forward, (("x", True), ("weight", True)), "y",
        scalars={"eps": 1e-5}, dims=("rows", "hidden"), row_scaled_grads=("dweight",),
    ),
    "swiglu": OpSpec("swiglu", swiglu_forward, (("a", True), ("b", True)), "c",
                     dims=("rows", "cols")),
    "geglu": OpSpec("geglu", geglu_forward, (("a", True), ("b", True)), "c",
                    dims=("rows", "cols")),
    "fused_add_rms_norm": OpSpec(
        "fused_add_rms_norm", fused_add_rms_norm_forward,
        (("x", True), ("r", True), ("weight", True)), "out",
        scalars={"eps": 1e-6}, dims=("rows", "cols"),
        tolerance_hook=_fused_add_rms_norm_tolerance, strict_exempt=("dweight",),
    ),
    # reference_dtype is float32 in the declaration: always check this operator
    # with oracle(..., reference_dtype=torch.float32).
    "llama3_decoder_layer": OpSpec(
        "llama3_decoder_layer", llama3_decoder_layer_forward,
        (("x", True), ("input_norm_weight", True), ("q_weight", True), ("k_weight", True),
         ("v_weight", True), ("o_weight", True), ("post_norm_weight", True), ("gate_weight", True),
         ("up_weight", True), ("down_weight", True), ("cos", False), ("sin", False)), "out",
        scalars={"eps": 1e-5},
        dims=("B", "T", "hidden", "head_dim", "q_out", "kv_out", "intermediate"),
        tolerances={"float32": (1e-4, 1e-4), "bfloat16": (5e-2, 2e-2)},
        tolerance_hook=_decoder_layer_tolerance,
    ),
    "evoattention": OpSpec(
        "evoattention", evoattention_forward,
        (("q", True), ("k", True), ("v", True), ("res_mask", False), ("pair_bias", True)), "o",
        dims=("B", "S", "H", "N", "D"),
        tolerances={"float16": (2e-2, 2e-2), "bfloat16": (4e-2, 4e-2)},  # evoattention/__init__.py
        tolerance_hook=lambda dims, dtype, result, atol, rtol:
            (atol * 2.0, rtol) if result == "d_pair_bias" else (atol, rtol),
        grad_overrides={"pair_bias": "d_pair_bias"},
    ),
    "rope": OpSpec("rope", rope_forward, (("x", True), ("cos", False), ("sin", False)), "y",
                   dims=("B", "n_heads", "T", "head_dim")),
    "causal_attention": OpSpec(
        "causal_attention", causal_attention_forward, (("q", True), ("k", True), ("v", True)), "o",
        dims=("B", "H", "S", "D"),
        tolerances={"float16": (2e-2, 2e-2), "bfloat16": (4e-2, 4e-2)},  # evoattention/__init__.py
    ),
}

# --------------------------------------------------------------------------
# (b) seeded input recipes


def _dt(name: str) -> torch.dtype:
    return getattr(torch, name)


def make_inputs(op: str, dims: dict, dtype: str, device: str = "cpu") -> dict:
    """The per-operator ``make_inputs`` hooks of the reference, same seeds and
    the same order of random draws, so CPU inputs are bit-identical to the
    reference's for a given torch version."""
    dt = _dt(dtype)
    if op == "softmax":  # softmax/__init__.py:44-51
        r, c = dims["rows"], dims["cols"]
        torch.manual_seed(r * 100003 + c)
        return {"x": torch.randn((r, c), device=device, dtype=dt),
                "dy": torch.randn((r, c), device=device, dtype=dt)}
    if op == "layernorm":  # layernorm/__init__.py:16-24
        r, h = dims["rows"], dims["hidden"]
        torch.manual_seed(r * 100000 + h)
        x = torch.randn((r, h), device=device, dtype=dt)
        w = torch.randn((h,), device=device, dtype=dt)
        b = torch.randn((h,), device=device, dtype=dt)
        dy = torch.randn((r, h), device=device, dtype=dt)
        return {"x": x, "weight": w, "bias": b, "eps": 1e-5, "dy": dy}
    if op == "rmsnorm":  # rmsnorm/__init__.py:20-32
        r, h = dims["rows"], dims["hidden"]
        torch.manual_seed(r * 100000 + h)
        x = torch.randn((r, h), device=device, dtype=dt)
        w = (1.0 + 0.1 * torch.randn((h,), device=device, dtype=torch.float32)).to(dt)
        dy = torch.randn((r, h), device=device, dtype=dt)
        return {"x": x, "weight": w, "eps": 1e-5, "dy": dy}
    if op == "swiglu":  # swiglu/__init__.py:44-52
        r, c = dims["rows"], dims["cols"]
        torch.manual_seed(r * 100003 + c)
        return {"a": torch.randn((r, c), device=device, dtype=dt),
                "b": torch.randn((r, c), device=device, dtype=dt),
                "dc": torch.randn((r, c), device=device, dtype=dt)}
    if op == "geglu":  # geglu/__init__.py:40-48
        r, c = dims["rows"], dims["cols"]
        torch.manual_seed(r * 100003 + c)
        return {"a": torch.randn((r, c), device=device, dtype=dt),
                "b": torch.randn((r, c), device=device, dtype=dt),
                "dc": torch.randn((r, c), device=device, dtype=dt)}
    if op == "fused_add_rms_norm":  # fused_add_rms_norm/__init__.py:55-66
        r, c = dims["rows"], dims["cols"]
        torch.manual_seed(r * 100003 + c)
        return {"x": torch.randn((r, c), device=device, dtype=dt),
                "r": torch.randn((r, c), device=device, dtype=dt),
                "weight": torch.randn((c,), device=device, dtype=dt),
                "eps": 1e-6,
                "dout": torch.randn((r, c), device=device, dtype=dt)}
    if op == "llama3_decoder_layer":  # llama3_decoder_layer/__init__.py:64-135
        B, T, hidden = dims["B"], dims["T"], dims["hidden"]
        hd, q_out, kv_out, inter = dims["head_dim"], dims["q_out"], dims["kv_out"], dims["intermediate"]
        if q_out % hd or kv_out % hd or (q_out // hd) % (kv_out // hd) or q_out != hidden:
            raise ValueError("inconsistent decoder-layer dimensions")
        torch.manual_seed(T * 100003 + hidden * 1009 + hd)

        def weight(o_f, i_f):  # fan-in scaling
            return (torch.randn((o_f, i_f), device=device, dtype=torch.float32) * i_f ** -0.5).to(dt)

        def gain(width):
            return (1.0 + 0.1 * torch.randn((width,), device=device, dtype=torch.float32)).to(dt)

        positions = torch.arange(T, device=device, dtype=torch.float32)[:, None]
        inv_freq = 500000.0 ** (-torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd)
        angles = torch.cat((positions * inv_freq[None, :],) * 2, dim=-1)
        # dict order = order of the random draws in the reference
        return {
            "x": torch.randn((B, T, hidden), device=device, dtype=dt) * 0.5,
            "input_norm_weight": gain(hidden),
            "q_weight": weight(q_out, hidden),
            "k_weight": weight(kv_out, hidden),
            "v_weight": weight(kv_out, hidden),
            "o_weight": weight(hidden, q_out),
            "post_norm_weight": gain(hidden),
            "gate_weight": weight(inter, hidden),
            "up_weight": weight(inter, hidden),
            "down_weight": weight(hidden, inter),
            "cos": angles.cos().to(dt),
            "sin": angles.sin().to(dt),
            "eps": 1e-5,
            "dout": torch.randn((B, T, hidden), device=device, dtype=dt) * 0.5 * (B * T) ** -0.5,
        }
    if op == "evoattention":  # evoattention/__init__.py:7-32
        b, sq, h, n, dim = dims["B"], dims["S"], dims["H"], dims["N"], dims["D"]
        torch.manual_seed((((b * 131 + sq) * 131 + h) * 131 + n) * 131 + dim)
        q, k, v, do = (torch.randn((b, sq, n, h, dim), device=device, dtype=dt) * 0.5
                       for _ in range(4))
        keep = torch.rand((b, sq, 1, 1, n), device=device) > 0.5
        keep[..., 0] = True  # key 0 is always kept: no query row is fully masked
        res_mask = torch.where(keep, torch.zeros((), device=device, dtype=torch.float32),
                               torch.full((), -1e9, device=device, dtype=torch.float32))
        pair_bias = torch.randn((b, 1, h, n, n), device=device, dtype=torch.float32) * 0.5
        return {"q": q, "k": k, "v": v, "res_mask": res_mask, "pair_bias": pair_bias, "do": do}
    if op == "rope":  # rope/__init__.py:30-62, theta = 500000 (models.py:259-261)
        B, H, T, D = dims["B"], dims["n_heads"], dims["T"], dims["head_dim"]
        if D % 2:
            raise ValueError(f"rope needs an even head_dim, got {D}")
        torch.manual_seed(T * 100003 + H * 1009 + D)
        x = torch.randn((B, H, T, D), device=device, dtype=dt) * 0.5
        cos, sin = rope_tables(T, D, theta=500000.0, device=device, dtype=dt, duplicate=True)
        dy = torch.randn((B, H, T, D), device=device, dtype=dt) * 0.5
        return {"x": x, "cos": cos, "sin": sin, "dy": dy}
    if op == "causal_attention":
        # No reference declaration: seed and 0.5 scaling follow the evoattention
        # recipe (evoattention/__init__.py:17-23) with its MSA axis fixed at 1.
        B, H, S, D = dims["B"], dims["H"], dims["S"], dims["D"]
        torch.manual_seed((((B * 131 + 1) * 131 + H) * 131 + S) * 131 + D)
        shape = (B, 1, S, H, D)  # the reference's [B, N_seq, N_res, Head, Dim] layout
        q, k, v, do = (torch.randn(shape, device=device, dtype=dt) * 0.5 for _ in range(4))
        to_bhsd = lambda t: t[:, 0].permute(0, 2, 1, 3).contiguous()
        return {"q": to_bhsd(q), "k": to_bhsd(k), "v": to_bhsd(v), "do": to_bhsd(do)}
    raise KeyError(op)


def rope_tables(tokens, head_dim, *, theta, device="cpu", dtype=torch.float32, duplicate=True):
    """cos/sin tables as rope/__init__.py:51-60 builds them: float32 angles
    position * theta**(-2i/head_dim), halves duplicated, cast to ``dtype``."""
    positions = torch.arange(tokens, device=device, dtype=torch.float32)[:, None]
    inv_freq = theta ** (-torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim)
    freqs = positions * inv_freq[None, :]
    angles = torch.cat((freqs, freqs), dim=-1) if duplicate else freqs
    return angles.cos().to(dtype), angles.sin().to(dtype)


# --------------------------------------------------------------------------
# (c) the oracle procedure


def oracle(op: str | OpSpec, inputs: dict, dout=None, *, reference_dtype=None, forward=None):
    """``(y, grads)`` exactly as opdecl/oracle.py:44-111 derives them.

    ``reference_dtype=torch.float32`` widens every floating input first and
    casts results back (oracle.py:70-110), which is how the stricter tolerances
    are checked; ``None`` is the same-dtype oracle the declared gate uses.
    """
    spec = OPS[op] if isinstance(op, str) else op
    fwd = forward or spec.forward
    positional, leaves, out_dtypes = [], [], {}
    for name, active in spec.args:
        value = inputs[name]
        if active:
            out_dtypes[spec.grad_name(name)] = value.dtype
            if reference_dtype is not None:
                value = value.to(reference_dtype)
            value = value.detach().clone().requires_grad_(True)
            leaves.append((spec.grad_name(name), value))
        elif reference_dtype is not None and torch.is_tensor(value) and value.is_floating_point():
            value = value.to(reference_dtype)
        positional.append(value)
    for name, default in spec.scalars.items():
        positional.append(inputs.get(name, default))
    y = fwd(*positional)
    if dout is None:
        dout = inputs[spec.upstream]
    y_dtype = dout.dtype
    if reference_dtype is not None:
        dout = dout.to(reference_dtype)
    grads = torch.autograd.grad(y, [t for _, t in leaves], grad_outputs=dout)
    by_name = {name: g for (name, _), g in zip(leaves, grads)}
    if reference_dtype is not None:
        y = y.to(y_dtype)
        by_name = {n: g.to(out_dtypes[n]) for n, g in by_name.items()}
    return y.detach(), {n: by_name[n].detach() for n in spec.grad_names()}


# --------------------------------------------------------------------------
# (d) the gate


@dataclass(frozen=True)
class Check:
    name: str
    ok: bool
    max_abs_err: float
    atol: float
    rtol: float
    detail: str = ""


def check(name, actual, expected, atol, rtol) -> Check:
    """opdecl/verify.py:85-115: same shape, same dtype, allclose in float32."""
    if not torch.is_tensor(actual):
        return Check(name, False, float("inf"), atol, rtol, f"not a tensor: {type(actual).__name__}")
    same_shape = tuple(actual.shape) == tuple(expected.shape)
    same_dtype = actual.dtype == expected.dtype
    if same_shape:
        a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
        err = (a - e).abs().max().item() if a.numel() else 0.0
        values_ok = torch.allclose(a, e, atol=atol, rtol=rtol)
    else:
        err, values_ok = float("inf"), False
    detail = ""
    if not same_shape:
        detail = f"shape {tuple(actual.shape)} != {tuple(expected.shape)}"
    elif not same_dtype:
        detail = f"dtype {actual.dtype} != {expected.dtype}"
    return Check(name, bool(same_shape and same_dtype and values_ok), err, atol, rtol, detail)


def verify_pair(op: str, module, inputs: dict, dims: dict, dtype: str, *, strict=False,
                reference_dtype=None):
    """opdecl/verify.py:118-143 for one case: run the candidate module's pair on
    ``inputs`` (on whatever device they live on) and compare with the oracle run
    on CPU copies. Returns a list of :class:`Check`."""
    spec = OPS[op]
    fwd = getattr(module, f"{op}_forward_with_saved", None) or getattr(module, "forward_with_saved")
    bwd = getattr(module, f"{op}_backward_from_saved", None) or getattr(module, "backward_from_saved")
    cpu_inputs = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in inputs.items()}
    y_ref, g_ref = oracle(spec, cpu_inputs, reference_dtype=reference_dtype)
    positional = [inputs[n] for n, _ in spec.args] + [inputs.get(n, d) for n, d in spec.scalars.items()]
    y, saved = fwd(*positional)
    import inspect

    params = inspect.signature(bwd).parameters
    kwargs = {n: inputs.get(n, d) for n, d in spec.scalars.items() if n in params}
    grads = bwd(inputs[spec.upstream], saved, **kwargs)
    grads = (grads,) if torch.is_tensor(grads) else tuple(grads)
    if len(grads) != len(spec.grad_names()):
        raise ValueError(f"backward returned {len(grads)} gradients, contract requires "
                         f"{len(spec.grad_names())}: {spec.grad_names()}")
    tol = ((lambda r: spec.strict_tolerance_for(dims, dtype, r)) if strict
           else (lambda r: spec.tolerance_for(dims, dtype, r)))
    out = [check(spec.output, y, y_ref, *tol(None))]
    for name, g in zip(spec.grad_names(), grads):
        out.append(check(name, g, g_ref[name], *tol(name)))
    return out
