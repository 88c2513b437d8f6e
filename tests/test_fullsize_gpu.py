"""The row-wise pairs at the sizes they are benchmarked at. The CPU oracle cannot
chew through whole tensors of that size in seconds, so the checks use what the
operators offer independently of size:

* rows are independent: the oracle applied to a sample of rows must reproduce
  those rows of y / dx (and, for the element-wise operators, any slice);
* parameter gradients are plain column sums: a float32 reference formed from the
  kernel's own inputs on the device bounds them with the row-scaled tolerance;
* backward is linear in the upstream gradient: scaling dy by a power of two
  scales every gradient by exactly that factor, bit for bit;
* softmax rows sum to one, RoPE preserves norms.
"""

import pytest
import torch

from _util import assert_checks, run_pair, to_device
from oracle import autograd_oracle as ao

pytestmark = pytest.mark.gpu


def _sample_rows(rows, n=48):
    g = torch.Generator().manual_seed(rows)
    idx = torch.randperm(rows, generator=g)[:n].sort().values
    idx[0], idx[-1] = 0, rows - 1
    return idx


def _gen_inputs(op, dims, dtype, device="cuda"):
    """Seeded inputs built on the device (host generation of gigabyte tensors is slow)."""
    return ao.make_inputs(op, dims, dtype, device=device)


def _check_row_sample(op, inputs, dims, dtype, y, grads, row_names, strict=True):
    spec = ao.OPS[op]
    idx = _sample_rows(dims["rows"])
    sub = {k: (v[idx].cpu() if (torch.is_tensor(v) and k in row_names) else
               (v.cpu() if torch.is_tensor(v) else v)) for k, v in inputs.items()}
    y_ref, g_ref = ao.oracle(spec, sub, reference_dtype=torch.float32 if strict else None)
    tol = ao.STRICT_TOLERANCES[dtype] if strict else spec.tolerances[dtype]
    checks = [ao.check(spec.output, y[idx], y_ref, *tol)]
    for name, g in zip(spec.grad_names(), grads):
        if g.ndim == 2 and g.shape[0] == dims["rows"]:
            checks.append(ao.check(name, g[idx], g_ref[name], *tol))
    assert_checks(checks, f"{op} full-size row sample")


@pytest.mark.parametrize("op,dims,eps", [
    ("layernorm", dict(rows=16384, hidden=4096), 1e-5),
    ("rmsnorm", dict(rows=32768, hidden=4096), 1e-6),
])
def test_norms_at_benchmark_size(op, dims, eps):
    dtype = "bfloat16"
    inputs = _gen_inputs(op, dims, dtype)
    inputs["eps"] = eps
    y, grads, _ = run_pair(op, inputs)
    _check_row_sample(op, inputs, dims, dtype, y, grads, ("x", "dy"))
    # parameter gradients: float32 column sums formed on the device from the same inputs
    x, dy, w = inputs["x"].float(), inputs["dy"].float(), inputs["weight"].float()
    if op == "layernorm":
        mean = x.mean(-1, keepdim=True)
        xh = (x - mean) * torch.rsqrt(((x - mean) ** 2).mean(-1, keepdim=True) + eps)
        refs = {"dweight": (dy * xh).sum(0), "dbias": dy.sum(0)}
    else:
        xh = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)
        refs = {"dweight": (dy * xh).sum(0)}
    spec = ao.OPS[op]
    for name, g in zip(spec.grad_names()[1:], grads[1:]):
        atol, rtol = spec.tolerance_for(dims, dtype, name)
        c = ao.check(name, g, refs[name].to(g.dtype), atol, rtol)
        assert c.ok, (op, c)
        # and much tighter than the declared bound: within two bf16 ulps of the float32 sum
        err = (g.float() - refs[name]).abs()
        assert (err <= 2 ** -7 * refs[name].abs() + 1e-2).all(), (name, err.max().item())
    # linearity: dy * 4 scales every gradient by exactly 4
    scaled = dict(inputs, dy=inputs["dy"] * 4)
    _, grads4, _ = run_pair(op, scaled)
    for g, g4 in zip(grads, grads4):
        assert torch.equal(g4.float(), g.float() * 4)


def test_softmax_float32_at_benchmark_size_against_the_full_oracle():
    dims, dtype = dict(rows=4096, cols=1024), "float32"
    inputs = ao.make_inputs("softmax", dims, dtype)  # small enough for the whole oracle
    dev = to_device(inputs)
    checks = ao.verify_pair("softmax", __import__("_util").load_pair("softmax"), dev, dims, dtype,
                            strict=True)
    assert_checks(checks, "softmax float32 [4096, 1024]")
    y, _, _ = run_pair("softmax", dev)
    assert torch.allclose(y.sum(-1), torch.ones(dims["rows"], device="cuda"), atol=1e-5, rtol=0)


def test_softmax_at_vocabulary_width():
    dims, dtype = dict(rows=4096, cols=128256), "bfloat16"
    inputs = _gen_inputs("softmax", dims, dtype)
    y, grads, _ = run_pair("softmax", inputs)
    _check_row_sample("softmax", inputs, dims, dtype, y, grads, ("x", "dy"))
    sums = y.float().sum(-1)  # bf16 rounding of 128256 small terms: a loose bound
    assert (sums - 1).abs().max().item() < 2e-2
    scaled = dict(inputs, dy=inputs["dy"] * 2)
    _, grads2, _ = run_pair("softmax", scaled)
    assert torch.equal(grads2[0].float(), grads[0].float() * 2)


@pytest.mark.parametrize("op", ["swiglu", "geglu"])
def test_glu_at_benchmark_size(op):
    dims, dtype = dict(rows=32768, cols=14336), "bfloat16"
    inputs = _gen_inputs(op, dims, dtype)
    c, grads, _ = run_pair(op, inputs)
    # declared gate against the same-dtype oracle (the reference rounds the
    # activation before the product, and so do the kernels)
    _check_row_sample(op, inputs, dims, dtype, c, grads, ("a", "b", "dc"), strict=False)
    scaled = dict(inputs, dc=inputs["dc"] * 2)
    _, grads2, _ = run_pair(op, scaled)
    for g, g2 in zip(grads, grads2):
        assert torch.equal(g2.float(), g.float() * 2)


def test_fused_add_rms_norm_at_benchmark_size():
    op, dims, dtype = "fused_add_rms_norm", dict(rows=32768, cols=4096), "bfloat16"
    inputs = _gen_inputs(op, dims, dtype)
    out, grads, _ = run_pair(op, inputs)
    assert grads[1] is grads[0] or torch.equal(grads[0], grads[1])
    _check_row_sample(op, inputs, dims, dtype, out, grads, ("x", "r", "dout"), strict=False)
    s = (inputs["x"] + inputs["r"])
    rstd = torch.rsqrt(s.float().pow(2).mean(-1, keepdim=True) + inputs["eps"])
    t = (s * rstd.to(s.dtype)).float()
    ref = (inputs["dout"].float() * t).sum(0)
    spec = ao.OPS[op]
    c = ao.check("dweight", grads[2], ref.to(grads[2].dtype), *spec.tolerance_for(dims, dtype, "dweight"))
    assert c.ok, c


def test_rope_q_and_k_at_benchmark_size():
    """q [8, 4096, 32, 128] and k with the same shape, float32 half-width tables:
    a sample of (batch, token) positions against the oracle, norms preserved,
    backward undoes forward up to rounding."""
    from evograd_b200 import ops

    B, S, H, D = 8, 4096, 32, 128
    g = torch.Generator(device="cuda").manual_seed(4096 * 100003 + 32 * 1009 + 128)
    q = torch.randn(B, S, H, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(B, S, H, D, device="cuda", generator=g).bfloat16()
    cos, sin = ao.rope_tables(S, D, theta=10000.0, device="cuda", dtype=torch.float32, duplicate=False)
    yq, yk = ops.rope_qk_fwd(q, k, cos, sin, layout="bthd")
    tok = _sample_rows(S, 24)
    cos_f, sin_f = torch.cat((cos, cos), -1)[tok].cpu(), torch.cat((sin, sin), -1)[tok].cpu()
    for x, y in ((q, yq), (k, yk)):
        xs = x[:, tok].transpose(1, 2).cpu()  # [B, H, tokens, D]
        ref = ao.rope_forward(xs, cos_f, sin_f)
        assert torch.equal(y[:, tok].transpose(1, 2).cpu(), ref)
        n_in, n_out = x.float().norm(dim=-1), y.float().norm(dim=-1)
        assert torch.allclose(n_in, n_out, rtol=2e-2, atol=1e-2)
    bq, bk = ops.rope_qk_bwd(yq, yk, cos, sin, layout="bthd")
    assert torch.allclose(bq.float(), q.float(), atol=6e-2, rtol=2e-2)
    # the backward on the same sample of positions against autograd of the oracle forward
    # (upstream gradients: the rotated tensors themselves)
    for up, got in ((yq, bq), (yk, bk)):
        ups = up[:, tok].transpose(1, 2).cpu()
        xs = torch.zeros_like(ups, dtype=torch.float32, requires_grad=True)
        ref_out = ao.rope_forward(xs, cos_f.float(), sin_f.float())
        (ref_grad,) = torch.autograd.grad(ref_out, xs, grad_outputs=ups.float())
        assert torch.equal(got[:, tok].transpose(1, 2).cpu(), ref_grad.to(got.dtype))
