"""Pins the CPU oracle restatement (oracle/autograd_oracle.py) against vectors
produced by the reference itself (tests/golden/make_golden.py): same seeded
inputs bit for bit, same outputs up to summation-order noise of the host BLAS /
vector width."""

import pytest
import torch

from conftest import golden_cases, load_golden
from oracle import autograd_oracle as ao

# Bound on host-to-host differences of one float32 reduction / one 16-bit ulp.
_TOL = {"float32": (2e-6, 2e-6), "float16": (1e-3, 2e-3), "bfloat16": (8e-3, 1.6e-2)}


def _inputs_of(meta, tensors):
    spec = ao.OPS[meta["op"]]
    names = [n for n, _ in spec.args] + [spec.upstream]
    inputs = {n: tensors[n] for n in names}
    inputs.update(meta["scalars"])
    return inputs


@pytest.mark.parametrize("name", golden_cases())
def test_input_recipe_matches_reference(name):
    meta, tensors = load_golden(name)
    made = ao.make_inputs(meta["op"], meta["dims"], meta["dtype"], device="cpu")
    for key, value in made.items():
        if torch.is_tensor(value):
            assert value.dtype == tensors[key].dtype
            assert torch.equal(value, tensors[key]), f"{name}: input {key} differs from the reference"
        else:
            assert value == pytest.approx(meta["scalars"][key])


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_matches_reference_same_dtype(name):
    meta, tensors = load_golden(name)
    spec = ao.OPS[meta["op"]]
    y, grads = ao.oracle(spec, _inputs_of(meta, tensors))
    atol, rtol = _TOL[meta["dtype"]]
    c = ao.check(spec.output, y, tensors[spec.output], atol, rtol)
    assert c.ok, (name, c)
    for g in spec.grad_names():
        c = ao.check(g, grads[g], tensors[g], atol, rtol)
        assert c.ok, (name, c)


@pytest.mark.parametrize("name", golden_cases())
def test_oracle_matches_reference_float32_promoted(name):
    meta, tensors = load_golden(name)
    spec = ao.OPS[meta["op"]]
    y, grads = ao.oracle(spec, _inputs_of(meta, tensors), reference_dtype=torch.float32)
    atol, rtol = _TOL[meta["dtype"]]
    c = ao.check(spec.output, y, tensors[spec.output + "__f32ref"], atol, rtol)
    assert c.ok, (name, c)
    for g in spec.grad_names():
        c = ao.check(g, grads[g], tensors[g + "__f32ref"], atol, rtol)
        assert c.ok, (name, c)


def test_sdpa_spelling_agrees_with_primitive_spelling():
    """The two causal-attention restatements must agree before either is trusted."""
    inputs = ao.make_inputs("causal_attention", dict(B=1, H=2, S=96, D=64), "float32")
    y1, g1 = ao.oracle("causal_attention", inputs)
    y2, g2 = ao.oracle("causal_attention", inputs, forward=ao.causal_attention_forward_sdpa)
    assert torch.allclose(y1, y2, atol=1e-5, rtol=1e-5)
    for n in g1:
        assert torch.allclose(g1[n], g2[n], atol=1e-5, rtol=1e-5), n


def test_gate_names_the_bad_tensor():
    """The gate is shape + dtype + allclose (opdecl/verify.py:85-115)."""
    e = torch.zeros(4, 4)
    assert ao.check("y", e.clone(), e, 1e-5, 1e-5).ok
    assert not ao.check("y", e.clone() + 1e-3, e, 1e-5, 1e-5).ok
    assert not ao.check("y", e.to(torch.float16), e, 1e-5, 1e-5).ok
    assert not ao.check("y", e[:2], e, 1e-5, 1e-5).ok
    assert not ao.check("y", None, e, 1e-5, 1e-5).ok


def test_bf16_parameter_gradient_tolerance_grows_with_rows():
    spec = ao.OPS["layernorm"]
    assert spec.tolerance_for({"rows": 8, "hidden": 4}, "bfloat16", "dweight") == (8e-2, 8e-2)
    atol, _ = spec.tolerance_for({"rows": 16384, "hidden": 4}, "bfloat16", "dbias")
    assert atol == pytest.approx(8e-2 * (16384 / 8) ** 0.5)
    assert spec.tolerance_for({"rows": 16384, "hidden": 4}, "bfloat16", "dx") == (8e-2, 8e-2)
