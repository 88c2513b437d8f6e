"""GPU parity of the EvoformerAttention pair (additive key mask, trainable pair
bias reduced over the MSA axis) against reference-generated vectors and the CPU
oracle, through the candidate module and the C ABI."""

import pytest
import torch

from _util import assert_checks, assert_unchanged, load_pair, run_pair, snapshot, to_device
from conftest import golden_cases, load_golden
from oracle import autograd_oracle as ao

pytestmark = pytest.mark.gpu
OP = "evoattention"


@pytest.mark.parametrize("name", golden_cases(OP))
def test_matches_reference_golden_vectors(name):
    meta, t = load_golden(name)
    dims, dtype = meta["dims"], meta["dtype"]
    spec = ao.OPS[OP]
    inputs = to_device({n: t[n] for n in [a for a, _ in spec.args] + [spec.upstream]})
    snap = snapshot(inputs)
    o, grads, saved = run_pair(OP, inputs)
    assert_unchanged(inputs, snap)
    got = {spec.output: o, **dict(zip(spec.grad_names(), grads))}
    assert got["d_pair_bias"].dtype == torch.float32
    assert tuple(got["d_pair_bias"].shape) == tuple(t["pair_bias"].shape)
    declared = [ao.check(n, g, t[n], *spec.tolerance_for(dims, dtype, n)) for n, g in got.items()]
    assert_checks(declared, f"{name} declared")
    # against the float32-promoted reference: o within the 16-bit gate, gradients 2e-2 max-abs
    strict = [ao.check("o", got["o"], t["o__f32ref"], 1e-2, 1.6e-2)]
    for n in ("dq", "dk", "dv", "d_pair_bias"):
        strict.append(ao.check(n, got[n], t[n + "__f32ref"], 2e-2, 1.6e-2))
    assert_checks(strict, f"{name} strict")


CASES = [
    (dict(B=1, S=1, H=4, N=23, D=8), "float16"), (dict(B=1, S=2, H=4, N=64, D=16), "float16"),
    (dict(B=1, S=1, H=8, N=80, D=32), "bfloat16"), (dict(B=2, S=2, H=4, N=128, D=64), "bfloat16"),
    (dict(B=1, S=1, H=4, N=48, D=128), "float16"), (dict(B=1, S=3, H=2, N=129, D=24), "bfloat16"),
    (dict(B=1, S=5, H=1, N=33, D=40), "float16"), (dict(B=1, S=16, H=4, N=256, D=32), "bfloat16"),
    # tensor-core path: head sizes 32 (heads in pairs) and 64, ragged residue counts
    (dict(B=1, S=1, H=16, N=384, D=64), "float16"), (dict(B=1, S=3, H=2, N=132, D=32), "bfloat16"),
    (dict(B=2, S=5, H=3, N=100, D=64), "bfloat16"), (dict(B=1, S=40, H=4, N=64, D=32), "float16"),
    (dict(B=1, S=2, H=6, N=260, D=32), "bfloat16"), (dict(B=1, S=64, H=8, N=128, D=32), "bfloat16"),
]


@pytest.mark.parametrize("dims,dtype", CASES)
def test_pair_passes_the_declared_gate(dims, dtype):
    inputs = ao.make_inputs(OP, dims, dtype)
    dev = to_device(inputs)
    snap = snapshot(dev)
    assert_checks(ao.verify_pair(OP, load_pair(OP), dev, dims, dtype), f"{OP} {dims} {dtype}")
    assert_unchanged(dev, snap)


def test_unstaged_path_gives_the_same_answer():
    """With staging disabled the kernels read K/V (Q/dO) rows straight from global memory."""
    from evograd_b200 import _cabi

    dims, dtype = dict(B=1, S=3, H=2, N=129, D=24), "bfloat16"
    inputs = to_device(ao.make_inputs(OP, dims, dtype))
    o1, g1, _ = run_pair(OP, inputs)
    try:
        _cabi.tune_set("evoattention.no_stage", 1)
        o2, g2, _ = run_pair(OP, inputs)
    finally:
        _cabi.tune_set("evoattention.no_stage", 0)
    assert torch.equal(o1, o2)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dims", [dict(B=1, S=4, H=2, N=100, D=32), dict(B=1, S=37, H=4, N=192, D=64),
                                  dict(B=1, S=4, H=3, N=101, D=32)])
def test_gradients_are_bit_reproducible(dims):
    inputs = to_device(ao.make_inputs(OP, dims, "bfloat16"))
    _, g1, _ = run_pair(OP, inputs)
    _, g2, _ = run_pair(OP, inputs)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)


@pytest.mark.parametrize("dims,dtype", [(dict(B=1, S=6, H=4, N=200, D=32), "bfloat16"),
                                        (dict(B=2, S=2, H=2, N=320, D=64), "float16")])
def test_tensor_core_and_cuda_core_kernels_agree(dims, dtype):
    """Head sizes 32 / 64 run on the tcgen05 kernels; ``evoattention.no_tc`` sends the
    same call to the CUDA-core kernels. Both must sit within the strict bounds of
    the float32-promoted oracle, and close to each other."""
    from evograd_b200 import _cabi

    inputs = ao.make_inputs(OP, dims, dtype)
    dev = to_device(inputs)
    o1, g1, _ = run_pair(OP, dev)
    try:
        _cabi.tune_set("evoattention.no_tc", 1)
        o2, g2, _ = run_pair(OP, dev)
    finally:
        _cabi.tune_set("evoattention.no_tc", 0)
    o_ref, g_ref = ao.oracle(OP, inputs, reference_dtype=torch.float32)
    names = ("dq", "dk", "dv", "d_pair_bias")
    for tag, o, g in (("tensor cores", o1, g1), ("cuda cores", o2, g2)):
        checks = [ao.check("o", o, o_ref, 1e-2, 1.6e-2)]
        checks += [ao.check(n, t, g_ref[n], 2e-2, 1.6e-2) for n, t in zip(names, g)]
        assert_checks(checks, f"{dims} {dtype} {tag}")
    assert (o1.float() - o2.float()).abs().max().item() <= 2e-2


def test_argument_checks():
    from evograd_b200 import ops

    q = torch.zeros(1, 1, 8, 2, 16, device="cuda", dtype=torch.bfloat16)
    mask = torch.zeros(1, 1, 1, 1, 8, device="cuda")
    bias = torch.zeros(1, 1, 2, 8, 8, device="cuda")
    with pytest.raises(ValueError):
        ops.evoattention_fwd(q, q, q, mask[..., :4], bias)
    with pytest.raises(ValueError):
        ops.evoattention_fwd(q, q, q, mask, bias.to(torch.bfloat16))
    with pytest.raises(ValueError):
        ops.evoattention_fwd(q[0], q[0], q[0], mask, bias)
