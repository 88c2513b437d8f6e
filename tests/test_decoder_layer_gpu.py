"""GPU parity of the Llama-3 decoder-layer pair (this package's kernels plus
library GEMMs) against the reference's float32-promoted oracle: the
declaration's own correctness workloads from reference-generated vectors, and
larger grouped-query shapes that reach the tensor-core attention kernels."""

import pytest
import torch

from _util import assert_checks, assert_unchanged, load_pair, run_pair, snapshot, to_device
from conftest import golden_cases, load_golden
from oracle import autograd_oracle as ao

pytestmark = pytest.mark.gpu
OP = "llama3_decoder_layer"


@pytest.fixture(autouse=True)
def _status():
    from evograd_b200 import ops

    yield
    ops.device_status()


@pytest.mark.parametrize("name", golden_cases(OP))
def test_matches_reference_golden_vectors(name):
    """The declaration sets reference_dtype = float32, so the gate compares with
    the float32-promoted outputs (cast back to the input dtype)."""
    meta, t = load_golden(name)
    dims, dtype = meta["dims"], meta["dtype"]
    spec = ao.OPS[OP]
    inputs = {n: t[n] for n in [a for a, _ in spec.args] + [spec.upstream]}
    inputs.update(meta["scalars"])
    inputs = to_device(inputs)
    snap = snapshot(inputs)
    y, grads, _ = run_pair(OP, inputs)
    assert_unchanged(inputs, snap)
    got = {spec.output: y, **dict(zip(spec.grad_names(), grads))}
    checks = [ao.check(n, g, t[n + "__f32ref"], *spec.tolerance_for(dims, dtype, n))
              for n, g in got.items()]
    assert_checks(checks, name)


CASES = [
    # head_dim 64 / 128 in 16-bit: tensor-core attention with 4 query heads per k/v head
    (dict(B=1, T=256, hidden=512, head_dim=64, q_out=512, kv_out=128, intermediate=1408), "bfloat16"),
    (dict(B=2, T=300, hidden=1024, head_dim=128, q_out=1024, kv_out=256, intermediate=2816), "bfloat16"),
    # float32 at a head size the tensor-core kernels also know: CUDA-core attention
    (dict(B=1, T=96, hidden=256, head_dim=64, q_out=256, kv_out=64, intermediate=704), "float32"),
]


@pytest.mark.parametrize("dims,dtype", CASES)
def test_pair_passes_the_declared_gate(dims, dtype):
    inputs = ao.make_inputs(OP, dims, dtype)
    dev_inputs = to_device(inputs)
    snap = snapshot(dev_inputs)
    checks = ao.verify_pair(OP, load_pair(OP), dev_inputs, dims, dtype,
                            reference_dtype=torch.float32)
    assert_checks(checks, f"{OP} {dims} {dtype}")
    assert_unchanged(dev_inputs, snap)


def test_gradients_are_bit_reproducible():
    dims, dtype = CASES[0]
    inputs = to_device(ao.make_inputs(OP, dims, dtype))
    _, g1, _ = run_pair(OP, inputs)
    _, g2, _ = run_pair(OP, inputs)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)
