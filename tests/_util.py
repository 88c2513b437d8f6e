"""Helpers shared by the parity tests."""

from __future__ import annotations

import importlib.util
from pathlib import Path

import torch

from oracle import autograd_oracle as ao

REPO = Path(__file__).resolve().parent.parent
PAIRS = REPO / "evograd_b200" / "pairs"


def load_pair(op: str):
    """Import a candidate module by FILE PATH, the way evograd's CLIs do
    (opdecl/verify_cli.py:22-28)."""
    path = PAIRS / f"{op}.py"
    spec = importlib.util.spec_from_file_location(f"candidate_{op}", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def to_device(inputs: dict, device="cuda") -> dict:
    return {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in inputs.items()}


def run_pair(op: str, inputs: dict):
    """fwd then bwd through the candidate module; returns (y, grads tuple, saved)."""
    import inspect

    spec = ao.OPS[op]
    mod = load_pair(op)
    fwd = getattr(mod, f"{op}_forward_with_saved")
    bwd = getattr(mod, f"{op}_backward_from_saved")
    positional = [inputs[n] for n, _ in spec.args] + [inputs.get(n, d) for n, d in spec.scalars.items()]
    y, saved = fwd(*positional)
    params = inspect.signature(bwd).parameters
    kwargs = {n: inputs.get(n, d) for n, d in spec.scalars.items() if n in params}
    grads = bwd(inputs[spec.upstream], saved, **kwargs)
    grads = (grads,) if torch.is_tensor(grads) else tuple(grads)
    return y, grads, saved


def assert_checks(checks, context=""):
    bad = [c for c in checks if not c.ok]
    assert not bad, f"{context}: " + "; ".join(
        f"{c.name} max_abs_err={c.max_abs_err:.3e} atol={c.atol} rtol={c.rtol} {c.detail}" for c in bad
    )


def snapshot(inputs: dict) -> dict:
    return {k: v.clone() for k, v in inputs.items() if torch.is_tensor(v)}


def assert_unchanged(inputs: dict, snap: dict):
    for k, v in snap.items():
        assert torch.equal(inputs[k], v), f"input {k} was mutated"
