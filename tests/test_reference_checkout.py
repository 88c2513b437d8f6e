"""Checks that need a checkout of the reference project: set ``EVOGRAD_SRC`` to
the directory that holds its ``evograd`` package (``.../src``). Without it every
test here is skipped; nothing else in the suite reads the reference.

* the in-tree ``causal_attention`` package (``evograd_b200/decls/in_tree``) is
  discovered as a built-in operator by the reference's own registry and passes
  its own correctness gate on CPU with a plain-torch candidate;
* (GPU) the reference's own ``verify`` accepts every candidate module under
  ``evograd_b200/pairs``.
"""

import json
import os
import shutil
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
SRC = os.environ.get("EVOGRAD_SRC")
needs_checkout = pytest.mark.skipif(
    not SRC or not (Path(SRC) / "evograd" / "ops" / "__init__.py").exists(),
    reason="EVOGRAD_SRC does not point at a reference checkout")

TORCH_CANDIDATE = textwrap.dedent('''
    import math
    import torch

    def causal_attention_forward_with_saved(q, k, v):
        scale = 1.0 / math.sqrt(q.shape[-1])
        s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
        mask = torch.ones(s.shape[-2:], dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        o = torch.matmul(p, v.float()).to(q.dtype)
        return o, (q, k, v, p)

    def causal_attention_backward_from_saved(do, saved):
        q, k, v, p = saved
        scale = 1.0 / math.sqrt(q.shape[-1])
        dof = do.float()
        dv = torch.matmul(p.transpose(-1, -2), dof)
        dp = torch.matmul(dof, v.float().transpose(-1, -2))
        ds = p * (dp - (dp * p).sum(-1, keepdim=True))
        dq = torch.matmul(ds, k.float()) * scale
        dk = torch.matmul(ds.transpose(-1, -2), q.float()) * scale
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)
''')


@pytest.fixture(scope="module")
def patched_checkout(tmp_path_factory):
    """A scratch copy of the reference's package with the in-tree operator dropped in."""
    root = tmp_path_factory.mktemp("evograd_src")
    shutil.copytree(Path(SRC) / "evograd", root / "evograd",
                    ignore=shutil.ignore_patterns("__pycache__"))
    shutil.copytree(REPO / "evograd_b200" / "decls" / "in_tree" / "causal_attention",
                    root / "evograd" / "ops" / "level1" / "causal_attention")
    return root


def _run(root, *args, timeout=600):
    env = dict(os.environ, PYTHONPATH=f"{root}{os.pathsep}{REPO}")
    env.pop("EVOGRAD_DECLARATION", None)
    return subprocess.run([sys.executable, *args], env=env, capture_output=True, text=True,
                          timeout=timeout, cwd=root)


@needs_checkout
def test_in_tree_package_is_discovered_as_a_builtin(patched_checkout):
    code = ("from evograd.ops import OPS, get_op; op = get_op('causal_attention'); "
            "assert 'causal_attention' in OPS; print(op.name, op.grad_names(), len(op.correctness))")
    out = _run(patched_checkout, "-c", code)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.split()[0] == "causal_attention"
    assert "dq" in out.stdout and "dv" in out.stdout


@needs_checkout
def test_reference_gate_passes_on_cpu_with_a_torch_candidate(patched_checkout, tmp_path):
    cand = tmp_path / "causal_attention.py"
    cand.write_text(TORCH_CANDIDATE)
    out = _run(patched_checkout, "-m", "evograd.opdecl.verify_cli", "--op", "causal_attention",
               "--device", "cpu", str(cand))
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-2000:])
    report = json.loads(out.stdout[out.stdout.index("{"):])
    assert report["metrics"]["correct"] == 1.0 and report["verify"]["ok"], report


PAIRS = sorted(p.stem for p in (REPO / "evograd_b200" / "pairs").glob("*.py") if p.stem != "__init__")


@needs_checkout
@pytest.mark.gpu
@pytest.mark.parametrize("op", PAIRS)
def test_reference_gate_accepts_the_cuda_candidates(patched_checkout, op):
    out = _run(patched_checkout, "-m", "evograd.opdecl.verify_cli", "--op", op,
               str(REPO / "evograd_b200" / "pairs" / f"{op}.py"), timeout=1800)
    assert out.returncode == 0, (out.stdout[-2000:], out.stderr[-2000:])
    report = json.loads(out.stdout[out.stdout.index("{"):])
    assert report["metrics"]["correct"] == 1.0 and report["verify"]["ok"], report
