"""Shared fixtures: the ``gpu`` marker, golden-vector loading, path setup."""

from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
GOLDEN = REPO / "tests" / "golden"
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_index() -> dict:
    return json.loads((GOLDEN / "index.json").read_text())


def load_golden(name: str):
    """Returns ``(meta, tensors)``; 16-bit tensors are rebuilt from their bit patterns."""
    with np.load(GOLDEN / f"{name}.npz") as z:
        meta = json.loads(str(z["__meta__"]))
        tensors = {}
        for key, dtype_name in meta["tensor_dtypes"].items():
            arr = z[key]
            dt = getattr(torch, dtype_name)
            if dt in (torch.bfloat16, torch.float16):
                t = torch.from_numpy(arr.view(np.int16).copy()).view(dt)
            else:
                t = torch.from_numpy(arr.copy())
            tensors[key] = t
    return meta, tensors


def golden_cases(op: str | None = None):
    idx = golden_index()
    return sorted(n for n, m in idx.items() if op is None or m["op"] == op)
