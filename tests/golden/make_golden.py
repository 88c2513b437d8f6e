"""Regenerates ``tests/golden/*.npz`` by running the REFERENCE itself
(akumdam2/evograd) on CPU: its ``make_case_inputs`` hooks build the seeded inputs
and its ``evograd.opdecl.oracle.oracle`` produces y and the gradients.

    python tests/golden/make_golden.py --reference /path/to/evograd/src

The reference is only needed to regenerate; the tests read the committed files.
Each file stores, for one (operator, shape, dtype) case, the inputs and the
same-dtype oracle outputs, plus the outputs of the float32-promoted oracle
(suffix ``__f32ref``). 16-bit tensors are stored as their raw bit patterns
(uint16) with the dtype recorded in ``__meta__``.

Causal attention has no declaration in the reference. Its vectors come from the
reference's ``evoattention`` operator with ``res_mask = 0`` and
``pair_bias = 0 / -inf`` causal mask (N_seq = 1), i.e. the reference's own
attention arithmetic applied to the causal case, transposed to [B, H, S, D].
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

CASES = {
    "softmax": [
        ({"rows": 8, "cols": 512}, "float32"),
        ({"rows": 16, "cols": 1024}, "float32"),
        ({"rows": 16, "cols": 2048}, "bfloat16"),
        ({"rows": 8, "cols": 4096}, "float16"),
        ({"rows": 5, "cols": 333}, "float32"),
    ],
    "layernorm": [
        ({"rows": 8, "hidden": 64}, "float32"),
        ({"rows": 17, "hidden": 128}, "float32"),
        ({"rows": 32, "hidden": 256}, "float16"),
        ({"rows": 64, "hidden": 512}, "bfloat16"),
        ({"rows": 17, "hidden": 127}, "bfloat16"),
        ({"rows": 17, "hidden": 1000}, "float32"),
    ],
    "rmsnorm": [
        ({"rows": 8, "hidden": 64}, "float32"),
        ({"rows": 17, "hidden": 128}, "float32"),
        ({"rows": 32, "hidden": 256}, "float16"),
        ({"rows": 64, "hidden": 512}, "bfloat16"),
        ({"rows": 17, "hidden": 513}, "float16"),
        ({"rows": 8, "hidden": 4096}, "bfloat16"),
    ],
    "swiglu": [
        ({"rows": 8, "cols": 64}, "float32"),
        ({"rows": 17, "cols": 128}, "float32"),
        ({"rows": 32, "cols": 256}, "float16"),
        ({"rows": 64, "cols": 512}, "bfloat16"),
        ({"rows": 17, "cols": 255}, "bfloat16"),
    ],
    "geglu": [
        ({"rows": 8, "cols": 64}, "float32"),
        ({"rows": 32, "cols": 256}, "float16"),
        ({"rows": 64, "cols": 512}, "bfloat16"),
        ({"rows": 17, "cols": 255}, "bfloat16"),
    ],
    "fused_add_rms_norm": [
        ({"rows": 8, "cols": 64}, "float32"),
        ({"rows": 32, "cols": 256}, "float16"),
        ({"rows": 64, "cols": 512}, "bfloat16"),
        ({"rows": 17, "cols": 513}, "bfloat16"),
        ({"rows": 8, "cols": 4096}, "bfloat16"),
    ],
    "rope": [
        ({"B": 1, "n_heads": 4, "T": 16, "head_dim": 64}, "float32"),
        ({"B": 1, "n_heads": 4, "T": 16, "head_dim": 64}, "float16"),
        ({"B": 1, "n_heads": 4, "T": 16, "head_dim": 64}, "bfloat16"),
        ({"B": 1, "n_heads": 2, "T": 129, "head_dim": 128}, "bfloat16"),
    ],
    "llama3_decoder_layer": [  # the declaration's own correctness workloads
        ({"B": 1, "T": 32, "hidden": 128, "head_dim": 32, "q_out": 128, "kv_out": 32,
          "intermediate": 352}, "float32"),
        ({"B": 2, "T": 17, "hidden": 64, "head_dim": 16, "q_out": 64, "kv_out": 16,
          "intermediate": 176}, "float32"),
        ({"B": 1, "T": 32, "hidden": 128, "head_dim": 32, "q_out": 128, "kv_out": 32,
          "intermediate": 352}, "bfloat16"),
        ({"B": 2, "T": 17, "hidden": 64, "head_dim": 16, "q_out": 64, "kv_out": 16,
          "intermediate": 176}, "bfloat16"),
    ],
    "evoattention": [  # the declaration's own correctness workloads (the fourth with B=1, H=2)
        ({"B": 1, "S": 1, "H": 4, "N": 23, "D": 8}, "float16"),
        ({"B": 1, "S": 2, "H": 4, "N": 64, "D": 16}, "float16"),
        ({"B": 1, "S": 1, "H": 8, "N": 80, "D": 32}, "bfloat16"),
        ({"B": 1, "S": 2, "H": 2, "N": 128, "D": 64}, "bfloat16"),
        ({"B": 1, "S": 1, "H": 4, "N": 48, "D": 128}, "float16"),
    ],
    "causal_attention": [
        ({"B": 1, "H": 1, "S": 160, "D": 128}, "bfloat16"),
        ({"B": 2, "H": 1, "S": 64, "D": 128}, "float16"),
        ({"B": 1, "H": 1, "S": 200, "D": 64}, "bfloat16"),
    ],
}


def _to_np(t: torch.Tensor):
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.view(torch.int16).numpy().view(np.uint16), str(t.dtype).replace("torch.", "")
    return t.numpy(), str(t.dtype).replace("torch.", "")


def case_name(op, dims, dtype):
    return f"{op}__" + "x".join(str(v) for v in dims.values()) + f"__{dtype}"


def _attention_case(evograd, dims, dtype):
    from evograd.opdecl import Workload
    from evograd.opdecl.inputs import make_case_inputs
    from evograd.opdecl.oracle import oracle
    from evograd.ops import get_op

    op = get_op("evoattention")
    B, H, S, D = dims["B"], dims["H"], dims["S"], dims["D"]
    wl = Workload(dims=dict(B=B, S=1, H=H, N=S, D=D), dtype=dtype)
    inputs = make_case_inputs(op, wl, device="cpu")
    inputs["res_mask"] = torch.zeros_like(inputs["res_mask"])
    causal = torch.full((S, S), float("-inf"), dtype=torch.float32).triu(1)
    inputs["pair_bias"] = causal.expand(B, 1, H, S, S).contiguous()
    outs = {}
    for suffix, use_ref in (("", False),):
        y, grads = oracle(op, inputs, use_reference_dtype=use_ref)
        outs["o" + suffix] = y
        for n in ("dq", "dk", "dv"):
            outs[n + suffix] = grads[n]
    # float32-promoted run of the same function
    promoted = {k: (v.float() if torch.is_tensor(v) else v) for k, v in inputs.items()}
    y32, g32 = oracle(op, promoted, use_reference_dtype=False)
    in_dtype = inputs["q"].dtype  # cast back, as oracle.py:106-110 does
    outs["o__f32ref"] = y32.to(in_dtype)
    for n in ("dq", "dk", "dv"):
        outs[n + "__f32ref"] = g32[n].to(in_dtype)
    to_bhsd = lambda t: t[:, 0].permute(0, 2, 1, 3).contiguous()
    tensors = {k: to_bhsd(inputs[k]) for k in ("q", "k", "v", "do")}
    tensors.update({k: to_bhsd(v) for k, v in outs.items()})
    return tensors, {}


def _declared_case(op_name, dims, dtype):
    import dataclasses

    from evograd.opdecl import Workload
    from evograd.opdecl.inputs import make_case_inputs
    from evograd.opdecl.oracle import oracle
    from evograd.ops import get_op

    op = get_op(op_name)
    wl = Workload(dims=dict(dims), dtype=dtype)
    inputs = make_case_inputs(op, wl, device="cpu")
    tensors, scalars = {}, {}
    for k, v in inputs.items():
        if torch.is_tensor(v):
            tensors[k] = v
        else:
            scalars[k] = v
    y, grads = oracle(op, inputs, use_reference_dtype=False)
    tensors[op.output.name] = y
    tensors.update(grads)
    op32 = dataclasses.replace(op, reference_dtype="float32")
    y32, g32 = oracle(op32, inputs, use_reference_dtype=True)
    tensors[op.output.name + "__f32ref"] = y32
    tensors.update({k + "__f32ref": v for k, v in g32.items()})
    return tensors, scalars


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True,
                    help="path to the reference's src/ directory (akumdam2/evograd checkout)")
    ap.add_argument("--only", nargs="*", default=None,
                    help="regenerate only these operators (the index keeps the others)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import evograd  # noqa: F401

    torch.set_num_threads(1)  # one summation order, whatever the host
    index = {}
    index_path = HERE / "index.json"
    if args.only and index_path.exists():
        index = json.loads(index_path.read_text())
    for op_name, cases in CASES.items():
        if args.only and op_name not in args.only:
            continue
        for dims, dtype in cases:
            if op_name == "causal_attention":
                tensors, scalars = _attention_case(evograd, dims, dtype)
            else:
                tensors, scalars = _declared_case(op_name, dims, dtype)
            arrays, meta = {}, {"op": op_name, "dims": dims, "dtype": dtype, "scalars": scalars,
                                "tensor_dtypes": {}, "torch": torch.__version__}
            for k, t in tensors.items():
                arrays[k], meta["tensor_dtypes"][k] = _to_np(t)
            name = case_name(op_name, dims, dtype)
            np.savez_compressed(HERE / f"{name}.npz", __meta__=np.array(json.dumps(meta)), **arrays)
            index[name] = {"op": op_name, "dims": dims, "dtype": dtype}
            print("wrote", name, {k: tuple(v.shape) for k, v in arrays.items()})
    (HERE / "index.json").write_text(json.dumps(index, indent=1, sort_keys=True) + "\n")


if __name__ == "__main__":
    main()
