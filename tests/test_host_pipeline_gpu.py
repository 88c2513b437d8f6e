"""The host-buffer pipeline (rows cut into chunks, copy-in / kernels / copy-out
overlapped on three streams) gives the same results as one whole-tensor call."""

import pytest
import torch

from oracle import autograd_oracle as ao

pytestmark = pytest.mark.gpu


def _pinned(t):
    return t.contiguous().pin_memory()


@pytest.mark.parametrize("op,dims", [
    ("layernorm", dict(rows=1000, hidden=1024)), ("rmsnorm", dict(rows=777, hidden=2048)),
    ("fused_add_rms_norm", dict(rows=515, cols=1024)), ("softmax", dict(rows=300, cols=4096)),
    ("swiglu", dict(rows=129, cols=1000)), ("geglu", dict(rows=64, cols=2048)),
])
@pytest.mark.parametrize("chunks", [1, 5, 8])
def test_pipeline_matches_the_direct_call_and_the_gate(op, dims, chunks):
    from evograd_b200 import ops
    from evograd_b200.host_pipeline import pipeline_for

    dtype = "bfloat16"
    inputs = ao.make_inputs(op, dims, dtype)
    spec = ao.OPS[op]
    row_names = [n for n, _ in spec.args if inputs[n].ndim == 2] + [spec.upstream]
    param_names = [n for n, _ in spec.args if inputs[n].ndim == 1]
    eps = inputs.get("eps", 1e-5)
    pipe, finish = pipeline_for(op, eps=eps, chunks=chunks)
    host_rows = {n: _pinned(inputs[n]) for n in row_names}
    params = {n: inputs[n].cuda() for n in param_names}
    like = host_rows[row_names[0]]
    out_names = [spec.output] + [g for g, (n, _) in zip(spec.grad_names(), spec.args)
                                 if inputs[n].ndim == 2 and g != "dr"]
    host_out = {n: torch.empty_like(like).pin_memory() for n in out_names}
    grad_names = [g for g, (n, _) in zip(spec.grad_names(), spec.args) if inputs[n].ndim == 1]
    host_grads = {g: torch.empty_like(inputs[param_names[0]]).pin_memory() for g in grad_names}
    pipe.run(host_rows, params, host_out, host_grads,
             (lambda total: finish(total, like.dtype)) if finish else None)
    torch.cuda.synchronize()
    ops.device_status()

    y_ref, g_ref = ao.oracle(op, inputs)
    checks = [ao.check(spec.output, host_out[spec.output], y_ref, *spec.tolerance_for(dims, dtype))]
    for g in out_names[1:]:
        checks.append(ao.check(g, host_out[g], g_ref[g], *spec.tolerance_for(dims, dtype, g)))
    for g in grad_names:
        checks.append(ao.check(g, host_grads[g], g_ref[g], *spec.tolerance_for(dims, dtype, g)))
    bad = [c for c in checks if not c.ok]
    assert not bad, bad

    # one chunk is the direct call: per-row outputs do not depend on the chunking at all
    pipe1, finish1 = pipeline_for(op, eps=eps, chunks=1)
    host_out1 = {n: torch.empty_like(like).pin_memory() for n in out_names}
    host_grads1 = {g: torch.empty_like(inputs[param_names[0]]).pin_memory() for g in grad_names}
    pipe1.run(host_rows, params, host_out1, host_grads1,
              (lambda total: finish1(total, like.dtype)) if finish1 else None)
    torch.cuda.synchronize()
    for n in out_names:
        assert torch.equal(host_out[n], host_out1[n]), n


def test_unpinned_input_is_refused():
    from evograd_b200.host_pipeline import pipeline_for

    pipe, _ = pipeline_for("softmax")
    x = torch.zeros(8, 64)
    with pytest.raises(ValueError, match="pinned"):
        pipe.run({"x": x, "dy": x}, {}, {"y": x, "dx": x})


def test_graph_replay_gives_the_same_bits_as_the_call_by_call_step():
    """run_graphed captures the whole step once per set of buffers and replays it;
    new host contents are picked up by the replay, results equal run()'s bit for bit."""
    from evograd_b200 import ops
    from evograd_b200.host_pipeline import pipeline_for

    rows, hidden = 1536, 1024
    torch.manual_seed(11)
    host_rows = {n: _pinned(torch.randn(rows, hidden).to(torch.bfloat16)) for n in ("x", "dy")}
    params = {"weight": torch.randn(hidden).to(torch.bfloat16).cuda(),
              "bias": torch.randn(hidden).to(torch.bfloat16).cuda()}

    def fresh():
        return ({n: torch.empty(rows, hidden, dtype=torch.bfloat16).pin_memory() for n in ("y", "dx")},
                {n: torch.empty(hidden, dtype=torch.bfloat16).pin_memory() for n in ("dweight", "dbias")})

    pipe, finish = pipeline_for("layernorm", chunks=12)
    fin = lambda total: finish(total, torch.bfloat16)  # noqa: E731
    out_g, grads_g = fresh()
    for _ in range(2):  # capture, then a replay on new inputs
        host_rows["x"].copy_(torch.randn(rows, hidden).to(torch.bfloat16))
        pipe.run_graphed(host_rows, params, out_g, grads_g, fin)
        torch.cuda.synchronize()
    out_e, grads_e = fresh()
    keep = pipe.run(host_rows, params, out_e, grads_e, fin)
    torch.cuda.synchronize()
    ops.device_status()
    del keep
    for n in out_e:
        assert torch.equal(out_e[n], out_g[n]), n
    for n in grads_e:
        assert torch.equal(grads_e[n], grads_g[n]), n
