"""Host logic of the sharded launcher with two ``gloo`` ranks on CPU: row
partitioning, the float32 all-reduce of parameter-gradient partial sums and the
single rounding after it. The local kernels are stand-ins built from the oracle
arithmetic (the CUDA kernels themselves are covered by the ``gpu`` tests)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from evograd_b200.sharded import NormKernels, ShardedNorm, block_range
from oracle import autograd_oracle as ao


def test_block_range_covers_everything_once():
    for total in (0, 1, 7, 128, 16384):
        for world in (1, 2, 3, 8):
            spans = [block_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        block_range(10, 2, 2)


def _cpu_kernels() -> NormKernels:
    """float32 closed forms of the local forward/backward (what the kernels compute)."""

    def ln_fwd(x, w, b, eps):
        xf = x.float()
        mean = xf.mean(-1)
        var = ((xf - mean[:, None]) ** 2).mean(-1)
        rstd = torch.rsqrt(var + eps)
        y = ((xf - mean[:, None]) * rstd[:, None] * w.float() + b.float()).to(x.dtype)
        return y, mean, rstd

    def ln_bwd(dy, x, w, mean, rstd, partials_f32=False):
        assert partials_f32
        xh = (x.float() - mean[:, None]) * rstd[:, None]
        g = dy.float() * w.float()
        dx = rstd[:, None] * (g - g.mean(-1, keepdim=True) - xh * (g * xh).mean(-1, keepdim=True))
        return dx.to(x.dtype), torch.stack(((dy.float() * xh).sum(0), dy.float().sum(0))), None

    def rms_fwd(x, w, eps):
        xf = x.float()
        rstd = torch.rsqrt((xf * xf).mean(-1) + eps)
        return (xf * rstd[:, None] * w.float()).to(x.dtype), rstd

    def rms_bwd(dy, x, w, rstd, partials_f32=False):
        assert partials_f32
        xh = x.float() * rstd[:, None]
        g = dy.float() * w.float()
        dx = (g - xh * (g * xh).mean(-1, keepdim=True)) * rstd[:, None]
        return dx.to(x.dtype), (dy.float() * xh).sum(0)

    def add_rms_fwd(x, r, w, eps):
        s_ = x + r  # rounded to the input dtype, as the trusted forward does
        rstd = torch.rsqrt(s_.float().pow(2).mean(-1) + eps)
        return (s_ * rstd[:, None].to(s_.dtype)) * w, rstd

    def add_rms_bwd(dout, x, r, w, rstd, partials_f32=False):
        assert partials_f32
        s_ = (x + r).float()
        rb = rstd.to(x.dtype).float()[:, None]
        g = dout.float() * w.float()
        c = (g * s_).mean(-1, keepdim=True)
        dx = g * rb - s_ * (rstd[:, None] ** 3) * c
        t = (s_ * rb).to(x.dtype).float()
        return dx.to(x.dtype), (dout.float() * t).sum(0)

    return NormKernels(ln_fwd, ln_bwd, rms_fwd, rms_bwd, lambda t, dtype: t.to(dtype),
                       add_rms_fwd, add_rms_bwd)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dims(kind):
    return dict(rows=37, cols=96) if kind == "fused_add_rms_norm" else dict(rows=37, hidden=96)


def _worker(rank, world, port, kind, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dims = _dims(kind)  # odd row count: shards of 19 and 18
        inputs = ao.make_inputs(kind, dims, "bfloat16")
        a, b = block_range(dims["rows"], world, rank)
        sn = ShardedNorm(kind, kernels=_cpu_kernels())
        if kind == "fused_add_rms_norm":
            y, saved = sn.forward_with_saved(inputs["x"][a:b], inputs["weight"], None,
                                             inputs["eps"], residual=inputs["r"][a:b])
            grads = sn.backward_from_saved(inputs["dout"][a:b], saved)
            assert grads[1] is grads[0]
            grads = (grads[0], grads[2])
        else:
            y, saved = sn.forward_with_saved(inputs["x"][a:b], inputs["weight"], inputs.get("bias"), 1e-5)
            grads = sn.backward_from_saved(inputs["dy"][a:b], saved)
        assert sn.collectives == 1
        out[rank] = {"span": (a, b), "y": y, "dx": grads[0], "params": [g for g in grads[1:]]}
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm", "fused_add_rms_norm"])
def test_two_ranks_match_the_full_input_oracle(kind):
    world, port = 2, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, kind, out), nprocs=world, join=True)
    dims = _dims(kind)
    inputs = ao.make_inputs(kind, dims, "bfloat16")
    y_ref, g_ref = ao.oracle(kind, inputs, reference_dtype=torch.float32)
    spec = ao.OPS[kind]
    param_names = [n for n in spec.grad_names() if n not in ("dx", "dr")]
    for rank in range(world):
        a, b = out[rank]["span"]
        assert ao.check("y", out[rank]["y"], y_ref[a:b], *ao.STRICT_TOLERANCES["bfloat16"]).ok
        assert ao.check("dx", out[rank]["dx"], g_ref["dx"][a:b], *ao.STRICT_TOLERANCES["bfloat16"]).ok
        for name, g in zip(param_names, out[rank]["params"]):
            assert g.dtype == torch.bfloat16
            c = ao.check(name, g, g_ref[name], *spec.strict_tolerance_for(dims, "bfloat16", name))
            assert c.ok, (name, c)
    # every rank holds the same rounded parameter gradients
    for g0, g1 in zip(out[0]["params"], out[1]["params"]):
        assert torch.equal(g0, g1)


def test_rounding_happens_after_the_sum():
    """Partial sums that each round to the same bf16 value must still add in float32."""
    k = _cpu_kernels()
    partial = torch.tensor([257.0, -256.0])  # 257 rounds to 256 in bf16 (spacing 2 there)
    early = partial.to(torch.bfloat16).sum()
    late = k.cast_from_f32(partial.sum(), torch.bfloat16)
    assert early.item() == 0.0 and late.item() == 1.0


def test_single_process_needs_no_group():
    inputs = ao.make_inputs("rmsnorm", dict(rows=8, hidden=64), "float32")
    sn = ShardedNorm("rmsnorm", kernels=_cpu_kernels())
    y, saved = sn.forward_with_saved(inputs["x"], inputs["weight"], None, 1e-5)
    dx, dw = sn.backward_from_saved(inputs["dy"], saved)
    y_ref, g_ref = ao.oracle("rmsnorm", inputs)
    assert sn.collectives == 0
    assert torch.allclose(y, y_ref, atol=1e-5, rtol=1e-5)
    assert torch.allclose(dx, g_ref["dx"], atol=1e-5, rtol=1e-5)
    assert torch.allclose(dw, g_ref["dweight"], atol=1e-5, rtol=1e-5)


class _FakeExchangeLib:
    """Stand-in for the C ABI: records the calls a PeerExchange makes; the "kernel"
    is an all_reduce, so two gloo ranks can run the host logic without a GPU."""

    def __init__(self, rank):
        self.rank = rank
        self.blob = None
        self.destroyed = 0

    def call(self, name, *args):
        import ctypes

        if name == "evg_exchange_create":
            max_floats, world, rank, out, handle = args
            ctypes.memmove(handle, bytes([rank + 1]) * 64, 64)
            out._obj.value = 1234
        elif name == "evg_exchange_connect":
            self.blob = ctypes.string_at(args[1], 128)
        elif name == "evg_exchange_sum_round":
            pass
        elif name == "evg_exchange_destroy":
            self.destroyed += 1
        else:
            raise AssertionError(name)


def _peer_exchange_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from evograd_b200.sharded import PeerExchange

        lib = _FakeExchangeLib(rank)
        ex = PeerExchange(64, lib=lib)
        # every rank receives all handles, in rank order
        assert lib.blob == bytes([1]) * 64 + bytes([2]) * 64, lib.blob
        with pytest.raises(ValueError):
            ex.sum_round(torch.zeros(65), torch.float32)
        with pytest.raises(TypeError):
            ex.sum_round(torch.zeros(8, dtype=torch.float64), torch.float32)
        out = ex.sum_round(torch.zeros(8), torch.bfloat16)
        assert out.dtype == torch.bfloat16 and out.shape == (8,) and ex.calls == 1
        ex.close()
        ex.close()
        assert lib.destroyed == 1
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_peer_exchange_gathers_handles_in_rank_order():
    world = 2
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_peer_exchange_worker, args=(world, port, results), nprocs=world, join=True)
        assert dict(results) == {0: "ok", 1: "ok"}
