"""The cross-GPU sum of parameter-gradient partial sums (``evg_exchange_*``) as far
as one GPU can show it: the one-rank case (publish, add, round; also under CUDA
graph replay, where the step counter lives on the device) and the bounded wait
for a peer whose flag nothing sets. The multi-rank sum itself runs with one
process per GPU (``bench.py --gpus N`` checks it against a float32 computation
over all ranks' rows before timing anything)."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _create(max_floats, n_ranks, rank):
    from evograd_b200 import _cabi

    handle = (ctypes.c_ubyte * 64)()
    x = ctypes.c_void_p()
    _cabi.call("evg_exchange_create", max_floats, n_ranks, rank, ctypes.byref(x),
               ctypes.cast(handle, ctypes.c_void_p))
    return x, bytes(handle)


def _sum_round(x, partial, dtype):
    from evograd_b200 import _cabi

    out = torch.empty(partial.shape, dtype=dtype, device=partial.device)
    out32 = torch.empty_like(partial)
    en = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    _cabi.call("evg_exchange_sum_round", x, partial.data_ptr(), partial.numel(), out.data_ptr(),
               en, out32.data_ptr(), torch.cuda.current_stream().cuda_stream)
    return out, out32


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_one_rank_sum_is_the_rounded_input(dtype):
    from evograd_b200 import _cabi, ops

    x, handle = _create(8192, 1, 0)
    try:
        assert any(handle)
        for seed, n in ((1, 8192), (2, 4096), (3, 7)):  # consecutive steps alternate the slots
            g = torch.Generator(device="cuda").manual_seed(seed)
            partial = torch.randn(n, device="cuda", generator=g) * 37.0
            out, out32 = _sum_round(x, partial, dtype)
            assert torch.equal(out32, partial)
            assert torch.equal(out, ops.cast_from_f32(partial, dtype))
        ops.device_status()
    finally:
        _cabi.call("evg_exchange_destroy", x)


def test_one_rank_sum_inside_a_replayed_graph():
    from evograd_b200 import _cabi, ops

    x, _ = _create(2 * 4096, 1, 0)
    try:
        partial = torch.randn(2, 4096, device="cuda")
        _sum_round(x, partial, torch.bfloat16)  # eager first: nothing lazy left for capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            outs = [_sum_round(x, partial, torch.bfloat16)[0] for _ in range(3)]  # odd count
        for _ in range(4):  # the slot parity differs from replay to replay
            partial.normal_()
            graph.replay()
            torch.cuda.synchronize()
            for o in outs:
                assert torch.equal(o, partial.to(torch.bfloat16))
        ops.device_status()
    finally:
        _cabi.call("evg_exchange_destroy", x)


def test_a_peer_that_never_arrives_ends_in_a_timeout_status():
    """Rank 0 of two, wired to a second buffer whose flag nothing ever sets: the
    kernel gives up after its cycle budget, returns, and the sticky status reports
    it; the context keeps working."""
    from evograd_b200 import _cabi, ops
    from evograd_b200._cabi import EvgError

    n = 1024
    x, _ = _create(n, 2, 0)
    silent = torch.zeros(48 * (n * 4 + 256) + 64 * 1024, device="cuda", dtype=torch.uint8)
    try:
        peers = (ctypes.c_void_p * 2)(_cabi.lib.evg_exchange_buffer(x), silent.data_ptr())
        _cabi.call("evg_exchange_connect_local", x, peers)
        _cabi.call("evg_exchange_set_wait_limit", x, 2_000_000)
        partial = torch.ones(n, device="cuda")
        _sum_round(x, partial, torch.float32)
        with pytest.raises(EvgError, match="EVG_ETIMEOUT"):
            ops.device_status()
        ops.device_status()  # cleared by the read above
        y, _ = ops.softmax_fwd(torch.randn(4, 64, device="cuda")), None
        assert torch.isfinite(y[0] if isinstance(y, tuple) else y).all()
    finally:
        _cabi.call("evg_exchange_destroy", x)


class _Handle:
    def __init__(self, x):
        self.handle = x


@pytest.mark.parametrize("op,rows,hidden,dtype", [
    ("layernorm", 700, 4096, torch.bfloat16), ("rmsnorm", 700, 4096, torch.bfloat16),
    ("layernorm", 33, 1000, torch.float32), ("rmsnorm", 2049, 1024, torch.float16),
])
def test_fused_column_reduce_and_exchange_with_one_rank(op, rows, hidden, dtype):
    """With one rank the sum over ranks is the rank's own sum: the fused second stage
    must give the bits of the plain backward, step after step (the slots alternate)."""
    from evograd_b200 import _cabi, ops

    x_h, _ = _create(2 * hidden, 1, 0)
    try:
        for seed in (1, 2, 3):
            g = torch.Generator(device="cuda").manual_seed(seed)
            x = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
            dy = torch.randn(rows, hidden, device="cuda", generator=g).to(dtype)
            w = torch.randn(hidden, device="cuda", generator=g).to(dtype)
            if op == "layernorm":
                b = torch.randn(hidden, device="cuda", generator=g).to(dtype)
                _, mean, rstd = ops.layernorm_fwd(x, w, b, 1e-5)
                ref = ops.layernorm_bwd(dy, x, w, mean, rstd)
                got = ops.layernorm_bwd(dy, x, w, mean, rstd, exchange=_Handle(x_h))
            else:
                _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
                ref = ops.rmsnorm_bwd(dy, x, w, rstd)
                got = ops.rmsnorm_bwd(dy, x, w, rstd, exchange=_Handle(x_h))
            for a, b_ in zip(ref, got):
                assert torch.equal(a, b_)
        ops.device_status()
    finally:
        _cabi.call("evg_exchange_destroy", x_h)


def test_fused_exchange_gives_up_on_a_silent_peer():
    from evograd_b200 import _cabi, ops
    from evograd_b200._cabi import EvgError

    hidden = 1024
    x_h, _ = _create(2 * hidden, 2, 0)
    silent = torch.zeros(48 * (2 * hidden * 4 + 256) + 64 * 1024, device="cuda", dtype=torch.uint8)
    try:
        peers = (ctypes.c_void_p * 2)(_cabi.lib.evg_exchange_buffer(x_h), silent.data_ptr())
        _cabi.call("evg_exchange_connect_local", x_h, peers)
        _cabi.call("evg_exchange_set_wait_limit", x_h, 2_000_000)
        x = torch.randn(64, hidden, device="cuda").to(torch.bfloat16)
        w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
        _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
        ops.rmsnorm_bwd(x, x, w, rstd, exchange=_Handle(x_h))
        with pytest.raises(EvgError, match="EVG_ETIMEOUT"):
            ops.device_status()
        ops.device_status()
        dx, dw = ops.rmsnorm_bwd(x, x, w, rstd)  # the context keeps working
        assert torch.isfinite(dx.float()).all() and torch.isfinite(dw.float()).all()
    finally:
        _cabi.call("evg_exchange_destroy", x_h)


def test_argument_checks():
    from evograd_b200 import _cabi

    handle = (ctypes.c_ubyte * 64)()
    x = ctypes.c_void_p()
    h = ctypes.cast(handle, ctypes.c_void_p)
    assert _cabi.lib.evg_exchange_create(0, 1, 0, ctypes.byref(x), h) == -1
    assert _cabi.lib.evg_exchange_create(16, 9, 0, ctypes.byref(x), h) == -1
    assert _cabi.lib.evg_exchange_create(16, 2, 2, ctypes.byref(x), h) == -1
    x, _ = _create(16, 2, 1)
    try:
        p = torch.zeros(16, device="cuda")
        # peers not connected yet
        assert _cabi.lib.evg_exchange_sum_round(x, p.data_ptr(), 16, p.data_ptr(), 0, None, None) == -8
    finally:
        _cabi.call("evg_exchange_destroy", x)
