"""The allocation-free RMSNorm backward (``evg_rmsnorm_bwd_noalloc``).

Some users of this library run where they cannot ask CUDA for memory: a plug-in
whose host process owns all GPU memory, or a loop that must not hit the device
synchronisation a ``cudaMalloc`` can cause. For them the library carries its own
fixed scratch array. These tests drive that entry point through the C ABI, on
consecutive calls of different shapes (each call sees the previous call's
leftovers in the shared array), and require bit-identical results to the regular
entry point that takes a caller-provided workspace. They also check that the
call takes no device memory from the driver (free bytes as CUDA reports them, not
torch's own counter), that launch shapes which may want more partial rows than
the scratch holds still give the right answer, and that shapes beyond the
built-in scratch are refused with a clear message instead of being run.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

_ENUM = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def _inputs(rows, hidden, dtype, seed):
    from evograd_b200 import ops

    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, hidden, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    dy = torch.randn(rows, hidden, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", dtype=torch.float32, generator=g)).to(dtype)
    _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
    return x, dy, w, rstd


def _workspace_call(x, dy, w, rstd):
    from evograd_b200 import _cabi

    rows, hidden = x.shape
    en = _ENUM[x.dtype]
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    dw32 = torch.empty(hidden, device="cuda", dtype=torch.float32)
    ws_bytes = _cabi.lib.evg_rmsnorm_bwd_workspace_bytes(rows, hidden, en)
    ws = torch.empty(ws_bytes, device="cuda", dtype=torch.uint8)
    _cabi.call("evg_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
               dx.data_ptr(), dw.data_ptr(), dw32.data_ptr(), ws.data_ptr(), ws_bytes,
               rows, hidden, en, torch.cuda.current_stream().cuda_stream)
    return dx, dw, dw32


def _noalloc_call(x, dy, w, rstd, check_free_bytes=False):
    from evograd_b200 import _cabi

    rows, hidden = x.shape
    # outputs are allocated up front; the call itself gets no memory
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    dw32 = torch.empty(hidden, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    torch_before = torch.cuda.memory_allocated()
    _cabi.call("evg_rmsnorm_bwd_noalloc", dy.data_ptr(), x.data_ptr(), w.data_ptr(),
               rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), dw32.data_ptr(), rows, hidden,
               _ENUM[x.dtype], torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == torch_before
    if check_free_bytes:
        # what the driver itself reports: a cudaMalloc inside the library would show here
        assert torch.cuda.mem_get_info()[0] >= free_before
    return dx, dw, dw32


def _assert_same(ref, got, what):
    for name, a, b in zip(("dx", "dweight", "dweight_f32"), ref, got):
        # same kernels, same summation order: the tolerance the other tests use
        # for bit-reproducible paths is exact equality
        assert torch.equal(a, b), f"{name} differs for {what}"


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    # two consecutive calls; the second (smaller) one runs over the first one's leftovers
    for rows, hidden, dtype, seed in ((4096, 4096, torch.bfloat16, 11), (513, 1024, torch.float32, 12)):
        args = _inputs(rows, hidden, dtype, seed)
        _assert_same(_workspace_call(*args), _noalloc_call(*args), f"{rows}x{hidden} {dtype}")


def test_noalloc_takes_no_device_memory_from_the_driver():
    args = _inputs(1024, 4096, torch.bfloat16, 13)
    _noalloc_call(*args)  # first call on the device: module load, address look-up
    ref = _workspace_call(*args)
    got = _noalloc_call(*args, check_free_bytes=True)
    _assert_same(ref, got, "1024x4096 bf16 (second call)")


@pytest.mark.parametrize("rows,hidden,dtype", [
    (600, 8192, torch.bfloat16),   # the widest rows the built-in scratch takes
    (64, 8191, torch.float32),     # odd width: the multi-pass kernel
    (3, 4096, torch.bfloat16),     # fewer rows than blocks
])
def test_noalloc_edge_shapes(rows, hidden, dtype):
    args = _inputs(rows, hidden, dtype, rows + hidden)
    _assert_same(_workspace_call(*args), _noalloc_call(*args), f"{rows}x{hidden} {dtype}")


@pytest.mark.parametrize("knobs", [
    {"norm_bwd.blocks_per_sm": 3},
    {"norm_bwd.blocks_per_sm": 3, "norm_bwd.no_ring": 1},
    {"norm_bwd.blocks_per_sm": 4, "rows.force_generic": 1},
])
def test_noalloc_when_the_launch_shape_asks_for_more_partial_rows(knobs):
    """The scratch holds 320 partial rows of 8192 floats. With more blocks per SM
    allowed, a kernel variant that fits three or more blocks on an SM would want
    more partial rows than that (444 on a 148-SM device), and the entry point must
    then launch fewer blocks. Whether the limit binds depends on the variant's
    occupancy, so the two entry points may run different launch shapes (another
    summation order): dx must still be identical, dweight is held to the float32
    column sum with the bound the reduction tests use."""
    from evograd_b200 import _cabi

    rows, hidden = 1024, 8192
    args = _inputs(rows, hidden, torch.bfloat16, 17)
    old = {k: _cabi.tune_get(k) for k in knobs}
    for k, v in knobs.items():
        _cabi.tune_set(k, v)
    try:
        ref = _workspace_call(*args)
        got = _noalloc_call(*args)
    finally:
        for k, v in old.items():
            _cabi.tune_set(k, v)
    assert torch.equal(ref[0], got[0]), "dx must not depend on the launch shape"
    x, dy, _w, rstd = args
    terms = dy.float() * (x.float() * rstd[:, None])
    exact = terms.double().sum(0)
    bound = 1e-5 * terms.abs().double().sum(0) + 1e-6
    assert ((got[2].double() - exact).abs() <= bound).all()
    assert ((ref[2].double() - exact).abs() <= bound).all()


def test_noalloc_refuses_shapes_beyond_the_built_in_scratch():
    from evograd_b200 import _cabi
    from evograd_b200._cabi import EvgError

    hidden = 16384
    x = torch.zeros(2, hidden, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda", dtype=torch.float32)
    w = torch.ones(hidden, device="cuda", dtype=torch.bfloat16)
    dx = torch.empty_like(x)
    with pytest.raises(EvgError, match="EVG_EUNSUPPORTED") as info:
        _cabi.call("evg_rmsnorm_bwd_noalloc", x.data_ptr(), x.data_ptr(), w.data_ptr(),
                   rstd.data_ptr(), dx.data_ptr(), None, None, 2, hidden, 2, None)
    assert "8192" in str(info.value)
