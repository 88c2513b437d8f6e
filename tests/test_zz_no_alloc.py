"""The allocation-free RMSNorm backward (``evg_rmsnorm_bwd_noalloc``).

Some users of this library run where they cannot ask CUDA for memory: a plug-in
whose host process owns all GPU memory, or a loop that must not hit the device
synchronisation a ``cudaMalloc`` can cause. For them the library carries its own
fixed scratch array. This test drives that entry point through the C ABI, twice
in a row on different shapes (the second call sees the first call's leftovers in
the shared array), and requires bit-identical results to the regular entry point
that takes a caller-provided workspace. It also checks that shapes beyond the
built-in scratch are refused with a clear message instead of being run.

The file name sorts last on purpose, so a run that stops at the first failure
has already executed every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(rows, hidden, dtype, seed):
    from evograd_b200 import _cabi, ops

    en = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, hidden, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    dy = torch.randn(rows, hidden, device="cuda", dtype=torch.float32, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden, device="cuda", dtype=torch.float32, generator=g)).to(dtype)
    _, rstd = ops.rmsnorm_fwd(x, w, 1e-6)
    stream = torch.cuda.current_stream().cuda_stream

    # regular entry point: caller-provided workspace
    dx_ref, dw_ref = torch.empty_like(x), torch.empty_like(w)
    dw32_ref = torch.empty(hidden, device="cuda", dtype=torch.float32)
    ws_bytes = _cabi.lib.evg_rmsnorm_bwd_workspace_bytes(rows, hidden, en)
    ws = torch.empty(ws_bytes, device="cuda", dtype=torch.uint8)
    _cabi.call("evg_rmsnorm_bwd", dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(),
               dx_ref.data_ptr(), dw_ref.data_ptr(), dw32_ref.data_ptr(), ws.data_ptr(), ws_bytes,
               rows, hidden, en, stream)

    # allocation-free entry point: outputs are allocated up front, the call itself gets none
    dx, dw = torch.empty_like(x), torch.empty_like(w)
    dw32 = torch.empty(hidden, device="cuda", dtype=torch.float32)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    _cabi.call("evg_rmsnorm_bwd_noalloc", dy.data_ptr(), x.data_ptr(), w.data_ptr(),
               rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), dw32.data_ptr(), rows, hidden, en,
               stream)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return (dx_ref, dw_ref, dw32_ref), (dx, dw, dw32)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    # two consecutive calls; the second (smaller) one runs over the first one's leftovers
    for rows, hidden, dtype, seed in ((4096, 4096, torch.bfloat16, 11), (513, 1024, torch.float32, 12)):
        ref, got = _run_both(rows, hidden, dtype, seed)
        for name, a, b in zip(("dx", "dweight", "dweight_f32"), ref, got):
            # same kernels, same summation order: the tolerance the other tests use
            # for bit-reproducible paths is exact equality
            assert torch.equal(a, b), f"{name} differs for rows={rows} hidden={hidden} {dtype}"


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
