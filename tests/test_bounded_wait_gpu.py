"""A device-side wait that nothing satisfies gives up after its cycle budget,
the kernel returns, the host reads EVG_ETIMEOUT, and the context keeps working.
The self-test kernel uses the same wait helper as every product kernel that
waits on an mbarrier; nothing here faults or spins without a bound."""

import pytest
import torch

from oracle import autograd_oracle as ao

pytestmark = pytest.mark.gpu


def test_wait_gives_up_and_the_context_stays_usable():
    from evograd_b200 import ops
    from evograd_b200._cabi import EvgError

    ops.device_status()  # clean to start with
    word = ops.selftest_bounded_wait(limit_cycles=2_000_000)  # about a millisecond
    assert word == 901
    with pytest.raises(EvgError, match="EVG_ETIMEOUT"):
        ops.device_status()
    ops.device_status()  # reading it cleared it

    # the same context still computes correct results afterwards
    inputs = ao.make_inputs("rmsnorm", dict(rows=64, hidden=512), "bfloat16")
    y, _ = ops.rmsnorm_fwd(inputs["x"].cuda(), inputs["weight"].cuda(), inputs["eps"])
    ref = ao.rmsnorm_forward(inputs["x"], inputs["weight"], inputs["eps"])
    assert torch.allclose(y.cpu().float(), ref.float(), atol=1e-2, rtol=1.6e-2)


def test_limit_is_validated():
    from evograd_b200 import _cabi
    from evograd_b200._cabi import EvgError

    for bad in (0, -5, 10**12):
        with pytest.raises(EvgError, match="EVG_EBADSHAPE"):
            _cabi.call("evg_selftest_bounded_wait", bad, None, None)
