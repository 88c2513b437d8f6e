"""Small stand-ins for pieces of evograd's benchmark harness that would
otherwise pull in Triton.

``L2Cache`` mirrors ``evograd.bench.fair.L2Cache`` (src/evograd/bench/fair.py:264-274):
an object whose ``clear()`` evicts the GPU's L2 between timed samples. The
reference borrows Triton's ``do_bench`` primitive (zeroing a 256 MB buffer); this
one overwrites a buffer of twice the device's L2 size with this package's own
flush kernel, so ``evograd bench`` / ``evograd suite`` can time these candidates
on a box without Triton.
"""

from __future__ import annotations

import torch

from . import ops


class L2Cache:
    """``clear()`` leaves no line of any other tensor in L2."""

    def __init__(self, device=None, min_bytes: int = 256 << 20):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        l2 = torch.cuda.get_device_properties(self.device).L2_cache_size
        self._cache = torch.empty(max(min_bytes, 2 * l2), device=self.device, dtype=torch.uint8)

    def clear(self) -> None:
        ops.flush_l2(self._cache)
