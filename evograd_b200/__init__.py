"""evograd_b200: sm_100a autograd pairs (forward that chooses what to save,
backward that consumes it) for softmax, LayerNorm, RMSNorm, SwiGLU, RoPE and
causal attention, behind evograd's candidate-module interface.

Layout
    csrc/      CUDA kernels and the C ABI (``include/evg_b200.h``)
    _cabi.py   ctypes binding of the shared library
    ops.py     tensor-level wrappers: validate, allocate outputs, enqueue
    pairs/     one candidate module per operator, importable by file path by
               ``evograd verify`` / ``bench`` / ``suite``
    decls/     external declarations (a ``b200`` suite, ``causal_attention``)
    sharded.py row / batch-head sharding across ranks with the dW all-reduce
    timing.py  CUDA-event timing, L2 flush, roofline arithmetic
"""

__version__ = "0.1.0"
