"""ctypes binding of ``libevg_b200.so`` (the C ABI declared in ``include/evg_b200.h``).

Importing this module never builds or falls back: if the shared library is
missing or does not export a declared symbol the import raises, so a caller
can not end up on a slower path without noticing.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libevg_b200.so"

EVG_F32, EVG_F16, EVG_BF16 = 0, 1, 2

STATUS_NAMES = {
    0: "EVG_OK",
    -1: "EVG_EBADSHAPE",
    -2: "EVG_EALIGN",
    -3: "EVG_EDTYPE",
    -4: "EVG_ELAUNCH",
    -5: "EVG_ETIMEOUT",
    -6: "EVG_ENULL",
    -7: "EVG_EWORKSPACE",
    -8: "EVG_EUNSUPPORTED",
}


class EvgError(RuntimeError):
    """A C-ABI entry point returned a negative status."""

    def __init__(self, fn: str, code: int, message: str):
        self.fn, self.code, self.message = fn, code, message
        super().__init__(f"{fn} failed with {STATUS_NAMES.get(code, code)}: {message}")


class RopeTensor(ctypes.Structure):
    """Mirror of ``evg_rope_tensor``."""

    _fields_ = [
        ("x", c_void_p),
        ("y", c_void_p),
        ("heads", c_int64),
        ("x_stride_b", c_int64),
        ("x_stride_h", c_int64),
        ("x_stride_t", c_int64),
        ("y_stride_b", c_int64),
        ("y_stride_h", c_int64),
        ("y_stride_t", c_int64),
    ]


# name -> (restype, argtypes); every symbol include/evg_b200.h declares.
SIGNATURES = {
    "evg_abi_version": (c_int, []),
    "evg_last_error": (c_char_p, []),
    "evg_built_for_sm": (c_int, []),
    "evg_tune_set": (c_int, [c_char_p, c_int]),
    "evg_tune_get": (c_int, [c_char_p]),
    "evg_softmax_fwd": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "evg_softmax_bwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "evg_layernorm_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float,
         c_int, c_void_p],
    ),
    "evg_layernorm_bwd_workspace_bytes": (c_int64, [c_int64, c_int64, c_int]),
    "evg_layernorm_bwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p],
    ),
    "evg_rmsnorm_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int, c_void_p],
    ),
    "evg_rmsnorm_bwd_workspace_bytes": (c_int64, [c_int64, c_int64, c_int]),
    "evg_rmsnorm_bwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64,
         c_int64, c_int64, c_int, c_void_p],
    ),
    "evg_rmsnorm_bwd_noalloc": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
         c_int, c_void_p],
    ),
    "evg_fused_add_rmsnorm_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_float, c_int,
         c_void_p],
    ),
    "evg_fused_add_rmsnorm_bwd_workspace_bytes": (c_int64, [c_int64, c_int64, c_int]),
    "evg_fused_add_rmsnorm_bwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p],
    ),
    "evg_causal_gqa_attention_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
         c_int64, c_float, c_int, c_void_p],
    ),
    "evg_causal_gqa_attention_bwd_workspace_bytes": (
        c_int64, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int]
    ),
    "evg_causal_gqa_attention_bwd": (
        c_int,
        [c_void_p] * 10 + [c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int,
                           c_void_p],
    ),
    "evg_causal_gqa_attention_fwd_tm": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
         c_int64, c_float, c_int, c_void_p],
    ),
    "evg_causal_gqa_attention_bwd_tm": (
        c_int,
        [c_void_p] * 10 + [c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int,
                           c_void_p],
    ),
    "evg_evoattention_fwd": (
        c_int,
        [c_void_p] * 7 + [c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_void_p],
    ),
    "evg_evoattention_bwd_workspace_bytes": (
        c_int64, [c_int64, c_int64, c_int64, c_int64, c_int64, c_int]
    ),
    "evg_evoattention_bwd": (
        c_int,
        [c_void_p] * 13 + [c_int64, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int,
                           c_void_p],
    ),
    "evg_selftest_bounded_wait": (c_int, [c_int64, c_void_p, c_void_p]),
    "evg_swiglu_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "evg_swiglu_bwd": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]
    ),
    "evg_geglu_fwd": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "evg_geglu_bwd": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p]
    ),
    "evg_rope": (
        c_int,
        [ctypes.POINTER(RopeTensor), c_int, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
         c_int, c_int, c_int, c_void_p],
    ),
    "evg_causal_attention_fwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int64,
         c_float, c_int, c_void_p],
    ),
    "evg_causal_attention_bwd_workspace_bytes": (
        c_int64, [c_int64, c_int64, c_int64, c_int64, c_int]
    ),
    "evg_causal_attention_bwd": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_void_p, c_int64, c_int64, c_int64, c_int64, c_int64, c_float, c_int, c_void_p],
    ),
    "evg_exchange_create": (c_int, [c_int64, c_int, c_int, ctypes.POINTER(c_void_p), c_void_p]),
    "evg_exchange_connect": (c_int, [c_void_p, c_void_p]),
    "evg_exchange_connect_local": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "evg_exchange_buffer": (c_void_p, [c_void_p]),
    "evg_exchange_set_wait_limit": (c_int, [c_void_p, c_int64]),
    "evg_exchange_sum_round": (c_int, [c_void_p, c_void_p, c_int64, c_void_p, c_int, c_void_p,
                                       c_void_p]),
    "evg_exchange_destroy": (c_int, [c_void_p]),
    "evg_layernorm_bwd_exchange": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
         c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p],
    ),
    "evg_rmsnorm_bwd_exchange": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
         c_int64, c_int, c_void_p, c_void_p],
    ),
    "evg_device_status": (c_int, [c_int]),
    "evg_cast_from_f32": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "evg_flush_l2": (c_int, [c_void_p, c_int64, c_void_p]),
}


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m evograd_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(os.fspath(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as exc:
            raise ImportError(f"{LIB_PATH} does not export {name}") from exc
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def last_error() -> str:
    msg = lib.evg_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(fn_name: str, code: int) -> None:
    """Turn a negative status into :class:`EvgError` carrying the library's message."""
    if code != 0:
        raise EvgError(fn_name, code, last_error())


def call(fn_name: str, *args) -> None:
    check(fn_name, getattr(lib, fn_name)(*args))


def tune_set(key: str, value: int) -> None:
    call("evg_tune_set", key.encode(), int(value))


def tune_get(key: str) -> int:
    return int(lib.evg_tune_get(key.encode()))
