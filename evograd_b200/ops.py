"""Tensor-level entry points: validate, allocate outputs with torch, enqueue the
C-ABI kernels on the current CUDA stream. No arithmetic happens in Python and
there is no non-CUDA path: a CPU tensor raises.
"""

from __future__ import annotations

import ctypes
import math

import torch

from . import _cabi
from ._cabi import EVG_BF16, EVG_F16, EVG_F32, RopeTensor, call, lib

_DTYPES = {torch.float32: EVG_F32, torch.float16: EVG_F16, torch.bfloat16: EVG_BF16}


def _dtype_enum(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32/float16/bfloat16") from None


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if not torch.is_tensor(t):
            raise TypeError(f"expected a tensor, got {type(t).__name__}")
        if not t.is_cuda:
            raise RuntimeError(
                "evograd_b200 kernels run on CUDA (sm_100a) tensors only; there is no CPU path"
            )
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _p(t) -> int | None:
    return None if t is None else t.data_ptr()


def _same(name_a, a, name_b, b, *, shape=True, dtype=True):
    if shape and tuple(a.shape) != tuple(b.shape):
        raise ValueError(f"{name_a} {tuple(a.shape)} and {name_b} {tuple(b.shape)} differ in shape")
    if dtype and a.dtype != b.dtype:
        raise ValueError(f"{name_a} is {a.dtype} but {name_b} is {b.dtype}")


def _rows_view(t: torch.Tensor, cols: int) -> torch.Tensor:
    return t.contiguous().view(-1, cols)


# ------------------------------------------------------------------ softmax
def softmax_fwd(x: torch.Tensor) -> torch.Tensor:
    dev = _require_cuda(x)
    if x.ndim < 1:
        raise ValueError("softmax needs at least one dimension")
    cols = x.shape[-1]
    x2 = _rows_view(x, cols)
    y = torch.empty_like(x2)
    if x2.numel() == 0:
        return y.view(x.shape)
    with torch.cuda.device(dev):
        call("evg_softmax_fwd", x2.data_ptr(), y.data_ptr(), x2.shape[0], cols, _dtype_enum(x),
             _stream(dev))
    return y.view(x.shape)


def softmax_bwd(y: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    dev = _require_cuda(y, dy)
    _same("y", y, "dy", dy)
    cols = y.shape[-1]
    y2, g2 = _rows_view(y, cols), _rows_view(dy, cols)
    dx = torch.empty_like(y2)
    if y2.numel() == 0:
        return dx.view(y.shape)
    with torch.cuda.device(dev):
        call("evg_softmax_bwd", y2.data_ptr(), g2.data_ptr(), dx.data_ptr(), y2.shape[0], cols,
             _dtype_enum(y), _stream(dev))
    return dx.view(y.shape)


# ----------------------------------------------------------- layernorm / rmsnorm
def _check_param(name: str, p: torch.Tensor, x: torch.Tensor):
    if p.ndim != 1 or p.shape[0] != x.shape[-1]:
        raise ValueError(f"{name} must be 1-D of length {x.shape[-1]}, got {tuple(p.shape)}")
    if p.dtype != x.dtype:
        raise ValueError(f"{name} is {p.dtype} but x is {x.dtype}")


def layernorm_fwd(x, weight, bias, eps: float = 1e-5):
    """Returns ``(y, mean, rstd)``; mean and rstd are float32 ``[rows]``."""
    dev = _require_cuda(x, weight, bias)
    _check_param("weight", weight, x)
    _check_param("bias", bias, x)
    hidden = x.shape[-1]
    x2 = _rows_view(x, hidden)
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    mean = torch.empty(rows, device=dev, dtype=torch.float32)
    rstd = torch.empty(rows, device=dev, dtype=torch.float32)
    if rows == 0:
        return y.view(x.shape), mean, rstd
    with torch.cuda.device(dev):
        call("evg_layernorm_fwd", x2.data_ptr(), weight.contiguous().data_ptr(),
             bias.contiguous().data_ptr(), y.data_ptr(), mean.data_ptr(), rstd.data_ptr(), rows,
             hidden, float(eps), _dtype_enum(x), _stream(dev))
    return y.view(x.shape), mean, rstd


def layernorm_bwd(dy, x, weight, mean, rstd, *, partials_f32: bool = False, exchange=None):
    """Returns ``(dx, dweight, dbias)``.

    With ``partials_f32`` the parameter gradients come back as ONE float32
    tensor ``[2, hidden]`` (row 0 dweight, row 1 dbias) instead of two tensors in
    the parameter dtype, for callers that sum them across ranks before rounding:
    ``(dx, dwdb_f32, None)``. With ``exchange`` (a connected
    :class:`evograd_b200.sharded.PeerExchange`; x and dy are this rank's row
    shard) dweight / dbias are the sums over ALL ranks' rows, formed inside the
    second stage of the column reduction, rounded once, identical on every rank.
    """
    dev = _require_cuda(dy, x, weight, mean, rstd)
    _same("dy", dy, "x", x)
    _check_param("weight", weight, x)
    hidden = x.shape[-1]
    x2, g2 = _rows_view(x, hidden), _rows_view(dy, hidden)
    rows = x2.shape[0]
    if mean.numel() != rows or rstd.numel() != rows or mean.dtype != torch.float32 \
            or rstd.dtype != torch.float32:
        raise ValueError("mean/rstd must be float32 with one entry per row")
    dx = torch.empty_like(x2)
    en = _dtype_enum(x)
    if rows == 0:
        z = torch.zeros(hidden, device=dev, dtype=x.dtype)
        if partials_f32:
            return dx.view(x.shape), torch.zeros(2, hidden, device=dev, dtype=torch.float32), None
        return dx.view(x.shape), z, z.clone()
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_layernorm_bwd_workspace_bytes(rows, hidden, en)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        if exchange is not None and not partials_f32:
            dwdb2 = torch.empty(2, hidden, device=dev, dtype=x.dtype)
            call("evg_layernorm_bwd_exchange", g2.data_ptr(), x2.data_ptr(),
                 weight.contiguous().data_ptr(), mean.contiguous().data_ptr(),
                 rstd.contiguous().data_ptr(), dx.data_ptr(), dwdb2[0].data_ptr(),
                 dwdb2[1].data_ptr(), ws.data_ptr(), ws_bytes, rows, hidden, en, exchange.handle,
                 _stream(dev))
            return dx.view(x.shape), dwdb2[0], dwdb2[1]
        if partials_f32:
            dwdb = torch.empty(2, hidden, device=dev, dtype=torch.float32)
            dweight = dbias = None
        else:
            dwdb = None
            dweight = torch.empty(hidden, device=dev, dtype=x.dtype)
            dbias = torch.empty(hidden, device=dev, dtype=x.dtype)
        call("evg_layernorm_bwd", g2.data_ptr(), x2.data_ptr(), weight.contiguous().data_ptr(),
             mean.contiguous().data_ptr(), rstd.contiguous().data_ptr(), dx.data_ptr(),
             _p(dweight), _p(dbias), _p(dwdb), ws.data_ptr(), ws_bytes, rows, hidden, en,
             _stream(dev))
    if partials_f32:
        return dx.view(x.shape), dwdb, None
    return dx.view(x.shape), dweight, dbias


def rmsnorm_fwd(x, weight, eps: float = 1e-5):
    """Returns ``(y, rstd)``; rstd is float32 ``[rows]``."""
    dev = _require_cuda(x, weight)
    _check_param("weight", weight, x)
    hidden = x.shape[-1]
    x2 = _rows_view(x, hidden)
    rows = x2.shape[0]
    y = torch.empty_like(x2)
    rstd = torch.empty(rows, device=dev, dtype=torch.float32)
    if rows == 0:
        return y.view(x.shape), rstd
    with torch.cuda.device(dev):
        call("evg_rmsnorm_fwd", x2.data_ptr(), weight.contiguous().data_ptr(), y.data_ptr(),
             rstd.data_ptr(), rows, hidden, float(eps), _dtype_enum(x), _stream(dev))
    return y.view(x.shape), rstd


def rmsnorm_bwd(dy, x, weight, rstd, *, partials_f32: bool = False, exchange=None):
    """Returns ``(dx, dweight)``; ``dweight`` is float32 when ``partials_f32``. With
    ``exchange`` (see :func:`layernorm_bwd`) dweight is the sum over all ranks' rows."""
    dev = _require_cuda(dy, x, weight, rstd)
    _same("dy", dy, "x", x)
    _check_param("weight", weight, x)
    hidden = x.shape[-1]
    x2, g2 = _rows_view(x, hidden), _rows_view(dy, hidden)
    rows = x2.shape[0]
    if rstd.numel() != rows or rstd.dtype != torch.float32:
        raise ValueError("rstd must be float32 with one entry per row")
    dx = torch.empty_like(x2)
    en = _dtype_enum(x)
    out_dtype = torch.float32 if partials_f32 else x.dtype
    if rows == 0:
        return dx.view(x.shape), torch.zeros(hidden, device=dev, dtype=out_dtype)
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_rmsnorm_bwd_workspace_bytes(rows, hidden, en)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        dweight = torch.empty(hidden, device=dev, dtype=out_dtype)
        if exchange is not None and not partials_f32:
            call("evg_rmsnorm_bwd_exchange", g2.data_ptr(), x2.data_ptr(),
                 weight.contiguous().data_ptr(), rstd.contiguous().data_ptr(), dx.data_ptr(),
                 dweight.data_ptr(), ws.data_ptr(), ws_bytes, rows, hidden, en, exchange.handle,
                 _stream(dev))
            return dx.view(x.shape), dweight
        call("evg_rmsnorm_bwd", g2.data_ptr(), x2.data_ptr(), weight.contiguous().data_ptr(),
             rstd.contiguous().data_ptr(), dx.data_ptr(),
             None if partials_f32 else dweight.data_ptr(),
             dweight.data_ptr() if partials_f32 else None, ws.data_ptr(), ws_bytes, rows, hidden,
             en, _stream(dev))
    return dx.view(x.shape), dweight


def fused_add_rmsnorm_fwd(x, residual, weight, eps: float = 1e-6):
    """``out = rmsnorm(x + residual) * weight`` with the reference's rounding points
    (ops/level2/fused_add_rms_norm/forward_ref.py:6-14). Returns ``(out, rstd)``;
    rstd is float32 ``[rows]``; the sum itself is not kept."""
    dev = _require_cuda(x, residual, weight)
    _same("x", x, "residual", residual)
    _check_param("weight", weight, x)
    hidden = x.shape[-1]
    x2, r2 = _rows_view(x, hidden), _rows_view(residual, hidden)
    rows = x2.shape[0]
    out = torch.empty_like(x2)
    rstd = torch.empty(rows, device=dev, dtype=torch.float32)
    if rows == 0:
        return out.view(x.shape), rstd
    with torch.cuda.device(dev):
        call("evg_fused_add_rmsnorm_fwd", x2.data_ptr(), r2.data_ptr(),
             weight.contiguous().data_ptr(), out.data_ptr(), rstd.data_ptr(), rows, hidden,
             float(eps), _dtype_enum(x), _stream(dev))
    return out.view(x.shape), rstd


def fused_add_rmsnorm_bwd(dout, x, residual, weight, rstd, *, partials_f32: bool = False):
    """Returns ``(dx, dweight)``; the gradient of ``residual`` equals ``dx``.
    ``dweight`` is float32 when ``partials_f32``."""
    dev = _require_cuda(dout, x, residual, weight, rstd)
    _same("dout", dout, "x", x)
    _same("x", x, "residual", residual)
    _check_param("weight", weight, x)
    hidden = x.shape[-1]
    x2, r2, g2 = _rows_view(x, hidden), _rows_view(residual, hidden), _rows_view(dout, hidden)
    rows = x2.shape[0]
    if rstd.numel() != rows or rstd.dtype != torch.float32:
        raise ValueError("rstd must be float32 with one entry per row")
    dx = torch.empty_like(x2)
    en = _dtype_enum(x)
    out_dtype = torch.float32 if partials_f32 else x.dtype
    if rows == 0:
        return dx.view(x.shape), torch.zeros(hidden, device=dev, dtype=out_dtype)
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_fused_add_rmsnorm_bwd_workspace_bytes(rows, hidden, en)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        dweight = torch.empty(hidden, device=dev, dtype=out_dtype)
        call("evg_fused_add_rmsnorm_bwd", g2.data_ptr(), x2.data_ptr(), r2.data_ptr(),
             weight.contiguous().data_ptr(), rstd.contiguous().data_ptr(), dx.data_ptr(),
             None if partials_f32 else dweight.data_ptr(),
             dweight.data_ptr() if partials_f32 else None, ws.data_ptr(), ws_bytes, rows, hidden,
             en, _stream(dev))
    return dx.view(x.shape), dweight


def cast_from_f32(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Round a float32 tensor to ``dtype`` (after an all-reduce of partial sums)."""
    dev = _require_cuda(src)
    if src.dtype != torch.float32:
        raise TypeError("cast_from_f32 expects float32")
    src = src.contiguous()
    dst = torch.empty(src.shape, device=dev, dtype=dtype)
    with torch.cuda.device(dev):
        call("evg_cast_from_f32", src.data_ptr(), dst.data_ptr(), src.numel(), _DTYPES[dtype],
             _stream(dev))
    return dst


# ------------------------------------------------------------ swiglu / geglu
def _glu_fwd(symbol, a, b):
    dev = _require_cuda(a, b)
    _same("a", a, "b", b)
    a2, b2 = a.contiguous(), b.contiguous()
    c = torch.empty_like(a2)
    if a2.numel() == 0:
        return c
    with torch.cuda.device(dev):
        call(symbol, a2.data_ptr(), b2.data_ptr(), c.data_ptr(), a2.numel(),
             _dtype_enum(a), _stream(dev))
    return c


def _glu_bwd(symbol, dc, a, b, in_place):
    dev = _require_cuda(dc, a, b)
    _same("a", a, "b", b)
    _same("dc", dc, "a", a)
    dc2 = dc.contiguous()
    if in_place:
        if not (a.is_contiguous() and b.is_contiguous()):
            raise ValueError("in_place backward needs contiguous a and b")
        a2, b2, da, db = a, b, a, b
    else:
        a2, b2 = a.contiguous(), b.contiguous()
        da, db = torch.empty_like(a2), torch.empty_like(b2)
    if a2.numel() == 0:
        return da, db
    with torch.cuda.device(dev):
        call(symbol, dc2.data_ptr(), a2.data_ptr(), b2.data_ptr(), da.data_ptr(),
             db.data_ptr(), a2.numel(), _dtype_enum(a), _stream(dev))
    return da, db


def swiglu_fwd(a, b):
    return _glu_fwd("evg_swiglu_fwd", a, b)


def swiglu_bwd(dc, a, b, *, in_place: bool = False):
    """Returns ``(da, db)``. ``in_place`` writes them over ``a`` and ``b`` (which
    must then be contiguous), as the swiglu declaration permits."""
    return _glu_bwd("evg_swiglu_bwd", dc, a, b, in_place)


def geglu_fwd(a, b):
    """c = gelu_tanh(a) * b (ops/level1/geglu/forward_ref.py:6-9)."""
    return _glu_fwd("evg_geglu_fwd", a, b)


def geglu_bwd(dc, a, b, *, in_place: bool = False):
    """Returns ``(da, db)`` of the geglu pair; ``in_place`` as for swiglu."""
    return _glu_bwd("evg_geglu_bwd", dc, a, b, in_place)


# --------------------------------------------------------------------- rope
def _rope_launch(xs, layout: str, cos, sin, inverse: bool, outs=None):
    """Rotate 1 or 2 tensors in one launch. ``layout`` is "bhtd" or "bthd" and names
    the axis order of the tensors' SHAPES; inputs and outputs may be strided views
    (last dimension contiguous), so a rotation can also change the memory layout
    (for example read [B, T, H, D] memory through a transposed view and write
    contiguous [B, H, T, D]). ``outs`` supplies the output tensors."""
    dev = _require_cuda(*xs, cos, sin)
    if layout not in ("bhtd", "bthd"):
        raise ValueError(f"layout must be 'bhtd' or 'bthd', got {layout!r}")
    x0 = xs[0]
    if any(x.ndim != 4 for x in xs):
        raise ValueError("rope expects 4-D tensors")
    t_axis, h_axis = (2, 1) if layout == "bhtd" else (1, 2)
    batch, tokens, head_dim = x0.shape[0], x0.shape[t_axis], x0.shape[3]
    if head_dim % 2:
        raise ValueError(f"rope needs an even head_dim, got {head_dim}")
    for x in xs[1:]:
        if x.shape[0] != batch or x.shape[t_axis] != tokens or x.shape[3] != head_dim \
                or x.dtype != x0.dtype:
            raise ValueError("tensors rotated together must share batch, tokens, head_dim, dtype")
    if cos.shape != sin.shape or cos.dtype != sin.dtype or cos.ndim != 2 or cos.shape[0] != tokens:
        raise ValueError(f"cos/sin must both be [tokens, head_dim or head_dim/2]; got "
                         f"{tuple(cos.shape)} and {tuple(sin.shape)}")
    if cos.shape[1] not in (head_dim, head_dim // 2):
        raise ValueError(f"table width {cos.shape[1]} is neither head_dim nor head_dim/2")
    cos, sin = cos.contiguous(), sin.contiguous()
    arr = (RopeTensor * len(xs))()
    given, outs = outs, []
    keep = []
    for i, x in enumerate(xs):
        if x.stride(3) != 1:
            x = x.contiguous()
        keep.append(x)
        if given is None:
            y = torch.empty(x.shape, device=dev, dtype=x.dtype)
        else:
            y = given[i]
            if tuple(y.shape) != tuple(x.shape) or y.dtype != x.dtype or y.stride(3) != 1 \
                    or y.device != x.device:
                raise ValueError("rope output must match the input's shape, dtype and device and "
                                 "have a contiguous last dimension")
        outs.append(y)
        arr[i] = RopeTensor(x.data_ptr(), y.data_ptr(), x.shape[h_axis], x.stride(0),
                            x.stride(h_axis), x.stride(t_axis), y.stride(0), y.stride(h_axis),
                            y.stride(t_axis))
    with torch.cuda.device(dev):
        call("evg_rope", arr, len(xs), cos.data_ptr(), sin.data_ptr(), batch, tokens, head_dim,
             cos.shape[1], _dtype_enum(cos), _dtype_enum(x0), 1 if inverse else 0, _stream(dev))
    return outs


def rope_fwd(x, cos, sin, *, layout: str = "bhtd", out=None):
    return _rope_launch([x], layout, cos, sin, False, None if out is None else [out])[0]


def rope_bwd(dy, cos, sin, *, layout: str = "bhtd", out=None):
    return _rope_launch([dy], layout, cos, sin, True, None if out is None else [out])[0]


def rope_qk_fwd(q, k, cos, sin, *, layout: str = "bthd", outs=None):
    """Rotate q and k (possibly different head counts) in one launch."""
    return tuple(_rope_launch([q, k], layout, cos, sin, False, outs))


def rope_qk_bwd(dq, dk, cos, sin, *, layout: str = "bthd", outs=None):
    return tuple(_rope_launch([dq, dk], layout, cos, sin, True, outs))


# --------------------------------------------------------- causal attention
def _check_qkv(q, k, v):
    if q.ndim != 4:
        raise ValueError(f"causal attention expects [B, H, S, D], got {tuple(q.shape)}")
    _same("q", q, "k", k)
    _same("q", q, "v", v)
    if q.dtype not in (torch.bfloat16, torch.float16):
        raise TypeError(f"causal attention runs in bfloat16/float16, got {q.dtype}")


def causal_attention_fwd(q, k, v, scale: float | None = None):
    """Returns ``(o, lse)`` with ``lse`` float32 ``[B, H, S]``."""
    dev = _require_cuda(q, k, v)
    _check_qkv(q, k, v)
    B, H, S, D = q.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    q2, k2, v2 = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q2)
    lse = torch.empty(B, H, S, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        call("evg_causal_attention_fwd", q2.data_ptr(), k2.data_ptr(), v2.data_ptr(), o.data_ptr(),
             lse.data_ptr(), B, H, S, D, float(scale), _dtype_enum(q), _stream(dev))
    return o, lse


def causal_attention_bwd(do, q, k, v, o, lse, scale: float | None = None):
    """Returns ``(dq, dk, dv)``."""
    dev = _require_cuda(do, q, k, v, o, lse)
    _check_qkv(q, k, v)
    _same("do", do, "q", q)
    _same("o", o, "q", q)
    B, H, S, D = q.shape
    if lse.dtype != torch.float32 or tuple(lse.shape) != (B, H, S):
        raise ValueError("lse must be float32 [B, H, S]")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    do2, q2, k2, v2, o2 = (t.contiguous() for t in (do, q, k, v, o))
    dq, dk, dv = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
    en = _dtype_enum(q)
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_causal_attention_bwd_workspace_bytes(B, H, S, D, en)
        ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
        call("evg_causal_attention_bwd", do2.data_ptr(), q2.data_ptr(), k2.data_ptr(),
             v2.data_ptr(), o2.data_ptr(), lse.contiguous().data_ptr(), dq.data_ptr(),
             dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws_bytes, B, H, S, D, float(scale), en,
             _stream(dev))
    return dq, dk, dv


def _check_gqa(q, k, v):
    if q.ndim != 4 or k.ndim != 4:
        raise ValueError(f"attention expects [B, H, S, D], got {tuple(q.shape)} / {tuple(k.shape)}")
    _same("k", k, "v", v)
    if q.dtype != k.dtype or q.device != k.device:
        raise ValueError("q and k must share dtype and device")
    B, Hq, S, D = q.shape
    if k.shape[0] != B or k.shape[2] != S or k.shape[3] != D or Hq % k.shape[1] != 0:
        raise ValueError(f"q {tuple(q.shape)} and k/v {tuple(k.shape)} do not form grouped-query "
                         "attention (same B, S, D; query heads a multiple of k/v heads)")
    return B, Hq, k.shape[1], S, D


def causal_gqa_attention_fwd(q, k, v, scale: float | None = None):
    """Causal attention with ``Hq`` query heads sharing ``Hkv`` key/value heads:
    q ``[B, Hq, S, D]``, k/v ``[B, Hkv, S, D]`` (any of float32 / float16 / bfloat16,
    D <= 256; 16-bit with D in {64, 128} runs on the tensor cores). Returns
    ``(o, lse)`` with ``lse`` float32 ``[B, Hq, S]``."""
    dev = _require_cuda(q, k, v)
    B, Hq, Hkv, S, D = _check_gqa(q, k, v)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    q2, k2, v2 = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q2)
    lse = torch.empty(B, Hq, S, device=dev, dtype=torch.float32)
    if q2.numel() == 0:
        return o, lse
    with torch.cuda.device(dev):
        call("evg_causal_gqa_attention_fwd", q2.data_ptr(), k2.data_ptr(), v2.data_ptr(),
             o.data_ptr(), lse.data_ptr(), B, Hq, Hkv, S, D, float(scale), _dtype_enum(q),
             _stream(dev))
    return o, lse


def causal_gqa_attention_bwd(do, q, k, v, o, lse, scale: float | None = None):
    """Returns ``(dq, dk, dv)``; dk/dv are summed over the query heads of each group."""
    dev = _require_cuda(do, q, k, v, o, lse)
    B, Hq, Hkv, S, D = _check_gqa(q, k, v)
    _same("do", do, "q", q)
    _same("o", o, "q", q)
    if lse.dtype != torch.float32 or tuple(lse.shape) != (B, Hq, S):
        raise ValueError("lse must be float32 [B, Hq, S]")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    do2, q2, k2, v2, o2 = (t.contiguous() for t in (do, q, k, v, o))
    dq, dk, dv = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
    if q2.numel() == 0:
        return dq, dk, dv
    en = _dtype_enum(q)
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_causal_gqa_attention_bwd_workspace_bytes(B, Hq, Hkv, S, D, en)
        ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
        call("evg_causal_gqa_attention_bwd", do2.data_ptr(), q2.data_ptr(), k2.data_ptr(),
             v2.data_ptr(), o2.data_ptr(), lse.contiguous().data_ptr(), dq.data_ptr(),
             dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws_bytes, B, Hq, Hkv, S, D, float(scale),
             en, _stream(dev))
    return dq, dk, dv


def _tensor_core_attention(q) -> bool:
    return q.dtype in (torch.float16, torch.bfloat16) and q.shape[-1] in (64, 128)


def causal_gqa_attention_fwd_tm(q, k, v_tm, scale: float | None = None):
    """:func:`causal_gqa_attention_fwd` for a decoder layer's layouts: ``v_tm`` is
    token-major ``[B, S, Hkv, D]`` (a view of its projection's output) and ``o`` comes
    back token-major ``[B, S, Hq, D]`` (what the output projection reads as
    ``[B*S, Hq*D]``); q and k are ``[B, H, S, D]``. The tensor-core kernels read and
    write those layouts directly; other shapes go through the head-major call and
    transposing copies."""
    dev = _require_cuda(q, k, v_tm)
    v = v_tm.transpose(1, 2)
    B, Hq, Hkv, S, D = _check_gqa(q, k, v)
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if not _tensor_core_attention(q) or q.numel() == 0:
        o, lse = causal_gqa_attention_fwd(q, k, v, scale)
        return o.transpose(1, 2).contiguous(), lse
    q2, k2, v2 = q.contiguous(), k.contiguous(), v_tm.contiguous()
    o = torch.empty(B, S, Hq, D, device=dev, dtype=q.dtype)
    lse = torch.empty(B, Hq, S, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev):
        call("evg_causal_gqa_attention_fwd_tm", q2.data_ptr(), k2.data_ptr(), v2.data_ptr(),
             o.data_ptr(), lse.data_ptr(), B, Hq, Hkv, S, D, float(scale), _dtype_enum(q),
             _stream(dev))
    return o, lse


def causal_gqa_attention_bwd_tm(do_tm, q, k, v_tm, o_tm, lse, scale: float | None = None):
    """Backward for token-major ``do_tm`` / ``o_tm`` ``[B, S, Hq, D]`` and ``v_tm``
    ``[B, S, Hkv, D]``; returns ``(dq, dk, dv_tm)`` with ``dv_tm`` token-major and dq, dk
    head-major."""
    dev = _require_cuda(do_tm, q, k, v_tm, o_tm, lse)
    v = v_tm.transpose(1, 2)
    B, Hq, Hkv, S, D = _check_gqa(q, k, v)
    for name, t in (("do_tm", do_tm), ("o_tm", o_tm)):
        if tuple(t.shape) != (B, S, Hq, D) or t.dtype != q.dtype:
            raise ValueError(f"{name} must be [B, S, Hq, D] in the dtype of q")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    if not _tensor_core_attention(q) or q.numel() == 0:
        dq, dk, dv = causal_gqa_attention_bwd(do_tm.transpose(1, 2), q, k, v,
                                              o_tm.transpose(1, 2), lse, scale)
        return dq, dk, dv.transpose(1, 2).contiguous()
    do2, q2, k2, v2, o2 = (t.contiguous() for t in (do_tm, q, k, v_tm, o_tm))
    dq, dk = torch.empty_like(q2), torch.empty_like(k2)
    dv = torch.empty(B, S, Hkv, D, device=dev, dtype=q.dtype)
    en = _dtype_enum(q)
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_causal_gqa_attention_bwd_workspace_bytes(B, Hq, Hkv, S, D, en)
        ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
        call("evg_causal_gqa_attention_bwd_tm", do2.data_ptr(), q2.data_ptr(), k2.data_ptr(),
             v2.data_ptr(), o2.data_ptr(), lse.contiguous().data_ptr(), dq.data_ptr(),
             dk.data_ptr(), dv.data_ptr(), ws.data_ptr(), ws_bytes, B, Hq, Hkv, S, D, float(scale),
             en, _stream(dev))
    return dq, dk, dv


# ------------------------------------------------------------- evoattention
def _check_evo(q, k, v, res_mask, pair_bias):
    if q.ndim != 5:
        raise ValueError(f"evoattention expects [B, S, N, H, D], got {tuple(q.shape)}")
    _same("q", q, "k", k)
    _same("q", q, "v", v)
    B, S, N, H, D = q.shape
    if res_mask.dtype != torch.float32 or res_mask.numel() != B * S * N:
        raise ValueError(f"res_mask must be float32 with B*S*N entries ([B, S, 1, 1, N]), got "
                         f"{res_mask.dtype} {tuple(res_mask.shape)}")
    if pair_bias.dtype != torch.float32 or pair_bias.numel() != B * H * N * N:
        raise ValueError(f"pair_bias must be float32 with B*H*N*N entries ([B, 1, H, N, N]), got "
                         f"{pair_bias.dtype} {tuple(pair_bias.shape)}")
    return B, S, N, H, D


def evoattention_fwd(q, k, v, res_mask, pair_bias, scale: float | None = None):
    """EvoformerAttention forward (ops/level1/evoattention/forward_ref.py:22-49).
    Returns ``(o, lse)``; ``lse`` is float32 ``[B, S, H, N]``."""
    dev = _require_cuda(q, k, v, res_mask, pair_bias)
    B, S, N, H, D = _check_evo(q, k, v, res_mask, pair_bias)
    if scale is None:
        scale = D ** -0.5
    q2, k2, v2 = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q2)
    lse = torch.empty(B, S, H, N, device=dev, dtype=torch.float32)
    if q2.numel() == 0:
        return o, lse
    with torch.cuda.device(dev):
        call("evg_evoattention_fwd", q2.data_ptr(), k2.data_ptr(), v2.data_ptr(),
             res_mask.contiguous().data_ptr(), pair_bias.contiguous().data_ptr(), o.data_ptr(),
             lse.data_ptr(), B, S, N, H, D, float(scale), _dtype_enum(q), _stream(dev))
    return o, lse


def evoattention_bwd(do, q, k, v, res_mask, pair_bias, o, lse, scale: float | None = None):
    """Returns ``(dq, dk, dv, d_pair_bias)``; d_pair_bias is float32, shaped like pair_bias."""
    dev = _require_cuda(do, q, k, v, res_mask, pair_bias, o, lse)
    B, S, N, H, D = _check_evo(q, k, v, res_mask, pair_bias)
    _same("do", do, "q", q)
    _same("o", o, "q", q)
    if lse.dtype != torch.float32 or lse.numel() != B * S * H * N:
        raise ValueError("lse must be float32 [B, S, H, N]")
    if scale is None:
        scale = D ** -0.5
    do2, q2, k2, v2, o2 = (t.contiguous() for t in (do, q, k, v, o))
    dq, dk, dv = torch.empty_like(q2), torch.empty_like(k2), torch.empty_like(v2)
    dbias = torch.empty(pair_bias.shape, device=dev, dtype=torch.float32)
    if q2.numel() == 0:
        return dq, dk, dv, dbias.zero_()
    en = _dtype_enum(q)
    with torch.cuda.device(dev):
        ws_bytes = lib.evg_evoattention_bwd_workspace_bytes(B, S, N, H, D, en)
        ws = torch.empty(max(ws_bytes, 16), device=dev, dtype=torch.uint8)
        call("evg_evoattention_bwd", do2.data_ptr(), q2.data_ptr(), k2.data_ptr(), v2.data_ptr(),
             res_mask.contiguous().data_ptr(), pair_bias.contiguous().data_ptr(), o2.data_ptr(),
             lse.contiguous().data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
             dbias.data_ptr(), ws.data_ptr(), ws_bytes, B, S, N, H, D, float(scale), en,
             _stream(dev))
    return dq, dk, dv, dbias


def device_status(reset: bool = True) -> None:
    """Synchronise and raise :class:`EvgError` (EVG_ETIMEOUT) if a bounded device-side
    wait (attention, norm backward rings, wide softmax) gave up since the last reset."""
    call("evg_device_status", 1 if reset else 0)


def selftest_bounded_wait(limit_cycles: int = 2_000_000, device=None) -> int:
    """Launch the bounded-wait self-test (a wait nothing satisfies, given up after
    ``limit_cycles``) and return the abort word the block recorded. The sticky
    status is left set: the next :func:`device_status` raises EVG_ETIMEOUT once."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = torch.zeros(1, device=dev, dtype=torch.int32)
    with torch.cuda.device(dev):
        call("evg_selftest_bounded_wait", int(limit_cycles), word.data_ptr(), _stream(dev))
    return int(word.item())


def flush_l2(buffer: torch.Tensor) -> None:
    """Overwrite ``buffer`` (larger than L2) so cached lines of other tensors are evicted."""
    dev = _require_cuda(buffer)
    with torch.cuda.device(dev):
        call("evg_flush_l2", buffer.data_ptr(), buffer.numel() * buffer.element_size(),
             _stream(dev))
