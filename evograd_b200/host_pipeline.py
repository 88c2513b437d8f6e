"""Host-buffer pipeline for the row-wise autograd pairs.

A caller whose activations live in (pinned) host memory pays for PCIe twice per
step: inputs in, results out. Doing those copies back to back with the kernels
leaves each direction of the link idle half of the time. The row-wise
operators are independent per row, so :class:`HostRowPipeline` cuts the rows
into chunks and keeps three things in flight at once on three CUDA streams:

    copy-in  stream   chunk c+1: host -> device (x, dy, ...)
    compute  stream   chunk c  : forward + backward kernels
    copy-out stream   chunk c-1: device -> host (y, dx, ...)

Parameter gradients (LayerNorm / RMSNorm dweight, dbias) are summed over the
chunks in float32 on the device and rounded once at the end, exactly as the
multi-GPU path rounds after its all-reduce, so the result does not depend on
the chunk count beyond float32 summation order.

The reference has no host-memory path (its harness times device-resident
tensors, src/evograd/bench/harness.py); this is the end-to-end entry point a
user with host-resident activations calls, and what bench.py's ``e2e`` leg times.
"""

from __future__ import annotations

import torch

from . import ops
from .sharded import block_range


class HostRowPipeline:
    """``chunk_fn(dev_rows: dict, params: dict) -> (row_outputs: dict, partial | None)``
    runs one forward + backward on a chunk of rows that is already on the device.
    ``partial`` is a float32 tensor of parameter-gradient partial sums."""

    def __init__(self, chunk_fn, *, chunks: int = 8, slots: int = 3, device=None):
        if chunks < 1 or slots < 2:
            raise ValueError("need at least one chunk and two buffer slots")
        self.chunk_fn = chunk_fn
        self.chunks = chunks
        self.slots = slots
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None \
            else torch.device(device)
        self.s_in = torch.cuda.Stream(self.device)
        self.s_cmp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._bufs = None  # [slot][name] device staging tensors for the row inputs

    def _staging(self, host_rows: dict, max_rows: int):
        key = tuple((n, t.dtype, tuple(t.shape[1:]), max_rows) for n, t in host_rows.items())
        if self._bufs is None or self._bufs[0] != key:
            bufs = [{n: torch.empty((max_rows, *t.shape[1:]), device=self.device, dtype=t.dtype)
                     for n, t in host_rows.items()} for _ in range(self.slots)]
            self._bufs = (key, bufs)
        return self._bufs[1]

    def run(self, host_rows: dict, params: dict, host_out: dict, host_param_grads=None,
            finish_params=None):
        """``host_rows``: pinned host tensors with rows on dim 0 (all the same row
        count). ``params``: device tensors every chunk sees whole. ``host_out``:
        pinned host tensors that receive the per-row outputs of ``chunk_fn`` under
        the same names. ``finish_params(partial_sum) -> dict`` turns the summed
        float32 partials into named parameter gradients, copied into
        ``host_param_grads``. Returns after enqueueing; the caller's current
        stream waits for everything (so events recorded on it afterwards cover
        the whole step). The returned list holds the device tensors the copy-out
        stream still reads: keep it until the next ``run`` has been issued or the
        device has been synchronised (dropping it earlier would let the caching
        allocator hand their memory to other work while the copies are queued;
        ``record_stream`` is not used because it defers reuse and makes a tight
        loop of steps allocate fresh memory every time)."""
        names = list(host_rows)
        rows = host_rows[names[0]].shape[0]
        for n, t in host_rows.items():
            if t.shape[0] != rows:
                raise ValueError(f"{n}: {t.shape[0]} rows, expected {rows}")
            if not t.is_pinned():
                raise ValueError(f"{n} must be in pinned host memory for asynchronous copies")
        chunks = max(1, min(self.chunks, rows))
        spans = [block_range(rows, chunks, c) for c in range(chunks)]
        bufs = self._staging(host_rows, max(b - a for a, b in spans))
        caller = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_cmp, self.s_out):
            s.wait_stream(caller)
        ev_in = [torch.cuda.Event() for _ in spans]
        ev_cmp = [torch.cuda.Event() for _ in spans]
        keep, total = [], None
        for c, (a, b) in enumerate(spans):
            slot = bufs[c % self.slots]
            with torch.cuda.stream(self.s_in):
                if c >= self.slots:  # the slot's previous chunk must have been consumed
                    self.s_in.wait_event(ev_cmp[c - self.slots])
                dev_rows = {}
                for n in names:
                    dst = slot[n][: b - a]
                    dst.copy_(host_rows[n][a:b], non_blocking=True)
                    dev_rows[n] = dst
                ev_in[c].record(self.s_in)
            with torch.cuda.stream(self.s_cmp):
                self.s_cmp.wait_event(ev_in[c])
                outs, partial = self.chunk_fn(dev_rows, params)
                if partial is not None:
                    total = partial if total is None else total.add_(partial)
                ev_cmp[c].record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_cmp[c])
                for n, t in outs.items():
                    host_out[n][a:b].copy_(t, non_blocking=True)
            keep.append(outs)
        if total is not None and finish_params is not None:
            with torch.cuda.stream(self.s_cmp):
                grads = finish_params(total)
                done = torch.cuda.Event()
                done.record(self.s_cmp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(done)
                for n, t in grads.items():
                    host_param_grads[n].copy_(t, non_blocking=True)
            keep.append(grads)
        for s in (self.s_in, self.s_cmp, self.s_out):
            caller.wait_stream(s)
        return keep

    def run_graphed(self, host_rows: dict, params: dict, host_out: dict, host_param_grads=None,
                    finish_params=None):
        """The same step replayed from a CUDA graph: with many small chunks the
        enqueueing of a step (a dozen calls per chunk) takes longer than the
        copies, and the link idles. The graph is captured on the first call for a
        given set of host and device buffers (addresses and shapes) and replayed
        on the caller's current stream afterwards; it holds the device tensors of
        the step, so nothing needs to be kept by the caller. ``finish_params`` must
        be capturable (no host synchronisation)."""
        def ident(d):
            return tuple((n, t.data_ptr(), tuple(t.shape), t.dtype) for n, t in (d or {}).items())

        key = (ident(host_rows), ident(params), ident(host_out), ident(host_param_grads),
               self.chunks, self.slots)
        cached = getattr(self, "_graph", None)
        if cached is None or cached[0] != key:
            # once outside a capture: staging buffers, lazy initialisation of the kernels
            self.run(host_rows, params, host_out, host_param_grads, finish_params)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=torch.cuda.Stream(self.device)):
                keep = self.run(host_rows, params, host_out, host_param_grads, finish_params)
            cached = (key, graph, keep)
            self._graph = cached
        cached[1].replay()
        return None


# ------------------------------------------------------------------ per operator
def _layernorm_chunk(eps):
    def fn(r, p):
        y, mean, rstd = ops.layernorm_fwd(r["x"], p["weight"], p["bias"], eps)
        dx, dwdb, _ = ops.layernorm_bwd(r["dy"], r["x"], p["weight"], mean, rstd, partials_f32=True)
        return {"y": y, "dx": dx}, dwdb
    return fn


def _rmsnorm_chunk(eps):
    def fn(r, p):
        y, rstd = ops.rmsnorm_fwd(r["x"], p["weight"], eps)
        dx, dw = ops.rmsnorm_bwd(r["dy"], r["x"], p["weight"], rstd, partials_f32=True)
        return {"y": y, "dx": dx}, dw
    return fn


def _fused_add_chunk(eps):
    def fn(r, p):
        out, rstd = ops.fused_add_rmsnorm_fwd(r["x"], r["r"], p["weight"], eps)
        dx, dw = ops.fused_add_rmsnorm_bwd(r["dout"], r["x"], r["r"], p["weight"], rstd,
                                           partials_f32=True)
        return {"out": out, "dx": dx}, dw
    return fn


def _softmax_chunk(r, p):
    y = ops.softmax_fwd(r["x"])
    return {"y": y, "dx": ops.softmax_bwd(y, r["dy"])}, None


def _glu_chunk(fwd, bwd):
    def fn(r, p):
        c = fwd(r["a"], r["b"])
        da, db = bwd(r["dc"], r["a"], r["b"])
        return {"c": c, "da": da, "db": db}, None
    return fn


def pipeline_for(op: str, *, eps: float = 1e-5, chunks: int = 8, slots: int = 3, device=None):
    """A :class:`HostRowPipeline` plus the ``finish_params`` callable for ``op``
    ("layernorm", "rmsnorm", "fused_add_rms_norm", "softmax", "swiglu", "geglu").
    ``finish_params(total, dtype)`` is None for operators without parameters."""
    if op == "layernorm":
        fn = _layernorm_chunk(eps)
        finish = lambda total, dtype: dict(zip(("dweight", "dbias"),  # noqa: E731
                                               ops.cast_from_f32(total, dtype)))
    elif op == "rmsnorm":
        fn = _rmsnorm_chunk(eps)
        finish = lambda total, dtype: {"dweight": ops.cast_from_f32(total, dtype)}  # noqa: E731
    elif op == "fused_add_rms_norm":
        fn = _fused_add_chunk(eps)
        finish = lambda total, dtype: {"dweight": ops.cast_from_f32(total, dtype)}  # noqa: E731
    elif op == "softmax":
        fn, finish = _softmax_chunk, None
    elif op == "swiglu":
        fn, finish = _glu_chunk(ops.swiglu_fwd, ops.swiglu_bwd), None
    elif op == "geglu":
        fn, finish = _glu_chunk(ops.geglu_fwd, ops.geglu_bwd), None
    else:
        raise KeyError(f"no host pipeline for operator {op!r}")
    return HostRowPipeline(fn, chunks=chunks, slots=slots, device=device), finish
