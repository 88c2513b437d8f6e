"""Sharding of the autograd pairs across ranks (one process per GPU).

The operators partition into independent units, so the only data exchanged
between ranks is the float32 parameter-gradient partial sums of LayerNorm /
RMSNorm (``[2, hidden]`` / ``[hidden]`` floats per step):

    softmax, swiglu     contiguous row blocks, no exchange
    rope                contiguous batch blocks, tables replicated, no exchange
    layernorm, rmsnorm, fused_add_rms_norm
                        contiguous row blocks; every rank forms float32
                        dweight/dbias over ITS rows, the sums of all ranks are
                        added and only then rounded to the parameter dtype
                        (rounding before the sum would not match a single-device
                        float32 accumulation). On one node the exchange is ONE
                        small kernel per rank that reads the other ranks' sums
                        through peer memory (:class:`PeerExchange`); the fallback
                        is all_reduce(SUM) followed by a rounding kernel.
    causal attention    contiguous blocks of the B*H (batch, head) units, no exchange

The reference has no distributed path (its ``--gpus`` runs independent searches);
this launcher is new. The local kernels are injected so that the host logic
(partitioning, reduction, rounding order) can be exercised with ``gloo`` ranks
on CPU against the oracle, while production uses ``evograd_b200.ops``.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def block_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous ``[start, stop)`` of ``total`` units for ``rank``; the first
    ``total % world`` ranks get one extra unit, so sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} for world size {world}")
    if total < 0:
        raise ValueError("total must be non-negative")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def _world(group) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


@dataclass
class NormKernels:
    """The local (single-device) entry points a :class:`ShardedNorm` drives."""

    layernorm_fwd: object
    layernorm_bwd: object  # (dy, x, w, mean, rstd, partials_f32=True) -> (dx, dwdb_f32, None)
    rmsnorm_fwd: object
    rmsnorm_bwd: object  # (dy, x, w, rstd, partials_f32=True) -> (dx, dw_f32)
    cast_from_f32: object
    add_rms_fwd: object = None  # (x, r, w, eps) -> (out, rstd)
    add_rms_bwd: object = None  # (dout, x, r, w, rstd, partials_f32=True) -> (dx, dw_f32)

    @staticmethod
    def cuda() -> "NormKernels":
        from . import ops

        return NormKernels(ops.layernorm_fwd, ops.layernorm_bwd, ops.rmsnorm_fwd, ops.rmsnorm_bwd,
                           ops.cast_from_f32, ops.fused_add_rmsnorm_fwd, ops.fused_add_rmsnorm_bwd)


class PeerExchange:
    """Sum of per-rank float32 vectors over the ranks of one node, rounded once,
    through peer memory: each rank owns a small device buffer, the others map it
    with CUDA IPC, and :meth:`sum_round` enqueues one single-block kernel per rank
    that writes this rank's values into every rank's buffer, waits (bounded) for
    the other ranks' values to arrive in its own and adds all of them in rank
    order. The IPC handles travel through
    ``torch.distributed.all_gather_object`` once, at construction; every rank
    must construct the object and call :meth:`sum_round` in the same order.

    ``lib`` is injectable so the host logic can run against a stand-in without a
    GPU."""

    def __init__(self, max_floats: int, group=None, lib=None):
        import ctypes

        if lib is None:
            from . import _cabi as lib
        self._lib = lib
        self.world, self.rank = _world(group)
        self.max_floats = int(max_floats)
        handle = (ctypes.c_ubyte * 64)()
        out = ctypes.c_void_p()
        lib.call("evg_exchange_create", self.max_floats, self.world, self.rank,
                 ctypes.byref(out), ctypes.cast(handle, ctypes.c_void_p))
        self._x = out
        self.handle = out  # what the C entry points that take an exchange expect
        if self.world > 1:
            gathered = [None] * self.world
            dist.all_gather_object(gathered, bytes(handle), group=group)
            blob = b"".join(gathered)
            buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
            lib.call("evg_exchange_connect", self._x, ctypes.cast(buf, ctypes.c_void_p))
        self.calls = 0

    def sum_round(self, partial: torch.Tensor, dtype: torch.dtype, out=None) -> torch.Tensor:
        """``partial``: contiguous float32 on this rank's device. Returns the sum over
        ranks rounded to ``dtype`` (same shape), identical bits on every rank. The
        kernel goes to the current stream; ``out`` may be preallocated."""
        if partial.dtype != torch.float32 or not partial.is_contiguous():
            raise TypeError("partial sums must be contiguous float32")
        if partial.numel() > self.max_floats:
            raise ValueError(f"{partial.numel()} values exceed the exchange buffer ({self.max_floats})")
        if out is None:
            out = torch.empty(partial.shape, dtype=dtype, device=partial.device)
        en = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]
        stream = torch.cuda.current_stream(partial.device).cuda_stream if partial.is_cuda else None
        self._lib.call("evg_exchange_sum_round", self._x, partial.data_ptr(), partial.numel(),
                       out.data_ptr(), en, None, stream)
        self.calls += 1
        return out

    def close(self):
        if getattr(self, "_x", None):
            self._lib.call("evg_exchange_destroy", self._x)
            self._x = None

    def __del__(self):  # best effort; explicit close() is preferred
        try:
            self.close()
        except Exception:
            pass


class ShardedNorm:
    """LayerNorm / RMSNorm autograd pair over a row shard with the cross-rank
    parameter-gradient reduction. ``kind`` is "layernorm", "rmsnorm" or
    "fused_add_rms_norm" (whose forward also takes ``residual`` and whose backward
    returns ``(dx, dr, dweight)`` with ``dr is dx``).

    ``exchange``: "peer" sums the partial sums with :class:`PeerExchange` (one node,
    one kernel per rank and step), "allreduce" uses ``all_reduce`` + a rounding
    kernel, "auto" (default) takes "peer" on CUDA ranks when the buffers of the
    other ranks can be mapped and "allreduce" otherwise. The choice is made at the
    first backward and is the same on every rank."""

    def __init__(self, kind: str, group=None, kernels: NormKernels | None = None,
                 exchange: str = "auto", hidden_max: int = 16384):
        if kind not in ("layernorm", "rmsnorm", "fused_add_rms_norm"):
            raise ValueError(f"kind must be layernorm, rmsnorm or fused_add_rms_norm, got {kind!r}")
        if exchange not in ("auto", "peer", "allreduce"):
            raise ValueError(f"exchange must be auto, peer or allreduce, got {exchange!r}")
        self.kind = kind
        self.group = group
        self.k = kernels or NormKernels.cuda()
        self.collectives = 0  # all_reduce calls issued so far
        self.exchange = exchange
        self._peer = None
        self._peer_tried = False
        self._hidden_max = hidden_max

    def exchange_name(self) -> str:
        if self._peer is not None:
            return ("peer memory (CUDA IPC): the column-reduce kernel's blocks write their float32 "
                    "sums into every rank's buffer and add what arrived in their own")
        return "nccl all_reduce of the float32 sums + rounding kernel"

    def _peer_exchange(self, partial):
        """The PeerExchange to use for this tensor, or None (all ranks agree)."""
        if self._peer is not None or self._peer_tried:
            return self._peer
        self._peer_tried = True
        world, _ = _world(self.group)
        want = self.exchange != "allreduce" and world > 1 and partial.is_cuda
        ok = 0
        peer = None
        if want:
            try:
                peer = PeerExchange(2 * self._hidden_max, self.group)
                ok = 1
            except Exception:
                if self.exchange == "peer":
                    raise
                ok = 0
        if world > 1:
            # take it only if every rank could map every other rank's buffer
            flag = torch.tensor([ok], device=partial.device, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
            ok = int(flag.item())
        if ok and peer is not None:
            self._peer = peer
        elif peer is not None:
            peer.close()
        return self._peer

    def forward_with_saved(self, x_shard, weight, bias=None, eps: float = 1e-5, residual=None):
        if self.kind == "fused_add_rms_norm":
            if residual is None:
                raise ValueError("fused_add_rms_norm needs the residual shard")
            out, rstd = self.k.add_rms_fwd(x_shard, residual, weight, eps)
            return out, (x_shard, residual, weight, rstd)
        if self.kind == "layernorm":
            if bias is None:
                raise ValueError("layernorm needs a bias")
            y, mean, rstd = self.k.layernorm_fwd(x_shard, weight, bias, eps)
            return y, (x_shard, weight, mean, rstd)
        y, rstd = self.k.rmsnorm_fwd(x_shard, weight, eps)
        return y, (x_shard, weight, rstd)

    def backward_from_saved(self, dy_shard, saved):
        """Returns ``(dx_shard, dweight[, dbias])`` with the parameter gradients
        summed over ALL ranks' rows and rounded once, identical on every rank."""
        world, _ = _world(self.group)
        # LayerNorm / RMSNorm with a peer exchange: the cross-rank sum happens inside the
        # second stage of the column reduction, no separate launch.
        if world > 1 and self.kind != "fused_add_rms_norm" and dy_shard.is_cuda:
            weight = saved[1]
            peer = self._peer_exchange(dy_shard)
            nv = 2 if self.kind == "layernorm" else 1
            if peer is not None and nv * weight.numel() <= peer.max_floats:
                if self.kind == "layernorm":
                    x, weight, mean, rstd = saved
                    return self.k.layernorm_bwd(dy_shard, x, weight, mean, rstd, exchange=peer)
                x, weight, rstd = saved
                return self.k.rmsnorm_bwd(dy_shard, x, weight, rstd, exchange=peer)
        if self.kind == "layernorm":
            x, weight, mean, rstd = saved
            dx, partial, _ = self.k.layernorm_bwd(dy_shard, x, weight, mean, rstd, partials_f32=True)
        elif self.kind == "fused_add_rms_norm":
            x, residual, weight, rstd = saved
            dx, partial = self.k.add_rms_bwd(dy_shard, x, residual, weight, rstd, partials_f32=True)
        else:
            x, weight, rstd = saved
            dx, partial = self.k.rmsnorm_bwd(dy_shard, x, weight, rstd, partials_f32=True)
        if partial.dtype != torch.float32:
            raise TypeError("local backward must return float32 partial sums")
        peer = self._peer_exchange(partial) if world > 1 else None
        if peer is not None and partial.numel() <= peer.max_floats:
            rounded = peer.sum_round(partial, weight.dtype)
        else:
            if world > 1:
                dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
                self.collectives += 1
            rounded = self.k.cast_from_f32(partial, weight.dtype)
        if self.kind == "layernorm":
            return dx, rounded[0], rounded[1]
        if self.kind == "fused_add_rms_norm":
            return dx, dx, rounded
        return dx, rounded


def shard_rows(t: torch.Tensor, group=None) -> torch.Tensor:
    """This rank's contiguous row block of a ``[rows, ...]`` tensor."""
    world, rank = _world(group)
    a, b = block_range(t.shape[0], world, rank)
    return t[a:b]


def shard_heads(t: torch.Tensor, group=None) -> torch.Tensor:
    """This rank's block of (batch, head) units of a ``[B, H, S, D]`` tensor,
    returned as ``[1, units, S, D]``."""
    world, rank = _world(group)
    B, H = t.shape[0], t.shape[1]
    a, b = block_range(B * H, world, rank)
    return t.reshape(1, B * H, *t.shape[2:])[:, a:b]
