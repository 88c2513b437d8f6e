#!/usr/bin/env python
"""Benchmark driver for the autograd-pair hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference      # the reference's CPU autograd path

A step is one forward + one backward of an operator pair over one batch of
seeded synthetic inputs of the shape the baseline configuration names. The
headline workload is LayerNorm bf16 [16384, 4096]; the other operators are
reported under ``per_op`` in the same JSON line (``--workload X`` makes X the
headline instead). Prints ONE JSON line on rank 0.

What is timed
    value     device-resident inputs, K steps between two CUDA events on the
              launching stream, barrier + synchronise on both sides, max over
              ranks. Inputs rotate through enough buffer sets that nothing a
              step reads is still in L2 from the previous use. The K steps are
              one CUDA graph; the graph is replayed at least five times (enough
              to cover 100 ms, as the reference's timing loops are sized,
              bench/fair.py:28-35) and the median replay is reported with its
              20 % / 80 % quantiles.
    e2e       the same step through the public pair API starting from pinned HOST
              buffers: host->device copies of the inputs and device->host copies
              of every result are inside the timed region.
    roofline  algorithmic bytes of the dominant launch / its device time,
              measured with CUDA events inside the timed loop, against the
              measured peak in MEASURED_PEAKS.json (stated fallback if absent).
    cpu_baseline / --impl reference
              the oracle port of the reference's CPU autograd path (the same
              forward under torch.autograd.grad) on the host cores.
Multi-GPU: the headline is weak scaling. Every rank processes a full-size shard
(global rows = N x 16384); LayerNorm/RMSNorm exchange their float32
dweight/dbias partial sums, everything else exchanges nothing. At N > 1 the line
also carries ``strong`` (the baseline shapes cut N ways: rows, batch or (batch,
head) units per rank, step time max over ranks, speed-up over the whole shape on
one GPU) and ``parity_n`` (each rank's dx rows and the exchanged dweight/dbias
checked against a float32 computation over all ranks' rows, untimed).
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import math
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

BF16, F32 = torch.bfloat16, torch.float32
MB = 1 << 20


# --------------------------------------------------------------------------
# workloads: shapes, seeds and input distributions of the baseline configs
def _gen(device, seed):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def _randn(shape, dtype, device, g, scale=1.0, shift=0.0):
    t = torch.randn(shape, device=device, dtype=torch.float32, generator=g)
    if scale != 1.0 or shift != 0.0:
        t = t * scale + shift
    return t.to(dtype)


class Workload:
    name = ""
    dtype = "bf16"
    bound = "hbm"
    collective = False
    kernels_per_step = 0
    pair = None  # operator whose candidate module provides fwd / bwd

    def __init__(self, device):
        self.device = device
        self._pair = None

    # The candidate module is imported on first use, so the CPU reference arm
    # never touches the CUDA library.
    @property
    def fwd(self):
        if self._pair is None:
            self._pair = _load_pair(self.pair)
        return self._pair[0]

    @property
    def bwd(self):
        if self._pair is None:
            self._pair = _load_pair(self.pair)
        return self._pair[1]

    # bytes (HBM-bound) or FLOPs (tensor-bound) that one fwd / bwd must move
    fwd_work = 0
    bwd_work = 0

    def forward(self, s):
        """-> (list of output tensors, saved state)"""
        raise NotImplementedError

    def backward(self, s, saved):
        """-> list of gradient tensors"""
        raise NotImplementedError

    def step(self, s, timer=None):
        run = timer.run if timer else (lambda _n, f: f())
        outs, saved = run("fwd", lambda: self.forward(s))
        grads = run("bwd", lambda: self.backward(s, saved))
        return [*outs, *grads]

    @property
    def step_work(self):
        return self.fwd_work + self.bwd_work

    def cpu_sample(self):
        """(work done by one cpu_step, description): the bounded sample of the
        workload that the host-CPU legs time."""
        return self.step_work, f"full {self.name} step"

    def pipeline_spec(self):
        """(operator, row inputs, parameters, row outputs, parameter gradients) for
        evograd_b200.host_pipeline, or None when the workload has no row pipeline."""
        return None

    def memory_inputs(self, s):
        """Tensors the saved state is measured against: the declaration's
        ``memory_input_names()`` (opdecl/activity.py:530-535), by default every
        tensor argument of the forward."""
        return [t for t in self.inputs_of(s) if torch.is_tensor(t)]

    @classmethod
    def shard_of(cls, world):
        """The class of one rank's share when the baseline shape is cut ``world``
        ways (strong scaling), or None if the shape does not divide."""
        return None


def _shard_class(cls, world, **attrs):
    for k, v in attrs.items():
        if v <= 0:
            return None
    name = getattr(cls, "name", "") or cls.__name__
    return type(f"{cls.__name__}Shard{world}", (cls,), dict(attrs, name=f"{name}/{world}"))


def _load_pair(op):
    path = os.path.join(ROOT, "evograd_b200", "pairs", f"{op}.py")
    spec = importlib.util.spec_from_file_location(f"bench_pair_{op}", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return getattr(mod, f"{op}_forward_with_saved"), getattr(mod, f"{op}_backward_from_saved")


class SoftmaxWL(Workload):
    name, dtype, kernels_per_step, pair = "softmax_f32_4096x1024", "f32", 2, "softmax"
    rows, cols = 4096, 1024

    def __init__(self, device):
        super().__init__(device)
        nb = self.rows * self.cols * 4
        self.fwd_work, self.bwd_work = 2 * nb, 3 * nb

    def make(self, device, salt=0):
        g = _gen(device, self.rows * 100003 + self.cols + salt)
        return {"x": _randn((self.rows, self.cols), F32, device, g),
                "dy": _randn((self.rows, self.cols), F32, device, g)}

    def inputs_of(self, s):
        return [s["x"], s["dy"]]

    def memory_inputs(self, s):
        return [s["x"]]

    @classmethod
    def shard_of(cls, world):
        return _shard_class(cls, world, rows=cls.rows // world) if cls.rows % world == 0 else None

    def forward(self, s):
        y, saved = self.fwd(s["x"])
        return [y], saved

    def backward(self, s, saved):
        return list(self.bwd(s["dy"], saved))

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        return ao.oracle("softmax", s)

    def pipeline_spec(self):
        return "softmax", ["x", "dy"], [], ["y", "dx"], []

    def config(self):
        return {"workload": self.name, "shape": [self.rows, self.cols], "saved": "y"}


class SoftmaxVocabWL(SoftmaxWL):
    """Softmax over Llama-3 logits rows (the reference's own benchmark grid,
    ops/level1/softmax/__init__.py:31-37): 128256 columns do not fit one block's
    registers, so this exercises the wide-row path."""
    name, dtype = "softmax_bf16_4096x128256", "bf16"
    rows, cols = 4096, 128256

    def __init__(self, device):
        Workload.__init__(self, device)
        nb = self.rows * self.cols * 2
        self.fwd_work, self.bwd_work = 2 * nb, 3 * nb

    def make(self, device, salt=0):
        g = _gen(device, self.rows * 100003 + self.cols + salt)
        return {"x": _randn((self.rows, self.cols), BF16, device, g),
                "dy": _randn((self.rows, self.cols), BF16, device, g)}


class NormWL(Workload):
    kind = "layernorm"
    rows, hidden, eps = 16384, 4096, 1e-5
    collective = True

    def __init__(self, device, group=None):
        super().__init__(device)
        nb = self.rows * self.hidden * 2
        self.fwd_work, self.bwd_work = 2 * nb, 3 * nb
        self.name = f"{self.kind}_bf16_{self.rows}x{self.hidden}"
        self.pair = self.kind
        self.world = torch.distributed.get_world_size() if torch.distributed.is_initialized() else 1
        self.sharded = None
        if self.world > 1:
            from evograd_b200.sharded import ShardedNorm

            self.sharded = ShardedNorm(self.kind, group)
        # fwd 1 kernel; bwd 2 (row kernel + column reduce); sharded adds the rounding kernel
        self.kernels_per_step = 3 + (1 if self.world > 1 else 0)

    def make(self, device, salt=0):
        g = _gen(device, self.rows * 100000 + self.hidden + salt)
        s = {"x": _randn((self.rows, self.hidden), BF16, device, g),
             "weight": _randn((self.hidden,), BF16, device, g, 0.1, 1.0)}
        if self.kind == "layernorm":
            s["bias"] = _randn((self.hidden,), BF16, device, g, 0.1, 0.0)
        s["dy"] = _randn((self.rows, self.hidden), BF16, device, g)
        s["eps"] = self.eps
        return s

    def inputs_of(self, s):
        return [s[k] for k in ("x", "weight", "bias", "dy") if k in s]

    def memory_inputs(self, s):
        return [s[k] for k in ("x", "weight", "bias") if k in s]

    @classmethod
    def shard_of(cls, world):
        return _shard_class(cls, world, rows=cls.rows // world) if cls.rows % world == 0 else None

    def forward(self, s):
        if self.sharded is not None:
            y, saved = self.sharded.forward_with_saved(s["x"], s["weight"], s.get("bias"), self.eps)
        elif self.kind == "layernorm":
            y, saved = self.fwd(s["x"], s["weight"], s["bias"], self.eps)
        else:
            y, saved = self.fwd(s["x"], s["weight"], self.eps)
        return [y], saved

    def backward(self, s, saved):
        if self.sharded is not None:
            return list(self.sharded.backward_from_saved(s["dy"], saved))
        return list(self.bwd(s["dy"], saved))

    def pipeline_spec(self):
        if self.kind == "layernorm":
            return "layernorm", ["x", "dy"], ["weight", "bias"], ["y", "dx"], ["dweight", "dbias"]
        return "rmsnorm", ["x", "dy"], ["weight"], ["y", "dx"], ["dweight"]

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        return ao.oracle(self.kind, s)

    def config(self):
        return {"workload": self.name, "shape": [self.rows, self.hidden], "eps": self.eps,
                "saved": "mean,rstd f32" if self.kind == "layernorm" else "rstd f32"}


class LayerNormWL(NormWL):
    kind = "layernorm"


class RMSNormWL(NormWL):
    kind, rows, eps = "rmsnorm", 32768, 1e-6


class SwiGLUWL(Workload):
    name, kernels_per_step, pair = "swiglu_bf16_32768x14336", 2, "swiglu"
    rows, cols = 32768, 14336

    def __init__(self, device):
        super().__init__(device)
        nb = self.rows * self.cols * 2
        self.fwd_work, self.bwd_work = 3 * nb, 5 * nb

    def make(self, device, salt=0):
        g = _gen(device, self.rows * 100003 + self.cols + salt)
        return {k: _randn((self.rows, self.cols), BF16, device, g) for k in ("a", "b", "dc")}

    def inputs_of(self, s):
        return [s["a"], s["b"], s["dc"]]

    def memory_inputs(self, s):
        return [s["a"], s["b"]]

    @classmethod
    def shard_of(cls, world):
        return _shard_class(cls, world, rows=cls.rows // world) if cls.rows % world == 0 else None

    def forward(self, s):
        c, saved = self.fwd(s["a"], s["b"])
        return [c], saved

    def backward(self, s, saved):
        return list(self.bwd(s["dc"], saved))

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        return ao.oracle("swiglu", s)

    def pipeline_spec(self):
        return self.pair, ["a", "b", "dc"], [], ["c", "da", "db"], []

    def config(self):
        return {"workload": self.name, "shape": [self.rows, self.cols], "saved": "a,b by reference"}


class GeGLUWL(SwiGLUWL):
    name, pair = "geglu_bf16_32768x14336", "geglu"

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        return ao.oracle("geglu", s)


class FusedAddRMSNormWL(Workload):
    """Residual add fused into RMSNorm at the Llama-3-8B hidden width."""
    name, kernels_per_step, pair = "fused_add_rms_norm_bf16_32768x4096", 3, "fused_add_rms_norm"
    rows, hidden, eps = 32768, 4096, 1e-6

    def __init__(self, device):
        super().__init__(device)
        nb = self.rows * self.hidden * 2
        self.fwd_work, self.bwd_work = 3 * nb, 4 * nb  # x, r -> out ; dout, x, r -> dx

    def make(self, device, salt=0):
        g = _gen(device, self.rows * 100003 + self.hidden + salt)
        s = {k: _randn((self.rows, self.hidden), BF16, device, g) for k in ("x", "r")}
        s["weight"] = _randn((self.hidden,), BF16, device, g)
        s["dout"] = _randn((self.rows, self.hidden), BF16, device, g)
        s["eps"] = self.eps
        return s

    def inputs_of(self, s):
        return [s["x"], s["r"], s["weight"], s["dout"]]

    def memory_inputs(self, s):
        return [s["x"], s["r"], s["weight"]]

    def forward(self, s):
        out, saved = self.fwd(s["x"], s["r"], s["weight"], self.eps)
        return [out], saved

    def backward(self, s, saved):
        dx, _dr, dw = self.bwd(s["dout"], saved)  # dr is dx itself
        return [dx, dw]

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        return ao.oracle("fused_add_rms_norm", s)

    def pipeline_spec(self):
        return "fused_add_rms_norm", ["x", "r", "dout"], ["weight"], ["out", "dx"], ["dweight"]

    def config(self):
        return {"workload": self.name, "shape": [self.rows, self.hidden], "eps": self.eps,
                "saved": "rstd f32 (x, r by reference; the sum is re-formed)"}


class RopeWL(Workload):
    name, kernels_per_step = "rope_bf16_qk_8x4096x32x128", 2
    B, S, H, D, theta = 8, 4096, 32, 128, 10000.0

    def __init__(self, device):
        super().__init__(device)
        nb = self.B * self.S * self.H * self.D * 2
        self.fwd_work, self.bwd_work = 4 * nb, 4 * nb  # q and k, read + write each way

    def make(self, device, salt=0):
        g = _gen(device, self.S * 100003 + self.H * 1009 + self.D + salt)
        shape = (self.B, self.S, self.H, self.D)
        s = {k: _randn(shape, BF16, device, g) for k in ("q", "k", "dq_out", "dk_out")}
        pos = torch.arange(self.S, device=device, dtype=F32)[:, None]
        inv = self.theta ** (-torch.arange(0, self.D, 2, device=device, dtype=F32) / self.D)
        s["cos"], s["sin"] = (pos * inv[None]).cos(), (pos * inv[None]).sin()  # f32 [S, D/2]
        return s

    def inputs_of(self, s):
        return [s["q"], s["k"], s["dq_out"], s["dk_out"], s["cos"], s["sin"]]

    def memory_inputs(self, s):
        return [s["q"], s["k"]]  # the declaration counts x only (ops/level1/rope/__init__.py:157)

    @classmethod
    def shard_of(cls, world):
        return _shard_class(cls, world, B=cls.B // world) if cls.B % world == 0 else None

    def forward(self, s):
        from evograd_b200 import ops
        return list(ops.rope_qk_fwd(s["q"], s["k"], s["cos"], s["sin"], layout="bthd")), None

    def backward(self, s, saved):
        from evograd_b200 import ops
        return list(ops.rope_qk_bwd(s["dq_out"], s["dk_out"], s["cos"], s["sin"], layout="bthd"))

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        cos = torch.cat((s["cos"], s["cos"]), -1)
        sin = torch.cat((s["sin"], s["sin"]), -1)
        out = []
        for x, dy in ((s["q"], s["dq_out"]), (s["k"], s["dk_out"])):
            out.append(ao.oracle("rope", {"x": x.transpose(1, 2), "cos": cos, "sin": sin,
                                          "dy": dy.transpose(1, 2)}))
        return out

    def config(self):
        return {"workload": self.name, "shape": [self.B, self.S, self.H, self.D],
                "tables": "f32 [4096,64]", "theta": self.theta, "saved": "none"}


class AttentionWL(Workload):
    name, bound, kernels_per_step, pair = "causal_attention_bf16_4x32x8192x128", "tensor", 4, \
        "causal_attention"
    B, H, S, D = 4, 32, 8192, 128

    def __init__(self, device):
        super().__init__(device)
        fwd = 4 * self.B * self.H * self.S * self.S * self.D * 0.5  # causal-halved
        self.fwd_work, self.bwd_work = fwd, 2.5 * fwd

    def make(self, device, salt=0):
        g = _gen(device, (((4 * 131 + 32) * 131 + 8192) * 131) + 128 + salt)
        shape = (self.B, self.H, self.S, self.D)
        return {k: _randn(shape, BF16, device, g) for k in ("q", "k", "v", "do")}

    def inputs_of(self, s):
        return [s["q"], s["k"], s["v"], s["do"]]

    def memory_inputs(self, s):
        return [s["q"], s["k"], s["v"]]

    @classmethod
    def shard_of(cls, world):
        units = cls.B * cls.H  # independent (batch, head) units
        return _shard_class(cls, world, B=1, H=units // world) if units % world == 0 else None

    def forward(self, s):
        o, saved = self.fwd(s["q"], s["k"], s["v"])
        return [o], saved

    def backward(self, s, saved):
        return list(self.bwd(s["do"], saved))

    def cpu_step(self, s, heads=2):
        from oracle import autograd_oracle as ao
        sl = {k: v[:1, :heads] for k, v in s.items()}
        return ao.oracle("causal_attention", sl, forward=ao.causal_attention_forward_sdpa)

    def cpu_sample(self):
        return (self.step_work * 2 / (self.B * self.H),
                f"2 of {self.B * self.H} (batch, head) units per step, rate scaled per unit")

    def config(self):
        return {"workload": self.name, "shape": [self.B, self.H, self.S, self.D],
                "scale": 1 / math.sqrt(self.D), "saved": "o, lse f32"}


class EvoAttentionWL(Workload):
    """AlphaFold-3 triangle attention (S == N == 256, 4 heads of 32): the largest
    family of the reference's evoattention grid
    (ops/level1/evoattention/__init__.py:44-56). Runs on the tcgen05 kernels."""
    name, bound, kernels_per_step, pair = "evoattention_bf16_1x256x4x256x32", "tensor", 4, \
        "evoattention"
    B, S, H, N, D = 1, 256, 4, 256, 32

    def __init__(self, device):
        super().__init__(device)
        fwd = 4 * self.B * self.S * self.H * self.N * self.N * self.D
        self.fwd_work, self.bwd_work = fwd, 2.5 * fwd

    def make(self, device, salt=0):
        g = _gen(device, ((((self.B * 131 + self.S) * 131 + self.H) * 131 + self.N) * 131) + self.D + salt)
        shape = (self.B, self.S, self.N, self.H, self.D)
        s = {k: _randn(shape, BF16, device, g, 0.5) for k in ("q", "k", "v", "do")}
        keep = torch.rand((self.B, self.S, 1, 1, self.N), device=device, generator=g) > 0.5
        keep[..., 0] = True
        s["res_mask"] = torch.where(keep, 0.0, -1e9).to(torch.float32)
        s["pair_bias"] = _randn((self.B, 1, self.H, self.N, self.N), F32, device, g, 0.5)
        return s

    def inputs_of(self, s):
        return [s[k] for k in ("q", "k", "v", "res_mask", "pair_bias", "do")]

    def memory_inputs(self, s):
        return [s[k] for k in ("q", "k", "v", "res_mask", "pair_bias")]

    def forward(self, s):
        o, saved = self.fwd(s["q"], s["k"], s["v"], s["res_mask"], s["pair_bias"])
        return [o], saved

    def backward(self, s, saved):
        return list(self.bwd(s["do"], saved))

    def cpu_step(self, s):
        from oracle import autograd_oracle as ao
        return ao.oracle("evoattention", s)

    def config(self):
        return {"workload": self.name, "shape": [self.B, self.S, self.N, self.H, self.D],
                "saved": "o, lse f32", "kernels": "tcgen05, 128 x 64 score tiles"}


class EvoAttentionPairBiasWL(EvoAttentionWL):
    """Pair-bias attention at 384 residues (S == 1, 16 heads of 64): the largest
    case of the reference grid's pair_bias family."""
    name = "evoattention_bf16_1x1x16x384x64"
    B, S, H, N, D = 1, 1, 16, 384, 64


class DecoderLayerWL(Workload):
    """One Llama-3-8B decoder layer at 4096 tokens (the largest timed case of
    ops/level3/llama3_decoder_layer/__init__.py:35-45): this package's kernels
    plus library GEMMs. Work = GEMM + attention FLOPs (causal-halved), backward
    2x the GEMMs and 2.5x the attention."""
    name, bound, pair = "llama3_decoder_layer_bf16_1x4096", "tensor", "llama3_decoder_layer"
    kernels_per_step = 8 + 17  # own launches: 8 forward, 17 backward (GEMMs not counted)
    B, T, hidden, hd, q_out, kv_out, inter = 1, 4096, 4096, 128, 4096, 1024, 14336

    def __init__(self, device):
        super().__init__(device)
        bt = self.B * self.T
        gemm = 2 * bt * (self.hidden * (self.q_out + 2 * self.kv_out) + self.q_out * self.hidden
                         + 3 * self.hidden * self.inter)
        attn = 4 * self.B * (self.q_out // self.hd) * self.T * self.T * self.hd * 0.5
        self.fwd_work, self.bwd_work = gemm + attn, 2 * gemm + 2.5 * attn

    def dims(self):
        return dict(B=self.B, T=self.T, hidden=self.hidden, head_dim=self.hd, q_out=self.q_out,
                    kv_out=self.kv_out, intermediate=self.inter)

    def make(self, device, salt=0):
        g = _gen(device, self.T * 100003 + self.hidden * 1009 + self.hd + salt)

        def weight(o_f, i_f):
            return _randn((o_f, i_f), BF16, device, g, i_f ** -0.5)

        pos = torch.arange(self.T, device=device, dtype=torch.float32)[:, None]
        inv = 500000.0 ** (-torch.arange(0, self.hd, 2, device=device, dtype=torch.float32) / self.hd)
        ang = torch.cat((pos * inv[None, :],) * 2, dim=-1)
        return {
            "x": _randn((self.B, self.T, self.hidden), BF16, device, g, 0.5),
            "input_norm_weight": _randn((self.hidden,), BF16, device, g, 0.1, 1.0),
            "q_weight": weight(self.q_out, self.hidden), "k_weight": weight(self.kv_out, self.hidden),
            "v_weight": weight(self.kv_out, self.hidden), "o_weight": weight(self.hidden, self.q_out),
            "post_norm_weight": _randn((self.hidden,), BF16, device, g, 0.1, 1.0),
            "gate_weight": weight(self.inter, self.hidden), "up_weight": weight(self.inter, self.hidden),
            "down_weight": weight(self.hidden, self.inter),
            "cos": ang.cos().to(BF16), "sin": ang.sin().to(BF16), "eps": 1e-5,
            "dout": _randn((self.B, self.T, self.hidden), BF16, device, g,
                           0.5 * (self.B * self.T) ** -0.5),
        }

    _ARGS = ("x", "input_norm_weight", "q_weight", "k_weight", "v_weight", "o_weight",
             "post_norm_weight", "gate_weight", "up_weight", "down_weight", "cos", "sin")

    def inputs_of(self, s):
        return [s[k] for k in self._ARGS] + [s["dout"]]

    def memory_inputs(self, s):
        return [s[k] for k in self._ARGS]

    def forward(self, s):
        out, saved = self.fwd(*[s[k] for k in self._ARGS], s["eps"])
        return [out], saved

    def backward(self, s, saved):
        return list(self.bwd(s["dout"], saved, s["eps"]))

    def cpu_step(self, s, tokens=512):
        from oracle import autograd_oracle as ao
        sl = dict(s)
        for k in ("x", "dout"):
            sl[k] = s[k][:, :tokens]
        for k in ("cos", "sin"):
            sl[k] = s[k][:tokens]
        return ao.oracle("llama3_decoder_layer", sl)

    def cpu_sample(self, tokens=512):
        bt = self.B * tokens
        gemm = 2 * bt * (self.hidden * (self.q_out + 2 * self.kv_out) + self.q_out * self.hidden
                         + 3 * self.hidden * self.inter)
        attn = 4 * self.B * (self.q_out // self.hd) * tokens * tokens * self.hd * 0.5
        return 3 * gemm + 3.5 * attn, f"the first {tokens} of {self.T} tokens per step"

    def config(self):
        return {"workload": self.name, **self.dims(),
                "saved": "rstd x2, rotated q/k, v, o, lse f32, residual stream, gate, up",
                "gemms": "cuBLAS via torch.mm/addmm"}


WORKLOADS = {"softmax": SoftmaxWL, "layernorm": LayerNormWL, "rmsnorm": RMSNormWL,
             "swiglu": SwiGLUWL, "rope": RopeWL, "attention": AttentionWL,
             "geglu": GeGLUWL, "fused_add_rms_norm": FusedAddRMSNormWL,
             "softmax_vocab": SoftmaxVocabWL, "decoder_layer": DecoderLayerWL,
             "evoattention": EvoAttentionWL, "evoattention_n384": EvoAttentionPairBiasWL}


# --------------------------------------------------------------------------
def _dist_setup(n_gpus):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
    if n_gpus != world:
        if rank == 0:
            print(f"[bench] --gpus {n_gpus} but WORLD_SIZE={world}; launch with torch.distributed.run",
                  file=sys.stderr)
        if world == 1 and n_gpus > 1:
            raise SystemExit(2)
    return world, rank, local


def _barrier_fn(world):
    if world <= 1:
        return None
    return lambda: torch.distributed.barrier()


def _max_over_ranks(ms, world):
    if world <= 1:
        return ms
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def measure_device(wl, steps, warmup, world, sections=True):
    """value leg: returns (ms for `steps` steps [max over ranks], section totals, launches)."""
    from evograd_b200.timing import SectionTimer, time_steps

    sets = _make_sets(wl)
    n_sets = len(sets)
    timer = SectionTimer() if sections else None
    live = [None]

    def step(i):
        live[0] = wl.step(sets[i % n_sets], timer if (timer and i >= warmup) else None)

    ms = time_steps(step, steps, warmup, barrier=_barrier_fn(world))
    ms = _max_over_ranks(ms, world)
    totals = timer.totals_ms() if timer else {}
    del sets, live
    torch.cuda.empty_cache()
    return ms, totals, wl.kernels_per_step * steps, n_sets


def _make_sets(wl):
    from evograd_b200.timing import rotation_count

    device = torch.device("cuda", torch.cuda.current_device())
    probe = wl.make(device)
    set_bytes = sum(t.numel() * t.element_size() for t in wl.inputs_of(probe))
    n_sets = 1 if set_bytes > 2 * torch.cuda.get_device_properties(device).L2_cache_size \
        else rotation_count(set_bytes)
    return [probe] + [wl.make(device, salt=i) for i in range(1, n_sets)]


REP_BUDGET_MS = 100.0  # per timed leg, as the reference sizes its loops (bench/fair.py:28-35)
MIN_REPS, MAX_REPS = 5, 60


def _quantile(sorted_vals, q):
    if len(sorted_vals) == 1:
        return sorted_vals[0]
    pos = q * (len(sorted_vals) - 1)
    lo = int(pos)
    hi = min(lo + 1, len(sorted_vals) - 1)
    return sorted_vals[lo] + (sorted_vals[hi] - sorted_vals[lo]) * (pos - lo)


def _replay_stats(graph, steps, world):
    """Replays a graph holding `steps` steps: one untimed replay, then at least
    MIN_REPS timed ones (enough to cover REP_BUDGET_MS), each between its own
    CUDA event pair with barrier + synchronise on both sides and the maximum
    over ranks taken per replay. Returns per-step milliseconds."""
    from evograd_b200.timing import time_steps

    barrier = _barrier_fn(world)
    first = _max_over_ranks(time_steps(lambda _i: graph.replay(), 1, 1, barrier=barrier), world)
    reps = max(MIN_REPS, min(MAX_REPS, int(REP_BUDGET_MS / max(first, 1e-3))))
    if world > 1:  # every rank must run the same number of replays
        t = torch.tensor([reps], device="cuda", dtype=torch.int64)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
        reps = int(t.item())
    samples = [first]
    for _ in range(reps - 1):
        samples.append(_max_over_ranks(time_steps(lambda _i: graph.replay(), 1, 0, barrier=barrier),
                                       world))
    per_step = sorted(v / steps for v in samples)
    return {"median": _quantile(per_step, 0.5), "q20": _quantile(per_step, 0.2),
            "q80": _quantile(per_step, 0.8), "reps": len(per_step)}


def _saved_accounting(wl, s, saved):
    """saved_bytes / input_bytes / saved_memory_ratio as bench/harness.py:128-131 and
    321-346 compute them (every tensor of the saved state counts, also those that
    are the inputs themselves), plus the split the reference's final report makes
    between inputs kept by reference and newly written state (bench/fair.py:297-322)."""
    tensors = [t for t in (saved if isinstance(saved, (tuple, list)) else (saved,))
               if torch.is_tensor(t)]
    inputs = wl.memory_inputs(s)
    input_ptrs = {t.untyped_storage().data_ptr() for t in wl.inputs_of(s) if torch.is_tensor(t)}
    total = sum(t.numel() * t.element_size() for t in tensors)
    retained = sum(t.numel() * t.element_size() for t in tensors
                   if t.untyped_storage().data_ptr() in input_ptrs)
    in_bytes = sum(t.numel() * t.element_size() for t in inputs)
    return {"saved_bytes": int(total), "input_bytes": int(in_bytes),
            "saved_memory_ratio": round(total / max(in_bytes, 1), 6),
            "retained_input_bytes": int(retained), "new_saved_bytes": int(total - retained)}


def measure_graphs(wl, steps, warmup, world):
    """Device leg with the host launch path removed: the K timed steps (cycling
    through the rotating input sets) are captured into ONE CUDA graph, for the
    full step, the forward alone and the backward alone, and each graph is
    replayed several times (see _replay_stats). W eager steps come first. (One
    graph per step would put a graph-launch gap of several microseconds between
    steps, which is a third of the float32 softmax step.)
    Returns (step, fwd, bwd statistics, n_sets, saved-state accounting)."""
    sets = _make_sets(wl)
    n = len(sets)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside capture (lazy init, attributes)
        for i in range(max(warmup, 1)):
            wl.step(sets[i % n])
        saved = [wl.forward(s_)[1] for s_ in sets]  # state the backward-only graph consumes
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    accounting = _saved_accounting(wl, sets[0], saved[0])

    def capture(body):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(steps):
                body(i)  # results are dropped: the graph's pool reuses their memory
        return g

    bodies = (lambda i: wl.step(sets[i % n]),
              lambda i: wl.forward(sets[i % n]),
              lambda i: wl.backward(sets[i % n], saved[i % n]))
    res = []
    for body in bodies:
        g = capture(body)
        res.append(_replay_stats(g, steps, world))
        del g
    del saved, sets
    torch.cuda.empty_cache()
    return res[0], res[1], res[2], n, accounting


def measure_e2e(wl, steps, warmup, world):
    """e2e leg: pinned host inputs -> H2D -> fwd -> bwd -> D2H of every result.
    Row-wise workloads go through evograd_b200.host_pipeline (rows cut into
    chunks; copy-in, kernels and copy-out of different chunks overlap on three
    streams); the others copy, compute and copy back in sequence."""
    from evograd_b200.timing import time_steps

    device = torch.device("cuda", torch.cuda.current_device())
    dev_set = wl.make(device)
    host = {k: (v.cpu().pin_memory() if torch.is_tensor(v) else v) for k, v in dev_set.items()}
    spec = wl.pipeline_spec()
    if spec is not None:
        from evograd_b200.host_pipeline import pipeline_for

        op, row_names, param_names, out_names, grad_names = spec
        # one rank: the whole step is replayed from a CUDA graph (4 % faster than enqueueing it
        # call by call; more than 8-16 chunks lose to the per-copy cost of the link either way);
        # several ranks (an all_reduce inside the step) enqueue it call by call
        graphed = world == 1 and os.environ.get("EVG_E2E_GRAPH", "1") != "0"
        n_chunks = int(os.environ.get("EVG_E2E_CHUNKS", "8"))
        pipe, finish = pipeline_for(op, eps=dev_set.get("eps", 1e-5), chunks=n_chunks)
        host_rows = {n: host[n] for n in row_names}
        params = {n: dev_set[n] for n in param_names}
        like = host[row_names[0]]
        host_out = {n: torch.empty_like(like).pin_memory() for n in out_names}
        host_grads = {n: torch.empty_like(host[param_names[0]]).pin_memory() for n in grad_names}
        dtype = like.dtype
        h2d = sum(t.numel() * t.element_size() for t in host_rows.values()) + \
            sum(host[n].numel() * host[n].element_size() for n in param_names)
        d2h = sum(t.numel() * t.element_size() for t in (*host_out.values(), *host_grads.values()))
        del dev_set
        live = [None]

        def finish_all(total):
            if world > 1:  # float32 partial sums of every rank's rows, then one rounding
                torch.distributed.all_reduce(total, op=torch.distributed.ReduceOp.SUM)
            return finish(total, dtype)

        def step(_i):
            for n in param_names:
                params[n].copy_(host[n], non_blocking=True)
            run = pipe.run_graphed if graphed else pipe.run
            live[0] = run(host_rows, params, host_out, host_grads, finish_all if finish else None)

        ms = time_steps(step, steps, warmup, barrier=_barrier_fn(world))
        ms = _max_over_ranks(ms, world)
        del live, params, host_rows, host_out
        torch.cuda.empty_cache()
        return ms, h2d, d2h, (f"host_pipeline: {n_chunks} row chunks, copy-in / kernels / copy-out "
                              "overlapped on three streams"
                              + (", the step replayed from one CUDA graph" if graphed else ""))
    outs = wl.step(dev_set)
    host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
    h2d = sum(v.numel() * v.element_size() for v in host.values() if torch.is_tensor(v))
    d2h = sum(o.numel() * o.element_size() for o in host_out)
    del outs

    def step(_i):
        for k, v in host.items():
            if torch.is_tensor(v):
                dev_set[k].copy_(v, non_blocking=True)
        results = wl.step(dev_set)
        for dst, src in zip(host_out, results):
            dst.copy_(src, non_blocking=True)

    ms = time_steps(step, steps, warmup, barrier=_barrier_fn(world))
    ms = _max_over_ranks(ms, world)
    del dev_set, host, host_out
    torch.cuda.empty_cache()
    return ms, h2d, d2h, "sequential: copy in, kernels, copy out"


def measure_cpu(wl, budget_s=12.0, max_reps=10, threads=None):
    """Reference CPU path (oracle port) on the host cores; returns (s/step, reps, cores)."""
    if threads:
        torch.set_num_threads(threads)
    s = wl.make(torch.device("cpu"))
    s = {k: v for k, v in s.items()}
    t0 = time.perf_counter()
    wl.cpu_step(s)  # warm-up
    first = time.perf_counter() - t0
    reps = max(1, min(max_reps, int(budget_s / max(first, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        wl.cpu_step(s)
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], reps, torch.get_num_threads()


def _rate(work, ms):
    """GB/s for bytes, TFLOP/s for FLOPs: both are work / (ms * 1e6) / 1e3... in their unit."""
    return work / (ms * 1e-3) / 1e9 if ms > 0 else 0.0


def _stat_keys(prefix, st):
    return {f"{prefix}_ms": round(st["median"], 5), f"{prefix}_ms_q20": round(st["q20"], 5),
            f"{prefix}_ms_q80": round(st["q80"], 5)}


def per_op_entry(wl, steps, warmup, world, peaks):
    launch = "cuda graph replay"
    accounting = {}
    try:
        st, sf, sb, n_sets, accounting = measure_graphs(wl, steps, warmup, world)
        reps = st["reps"]
    except Exception as exc:  # capture refused: time the same calls eagerly
        launch = f"eager ({type(exc).__name__})"
        torch.cuda.synchronize()
        ms, totals, _launches, n_sets = measure_device(wl, steps, warmup, world)
        one = lambda v: {"median": v, "q20": v, "q80": v}  # noqa: E731
        st = one(ms / steps)
        sf = one(totals["fwd"][0] / totals["fwd"][1])
        sb = one(totals["bwd"][0] / totals["bwd"][1])
        reps = 1
    step_ms, fwd_ms, bwd_ms = st["median"], sf["median"], sb["median"]
    e = {**_stat_keys("step", st), **_stat_keys("fwd", sf), **_stat_keys("bwd", sb),
         # the reference's report keys for the same three timings (bench/harness.py:328-331)
         "forward_ms": round(fwd_ms, 5), "backward_from_saved_ms": round(bwd_ms, 5),
         "forward_backward_full_step_ms": round(step_ms, 5),
         "reps": reps, "steps_per_rep": steps, "buffer_sets": n_sets, "launch": launch,
         **accounting}
    if wl.bound == "hbm":
        peak = peaks["hbm_gbs"]
        e.update({"algorithmic_MB": round(wl.step_work / 1e6, 1),
                  "gbs": round(_rate(wl.step_work, step_ms) * world, 1),
                  "fwd_gbs": round(_rate(wl.fwd_work, fwd_ms), 1),
                  "bwd_gbs": round(_rate(wl.bwd_work, bwd_ms), 1),
                  "frac_of_hbm_peak": round(_rate(wl.step_work, step_ms) / peak, 4)})
    else:
        bwd_tf = wl.bwd_work / (bwd_ms * 1e-3) / 1e12
        e.update({"fwd_tflops": round(wl.fwd_work / (fwd_ms * 1e-3) / 1e12, 1),
                  "bwd_tflops": round(bwd_tf, 1),
                  "tflops": round(wl.step_work / (step_ms * 1e-3) / 1e12 * world, 1),
                  "bwd_frac_of_burst": round(bwd_tf / peaks["bf16_tflops"], 4),
                  "bwd_frac_of_sustained": round(bwd_tf / peaks["bf16_tflops_sustained"], 4)})
    return e


# Row shapes away from the baseline configurations (narrow rows, rows that do not
# fill a power-of-two group, very wide rows): LayerNorm / RMSNorm forward and
# backward as fractions of the copy bandwidth, same method as per_op.
OFF_BASELINE_SHAPES = [(65536, 1024), (49152, 1536), (32768, 3072), (8192, 5120), (2048, 16384)]


def off_baseline_table(device, steps, warmup, peaks):
    table = []
    for rows, hidden in OFF_BASELINE_SHAPES:
        entry = {"shape": [rows, hidden], "dtype": "bf16"}
        for kind, base in (("layernorm", LayerNormWL), ("rmsnorm", RMSNormWL)):
            cls = type(f"{base.__name__}Off", (base,), {"rows": rows, "hidden": hidden})
            w = cls(device)
            e = per_op_entry(w, steps, warmup, 1, peaks)
            entry[kind] = {"fwd_ms": e["fwd_ms"], "bwd_ms": e["bwd_ms"],
                           "fwd_frac_of_hbm_peak": round(e["fwd_gbs"] / peaks["hbm_gbs"], 4),
                           "bwd_frac_of_hbm_peak": round(e["bwd_gbs"] / peaks["hbm_gbs"], 4),
                           "buffer_sets": e["buffer_sets"]}
            del w
            torch.cuda.empty_cache()
        table.append(entry)
    return table


def strong_scaling(world, steps, warmup, peaks):
    """The baseline shapes cut `world` ways (rows, batch or (batch, head) units per
    rank; LayerNorm/RMSNorm with the cross-rank dweight/dbias exchange): step
    time of the shard (max over ranks) against the whole shape on one GPU with no
    exchange, both as graph replays in this run."""
    device = torch.device("cuda", torch.cuda.current_device())
    out = {}
    for name in ("softmax", "layernorm", "rmsnorm", "swiglu", "rope", "attention"):
        cls = WORKLOADS[name]
        shard_cls = cls.shard_of(world)
        if shard_cls is None:
            out[name] = None
            continue
        whole = cls(device)
        if getattr(whole, "sharded", None) is not None:
            whole.sharded = None  # the one-GPU reference point exchanges nothing
        t1 = measure_graphs(whole, steps, warmup, 1)[0]["median"]
        del whole
        torch.cuda.empty_cache()
        t1 = _max_over_ranks(t1, world)
        shard = shard_cls(device)
        tn = measure_graphs(shard, steps, warmup, world)[0]
        out[name] = {"shard": shard.config().get("shape"), "whole_shape_1gpu_ms": round(t1, 5),
                     "shard_step_ms": round(tn["median"], 5), "shard_step_ms_q20": round(tn["q20"], 5),
                     "shard_step_ms_q80": round(tn["q80"], 5),
                     "speedup": round(t1 / tn["median"], 3),
                     "efficiency": round(t1 / tn["median"] / world, 4),
                     "exchange": "float32 dweight/dbias partial sums" if cls.collective else "none"}
        del shard
        torch.cuda.empty_cache()
    return out


def parity_n(world, rank):
    """Untimed check of the N > 1 path on the baseline LayerNorm / RMSNorm shapes cut
    by rows: this rank's y and dx against a float32 computation of the same rows,
    the exchanged dweight/dbias against the float32 column sums over ALL ranks'
    rows (per-rank float32 sums, added across ranks). Raises on a mismatch."""
    from evograd_b200.sharded import ShardedNorm

    device = torch.device("cuda", torch.cuda.current_device())
    report = {}
    for kind, cls in (("layernorm", LayerNormWL), ("rmsnorm", RMSNormWL)):
        rows, hidden, eps = cls.rows // world, cls.hidden, cls.eps
        g = _gen(device, cls.rows * 100000 + hidden)
        w = _randn((hidden,), BF16, device, g, 0.1, 1.0)  # same seed: identical on every rank
        b = _randn((hidden,), BF16, device, g, 0.1, 0.0) if kind == "layernorm" else None
        g = _gen(device, cls.rows * 100000 + hidden + 7919 * (rank + 1))
        x = _randn((rows, hidden), BF16, device, g)
        dy = _randn((rows, hidden), BF16, device, g)
        sn = ShardedNorm(kind)
        y, saved = sn.forward_with_saved(x, w, b, eps)
        grads = sn.backward_from_saved(dy, saved)
        xf, dyf, wf = x.float(), dy.float(), w.float()
        if kind == "layernorm":
            mu = xf.mean(-1, keepdim=True)
            xh = (xf - mu) * torch.rsqrt(((xf - mu) ** 2).mean(-1, keepdim=True) + eps)
            y_ref = xh * wf + b.float()
            gg = dyf * wf
            dx_ref = torch.rsqrt(((xf - mu) ** 2).mean(-1, keepdim=True) + eps) * (
                gg - gg.mean(-1, keepdim=True) - xh * (gg * xh).mean(-1, keepdim=True))
            sums = torch.stack(((dyf * xh).sum(0), dyf.sum(0)))
            mags = torch.stack(((dyf * xh).abs().sum(0), dyf.abs().sum(0)))
        else:
            rs = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
            xh = xf * rs
            y_ref = xh * wf
            gg = dyf * wf
            dx_ref = (gg - xh * (gg * xh).mean(-1, keepdim=True)) * rs
            sums = (dyf * xh).sum(0)[None]
            mags = (dyf * xh).abs().sum(0)[None]
        torch.distributed.all_reduce(sums)
        torch.distributed.all_reduce(mags)
        errs = {}
        for nm, got, ref in (("y", y, y_ref), ("dx", grads[0], dx_ref)):
            err = (got.float() - ref).abs()
            ok = bool((err <= 1e-2 + 1.6e-2 * ref.abs()).all())
            errs[nm] = float(err.max())
            if not ok:
                raise AssertionError(f"parity at N={world}: {kind} {nm} max-abs {errs[nm]:.3e}")
        for i, nm in enumerate(("dweight", "dbias")[: sums.shape[0]]):
            got = grads[1 + i].float()
            # one rounding to bf16 (half an ulp = 2^-9 relative; two ulps allowed) on top of
            # float32 summation noise proportional to the summed magnitudes
            bound = 2.0 ** -7 * sums[i].abs() + 1e-5 * mags[i] + 1e-3
            err = (got - sums[i]).abs()
            errs[nm] = float(err.max())
            if not bool((err <= bound).all()):
                raise AssertionError(f"parity at N={world}: {kind} {nm} max-abs {errs[nm]:.3e}")
            # and every rank holds the same bits
            bits = grads[1 + i].contiguous().view(torch.int16).to(torch.int32)
            lo, hi = bits.clone(), bits.clone()
            torch.distributed.all_reduce(lo, op=torch.distributed.ReduceOp.MIN)
            torch.distributed.all_reduce(hi, op=torch.distributed.ReduceOp.MAX)
            if not torch.equal(lo, hi):
                raise AssertionError(f"parity at N={world}: {kind} {nm} differs between ranks")
        report[kind] = {"rows_per_rank": rows, "max_abs_err": {k: round(v, 6) for k, v in errs.items()},
                        "exchange": sn.exchange_name()}
        del x, dy, y, saved, grads, xf, dyf
        torch.cuda.empty_cache()
    return {"status": "ok", **report}


def _common_config(wl, world):
    """The workload description both arms print (what is computed, on what)."""
    return {**wl.config(), "parallelism": f"rows x{world}" if world > 1 else "1 gpu"}


def _metric_of(wl):
    if wl.bound == "hbm":
        return f"fwd+bwd achieved HBM GB/s ({wl.name})", "GB/s"
    return f"fwd+bwd TFLOP/s ({wl.name}; attention bwd TFLOP/s under per_op)", "TFLOP/s"


def run_ours(args):
    from evograd_b200 import _cabi  # noqa: F401  (fails loudly if the library is missing)
    from evograd_b200.timing import ClockSampler, measured_peaks

    world, rank, local = _dist_setup(args.gpus)
    device = torch.device("cuda", torch.cuda.current_device())
    peaks, peak_source = measured_peaks()
    wl = WORKLOADS[args.workload](device)

    parity = None
    if world > 1 and not args.no_parity:
        parity = parity_n(world, rank)  # raises if the N > 1 results are wrong

    # Leg 1 (value): K steps between one event pair, captured as one CUDA graph of
    # the public pair calls (forward, backward, and at N > 1 the cross-rank
    # exchange), so the host's launch path is not what is being timed; the graph
    # is replayed several times and the median replay is the value.
    # Leg 2 (roofline): K backward launches alone (row kernel and column reduce),
    # timed the same way; if capture is refused, the same K steps launched
    # eagerly with an event pair around forward and backward.
    launch_mode = "cuda graph replay (the K steps captured in one graph)"
    roofline_loop = ("replays of a graph holding K backward launches, each between one CUDA "
                     "event pair; median")
    spread = None
    with ClockSampler(local) as clocks:
        try:
            st, _sf, sb, n_sets, _acc = measure_graphs(wl, args.steps, args.warmup, world)
            step_ms, bwd_ms = st["median"], sb["median"]
            spread = {"reps": st["reps"], "ms_per_step_q20": round(st["q20"], 5),
                      "ms_per_step_q80": round(st["q80"], 5)}
            launches = wl.kernels_per_step * args.steps
        except Exception as exc:  # capture refused: the same calls, launched eagerly
            launch_mode = f"eager, current stream ({type(exc).__name__})"
            roofline_loop = "same K steps launched eagerly with CUDA events around forward and backward"
            torch.cuda.synchronize()
            ms, _unused, launches, n_sets = measure_device(wl, args.steps, args.warmup, world,
                                                           sections=False)
            step_ms = ms / args.steps
            _ms2, totals, _l2, _n2 = measure_device(wl, args.steps, args.warmup, world,
                                                    sections=True)
            bwd_total, bwd_n = totals["bwd"]
            bwd_ms = bwd_total / bwd_n
    metric, unit = _metric_of(wl)
    if wl.bound == "hbm":
        value = _rate(wl.step_work, step_ms) * world
    else:
        value = wl.step_work / (step_ms * 1e-3) / 1e12 * world

    # roofline of the dominant launch: the backward (largest share of the step)
    traffic, traffic_source = ncu_traffic(args.workload)
    if wl.bound == "hbm":
        achieved, peak, runit = _rate(wl.bwd_work, bwd_ms), peaks["hbm_gbs"], "GB/s"
        peak_note = f"of {peak_source} (copy bandwidth)"
    else:
        achieved, peak, runit = (wl.bwd_work / (bwd_ms * 1e-3) / 1e12,
                                 peaks["bf16_tflops_sustained"], "TFLOP/s")
        peak_note = f"of {peak_source} (sustained bf16 GEMM rate; the kernel runs under the power cap)"
    roofline = {"kernel": f"{args.workload} backward", "bound": wl.bound, "achieved": round(achieved, 1),
                "peak": peak, "unit": runit, "frac": round(achieved / peak, 4),
                "peak_source": peak_note, "per_launch_ms": round(bwd_ms, 4),
                "traffic": traffic, "traffic_source": traffic_source}
    if wl.bound != "hbm":
        roofline["frac_of_burst"] = round(achieved / peaks["bf16_tflops"], 4)

    e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        e2e_ms, h2d, d2h, e2e_mode = measure_e2e(wl, e2e_steps, max(3, min(args.warmup, 3)), world)
        e2e_step_ms = e2e_ms / e2e_steps
        e2e_value = (_rate(wl.step_work, e2e_step_ms) if wl.bound == "hbm"
                     else wl.step_work / (e2e_step_ms * 1e-3) / 1e12) * world
        e2e = {"value": round(e2e_value, 2), "unit": unit, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_step_ms, 4), "steps": e2e_steps,
               "path": e2e_mode}

    line = {
        "metric": metric, "value": round(value, 2), "unit": unit, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(step_ms, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": wl.dtype, "data": "synthetic",
        "config": _common_config(wl, world),
        "run": {"l2": f"{n_sets} rotating input set(s), each pass reads data not in L2",
                "launch": launch_mode, "roofline_loop": roofline_loop, "spread": spread,
                "exchange": (wl.sharded.exchange_name() if getattr(wl, "sharded", None) else None)},
        "e2e": e2e,
        "gpu_launches": launches,
        "roofline": roofline,
        "clocks": clocks.summary(),
    }
    if parity is not None:
        line["parity_n"] = parity

    if not args.no_per_op:
        per_op = {}
        for name, cls in WORKLOADS.items():
            w2 = wl if name == args.workload else cls(device)
            per_op[name] = per_op_entry(w2, max(3, args.steps // 2), max(3, args.warmup), world, peaks)
            del w2
            torch.cuda.empty_cache()
        line["per_op"] = per_op

    if world == 1 and not args.no_per_op:
        line["off_baseline"] = off_baseline_table(device, max(3, args.steps // 2),
                                                  max(3, args.warmup), peaks)

    if world > 1 and not args.no_strong:
        line["strong"] = strong_scaling(world, max(3, args.steps // 2), max(3, args.warmup), peaks)

    if rank == 0 and world == 1 and not args.no_cpu:
        sec, reps, cores = measure_cpu(wl)
        work, sample = wl.cpu_sample()
        div = 1e9 if wl.bound == "hbm" else 1e12
        line["cpu_baseline"] = {"value": round(work / sec / div, 3), "unit": unit, "cores": cores,
                                "kind": "port", "sample": f"{sample} x{reps} (median)",
                                "s_per_step": round(sec, 4)}
        sec1, reps1, _ = measure_cpu(wl, budget_s=6.0, max_reps=3, threads=1)
        line["cpu_baseline"]["one_thread"] = {"value": round(work / sec1 / div, 4), "unit": unit,
                                              "cores": 1, "sample": f"{sample} x{reps1} (median)",
                                              "s_per_step": round(sec1, 4)}

    from evograd_b200 import ops
    ops.device_status()
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


# dram__bytes_read.sum + dram__bytes_write.sum per backward launch from ncu
# captures: bytes (already scaled to the bench's row count where the capture ran
# on fewer rows), the file the summary of the capture is in, the kernel sources
# the capture belongs to and the digest of those sources when it was taken.
_ROW_HEADERS = ["evg_common.cuh", "rowcfg.cuh", "norm_reduce.cuh", "sm100_umma.cuh"]
TRAFFIC_SOURCES = {
    "layernorm": ["norm_bwd.cu", *_ROW_HEADERS],
    "rmsnorm": ["norm_bwd.cu", *_ROW_HEADERS],
    "fused_add_rms_norm": ["add_rms_norm.cu", *_ROW_HEADERS],
    "geglu": ["glu.cu", "evg_common.cuh"],
    "swiglu": ["glu.cu", "evg_common.cuh"],
    "softmax_vocab": ["softmax_wide.cu", "softmax_wide.cuh", "evg_common.cuh", "sm100_umma.cuh"],
    "softmax": ["softmax.cu", "evg_common.cuh", "rowcfg.cuh"],
    "rope": ["rope.cu", "evg_common.cuh"],
}
TRAFFIC_NCU = {
    # python bench.py --source-digest NAME prints the digest of a workload's kernel sources as
    # they are now; an entry whose digest no longer matches is reported as stale, not used
    "layernorm": {"bytes": 382200000, "profile": "profiles/layernorm_bf16_16384x4096.md",
                 "sources": TRAFFIC_SOURCES["layernorm"], "digest": "eeb8977e8240"},
    "rmsnorm": {"bytes": 674900000, "profile": "profiles/rmsnorm_and_fused_add_bf16_8192x4096.md (8192 rows, scaled x 4)",
               "sources": TRAFFIC_SOURCES["rmsnorm"], "digest": "eeb8977e8240"},
    "fused_add_rms_norm": {"bytes": 971700000, "profile": "profiles/rmsnorm_and_fused_add_bf16_8192x4096.md (8192 rows, scaled x 4)",
                          "sources": TRAFFIC_SOURCES["fused_add_rms_norm"], "digest": "dd18f66879bf"},
    "geglu": {"bytes": 4306000000, "profile": "profiles/geglu_bf16_4096x14336.md (4096 rows, scaled x 8)",
             "sources": TRAFFIC_SOURCES["geglu"], "digest": "70fc4295b6b2"},
    "swiglu": {"bytes": 4307000000, "profile": "profiles/swiglu_bf16_4096x14336.md (4096 rows, scaled x 8)",
              "sources": TRAFFIC_SOURCES["swiglu"], "digest": "70fc4295b6b2"},
    "softmax_vocab": {"bytes": 2859000000, "profile": "profiles/softmax_bf16_512x128256.md (512 rows, scaled x 8)",
                     "sources": TRAFFIC_SOURCES["softmax_vocab"], "digest": "73990a043930"},
    "softmax": {"bytes": 33600000, "profile": "profiles/softmax_f32_4096x1024.md",
               "sources": TRAFFIC_SOURCES["softmax"], "digest": "1c5eac59092e"},
    "rope": {"bytes": 844400000, "profile": "profiles/rope_bf16_qk_2x4096x32x128.md (batch 2, scaled x 4)",
            "sources": TRAFFIC_SOURCES["rope"], "digest": "dec1e5bf9493"},
}


TRAFFIC_NOTES = {
    # tensor-bound workloads: the DRAM bytes of the small-case captures do not grow in proportion
    # to the work (tiles are re-read from L2), so no per-launch figure is scaled from them
    "attention": "not scaled: 287 MB per fused backward launch at [1, 32, 4096, 128] "
                 "(profiles/causal_attention_bf16_1x32x4096x128.md), DRAM throughput 8 %",
    "decoder_layer": "not scaled: see profiles/llama3_decoder_layer_bf16_1x4096.md",
    "evoattention": "not scaled: see profiles/evoattention_bf16_1x64x4x256x32.md",
    "evoattention_n384": "not scaled: see profiles/evoattention_bf16_1x64x4x256x32.md",
}


def _source_digest(files):
    import hashlib

    h = hashlib.sha256()
    for f in files:
        with open(os.path.join(ROOT, "evograd_b200", "csrc", f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:12]


def ncu_traffic(workload):
    """(bytes per launch, where they come from); bytes are None when no capture
    exists or the kernel sources changed after it was taken."""
    entry = TRAFFIC_NCU.get(workload)
    if entry is None:
        return None, TRAFFIC_NOTES.get(workload, "no ncu capture for this workload")
    try:
        now = _source_digest(entry["sources"])
    except OSError:
        now = "unreadable"
    where = f"{entry['profile']} @ csrc digest {entry['digest']}"
    if now != entry["digest"]:
        return None, f"stale: {where}, sources now {now}"
    return entry["bytes"], where


def run_reference(args):
    """The reference's own implementation of the path: its CPU autograd oracle
    (restated in oracle/), all host threads, on the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    # a launcher sets OMP_NUM_THREADS=1 for its ranks; only this rank computes
    torch.set_num_threads(os.cpu_count() or 1)
    wl = WORKLOADS[args.workload](torch.device("cpu"))
    s = wl.make(torch.device("cpu"))
    for _ in range(min(args.warmup, 1)):
        wl.cpu_step(s)
    steps = max(1, args.steps)
    # bound the whole run to a few minutes
    t0 = time.perf_counter()
    wl.cpu_step(s)
    one = time.perf_counter() - t0
    steps = max(1, min(steps, int(150.0 / max(one, 1e-3))))
    t0 = time.perf_counter()
    for _ in range(steps):
        wl.cpu_step(s)
    sec = (time.perf_counter() - t0) / steps
    hbm = wl.bound == "hbm"
    metric, unit = _metric_of(wl)
    work, sample = wl.cpu_sample()
    value = work / sec / (1e9 if hbm else 1e12)
    cores = torch.get_num_threads()
    line = {
        "impl": "reference",
        "metric": metric,
        "value": round(value, 4), "unit": unit, "n_gpus": args.gpus, "steps": steps,
        "warmup": min(args.warmup, 1) + 1, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic", "config": _common_config(wl, max(world, args.gpus)),
        "run": {"device": "host CPU", "threads": cores},
        "cpu_baseline": {"value": round(value, 4), "unit": unit, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 4), "unit": unit, "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="layernorm")
    ap.add_argument("--source-digest", default=None, metavar="WORKLOAD",
                    help="print the digest of a workload's kernel sources and exit")
    ap.add_argument("--no-per-op", action="store_true", help="skip the per-operator table")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-strong", action="store_true", help="N > 1: skip the strong-scaling table")
    ap.add_argument("--no-parity", action="store_true", help="N > 1: skip the untimed result check")
    ap.add_argument("--attention-shape", default=None, metavar="B,H,S",
                    help="smaller causal-attention case (profiling captures only; head_dim stays 128)")
    ap.add_argument("--rows", type=int, default=None,
                    help="fewer rows for the chosen row-wise workload (profiling captures only)")
    ap.add_argument("--hidden", type=int, default=None,
                    help="another row width for a norm workload (profiling captures only)")
    ap.add_argument("--rope-batch", type=int, default=None,
                    help="smaller batch for the rope workload (profiling captures only)")
    ap.add_argument("--evo-shape", default=None, metavar="B,S,H,N,D",
                    help="another evoattention case (profiling captures only)")
    args = ap.parse_args()
    if args.source_digest:
        print(_source_digest(TRAFFIC_SOURCES[args.source_digest]))
        return
    if args.rows:
        cls = WORKLOADS[args.workload]
        if not hasattr(cls, "rows"):
            ap.error(f"--rows does not apply to workload {args.workload}")
        cls.rows = args.rows
        if isinstance(getattr(cls, "name", None), str) and cls.name:
            cls.name = f"{cls.name}_rows{args.rows}"
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.attention_shape:
        b, h, sq = (int(t) for t in args.attention_shape.split(","))
        AttentionWL.B, AttentionWL.H, AttentionWL.S = b, h, sq
        AttentionWL.name = f"causal_attention_bf16_{b}x{h}x{sq}x128"
    if args.hidden:
        cls = WORKLOADS[args.workload]
        if not hasattr(cls, "hidden"):
            ap.error(f"--hidden does not apply to workload {args.workload}")
        cls.hidden = args.hidden
    if args.rope_batch:
        RopeWL.B = args.rope_batch
        RopeWL.name = f"rope_bf16_qk_{args.rope_batch}x4096x32x128"
    if args.evo_shape:
        b, sq, h, n, dd = (int(t) for t in args.evo_shape.split(","))
        EvoAttentionWL.B, EvoAttentionWL.S, EvoAttentionWL.H = b, sq, h
        EvoAttentionWL.N, EvoAttentionWL.D = n, dd
        EvoAttentionWL.name = f"evoattention_bf16_{b}x{sq}x{h}x{n}x{dd}"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
