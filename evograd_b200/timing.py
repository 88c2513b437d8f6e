"""Device-side timing for the benchmark driver: CUDA events on the launching
stream, buffer rotation so that every timed iteration reads data that is not in
L2, max over ranks, clock sampling, roofline arithmetic."""

from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent.parent

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def measured_peaks() -> tuple[dict, str]:
    """Roofline denominators: the pool's measured copy bandwidth and bf16 GEMM
    rate when ``MEASURED_PEAKS.json`` is present, else the stated fallback."""
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return {k: float(data[k]) for k in FALLBACK_PEAKS if k in data} | {}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


def l2_bytes(device=None) -> int:
    return int(torch.cuda.get_device_properties(device or torch.cuda.current_device()).L2_cache_size)


def rotation_count(bytes_per_set: int, device=None) -> int:
    """How many independent buffer sets to cycle through so that a set's lines
    have been evicted from L2 (2x its size written since) when it comes round."""
    need = 2 * l2_bytes(device)
    return max(2, -(-need // max(1, bytes_per_set)) + 1)


def time_steps(step, steps: int, warmup: int, *, barrier=None, finalize=None) -> float:
    """Runs ``step(i)`` warmup+steps times; returns milliseconds for EXACTLY
    ``steps`` iterations measured with CUDA events on the current stream,
    bracketed by a barrier and a device synchronise on both sides."""
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step(warmup + i)
    if finalize is not None:
        finalize()  # e.g. join a side stream: everything a step produced is done before `stop`
    stop.record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return start.elapsed_time(stop)


class SectionTimer:
    """Per-section device time inside a timed loop: records an event pair around
    each call on the current stream and sums them after the final synchronise."""

    def __init__(self):
        self.pairs: dict[str, list] = {}

    def run(self, name: str, fn):
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        out = fn()
        b.record()
        self.pairs.setdefault(name, []).append((a, b))
        return out

    def totals_ms(self) -> dict[str, tuple[float, int]]:
        torch.cuda.synchronize()
        return {k: (sum(a.elapsed_time(b) for a, b in v), len(v)) for k, v in self.pairs.items()}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed
    region runs (read-only; no setting is changed)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int, period_ms: int = 100):
        self.device_index = device_index
        self.period_ms = period_ms
        self.proc = None
        self.lines: list[str] = []
        self._thread = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self._thread = threading.Thread(target=self._pump, daemon=True)
            self._thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self) -> dict:
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        want = str(self.device_index)
        if visible:
            ids = [v.strip() for v in visible.split(",")]
            if self.device_index < len(ids) and ids[self.device_index].isdigit():
                want = ids[self.device_index]
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9 or parts[0] != want:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax),
                "reasons": sorted(reasons), "samples": len(sm)}
