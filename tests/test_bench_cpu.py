"""Host-side logic of bench.py that needs no GPU: replay statistics, the shard
classes of the strong-scaling table, the stale-capture rule of the traffic table
and the reference arm's JSON line."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(REPO))
import bench  # noqa: E402


def test_quantiles_interpolate():
    vals = sorted([1.0, 2.0, 3.0, 4.0, 5.0])
    assert bench._quantile(vals, 0.5) == 3.0
    assert bench._quantile(vals, 0.2) == pytest.approx(1.8)
    assert bench._quantile(vals, 0.8) == pytest.approx(4.2)
    assert bench._quantile([7.0], 0.8) == 7.0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_strong_scaling_shards_cut_the_baseline_shapes(world):
    for name in ("softmax", "layernorm", "rmsnorm", "swiglu"):
        cls = bench.WORKLOADS[name]
        shard = cls.shard_of(world)
        assert shard is not None and shard.rows * world == cls.rows
    rope = bench.RopeWL.shard_of(world)
    assert rope.B * world == bench.RopeWL.B and rope.S == bench.RopeWL.S
    attn = bench.AttentionWL.shard_of(world)
    assert attn.B * attn.H * world == bench.AttentionWL.B * bench.AttentionWL.H
    assert bench.SoftmaxWL.shard_of(3) is None  # 4096 rows do not divide by 3


def test_traffic_is_withheld_when_the_sources_changed(monkeypatch):
    files = bench.TRAFFIC_SOURCES["layernorm"]
    digest = bench._source_digest(files)
    monkeypatch.setitem(bench.TRAFFIC_NCU, "layernorm",
                        {"bytes": 1.0e6, "profile": "profiles/x.md", "sources": files, "digest": digest})
    assert bench.ncu_traffic("layernorm") == (1.0e6, f"profiles/x.md @ csrc digest {digest}")
    monkeypatch.setitem(bench.TRAFFIC_NCU, "layernorm",
                        {"bytes": 1.0e6, "profile": "profiles/x.md", "sources": files, "digest": "0" * 12})
    value, where = bench.ncu_traffic("layernorm")
    assert value is None and where.startswith("stale")
    assert bench.ncu_traffic("no such workload") == (None, "no ncu capture for this workload")


def test_committed_traffic_entries_match_the_sources():
    """An entry whose digest no longer matches reads as null in the bench line; this
    test says so before a benchmark run does."""
    stale = [k for k in bench.TRAFFIC_NCU if bench.ncu_traffic(k)[0] is None]
    assert not stale, f"re-capture or drop: {stale}"


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(REPO / "bench.py"), "--impl", "reference", "--workload",
                          "softmax", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=REPO)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["gpu_launches"] == 0
    assert line["unit"] == "GB/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["config"] == {"workload": "softmax_f32_4096x1024", "shape": [4096, 1024],
                              "saved": "y", "parallelism": "1 gpu"}
