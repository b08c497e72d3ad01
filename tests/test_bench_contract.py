"""bench.py contract checks that need no GPU: the reference arm (the reference's math on the host CPU)
runs anywhere and must print one JSON line with the agreed keys; flops accounting is pinned."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT


@pytest.mark.timeout(300)
def test_reference_arm_prints_the_contract_line():
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=280, cwd=ROOT)
    assert res.returncode == 0, res.stderr
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "causal_attention_fwd_bwd_tflops" and d["unit"] == "TFLOP/s"
    assert d["higher_is_better"] is True and d["value"] > 0 and d["n_gpus"] == 1
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "c2" in d["config"]["workload"]


def test_flop_accounting_matches_the_benchmark_spec():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.flops(8, 12, 1024, 64) == pytest.approx(45.10e9, rel=1e-3)      # config 2
    assert bench.flops(2, 16, 8192, 128) == pytest.approx(1.924e12, rel=1e-3)    # config 3
    assert bench.flops(2, 32, 16384, 128) == pytest.approx(15.39e12, rel=1e-3)   # longest sweep point
    assert bench.WORKLOADS["c2"] == (8, 12, 1024, 64)


def test_other_ranks_of_the_reference_arm_exit_quietly():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""


def test_sampled_launches_of_the_timed_region():
    """Events around a kernel undo its back-to-back launch, so a short timed region carries four sampled steps and a
    long one about eight; together with the eight steps sampled behind the region every run has at least eight samples."""
    sys.path.insert(0, ROOT)
    import bench
    for steps in (1, 3, 8, 20, 50, 159, 160, 2000):
        stride = bench.default_event_stride(steps)
        inside = steps // stride
        assert stride >= 1 and 1 <= inside <= 8, (steps, stride, inside)
        assert inside + bench.SAMPLED_STEPS_AFTER >= 8
    assert bench.default_event_stride(20) == 5 and bench.default_event_stride(2000) == 250
