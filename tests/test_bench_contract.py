"""The benchmark's CPU arm runs without a GPU and prints the contracted JSON line."""
import json
import os
import subprocess
import sys

from conftest import ROOT


def test_reference_arm_prints_the_contract_line():
    env = dict(os.environ)
    env.pop("RANK", None)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--cpu-seconds", "0.5", "--k", "1024"],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["value"] > 0 and d["unit"] == "TOPS" and d["higher_is_better"] is True
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]


def test_reference_arm_is_silent_on_other_ranks():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_own_arm_refuses_to_run_without_a_gpu():
    """There is no CPU path behind bench.py's own arm: without a CUDA device it stops
    with an error instead of timing something else."""
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a CUDA device is present")
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0", "--m", "256",
                          "--n", "256", "--k", "256"], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode != 0 and out.stdout.strip() == ""
    assert "CUDA" in out.stderr


import pytest


@pytest.mark.gpu
def test_own_arm_prints_the_contract_line_with_parity(cuda):
    """bench.py's own arm on a small problem: the contracted keys, a roofline block, an end-to-end leg through
    the C ABI with host buffers, kernel launches counted, and the samples compared with the oracle all equal."""
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "3", "--warmup", "3", "--m", "2048", "--n", "2048",
                          "--k", "1024", "--no-cpu", "--no-sweep", "--no-secondary", "--no-probe"],
                         capture_output=True, text=True, timeout=900, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "clocks", "gpu_launches", "e2e", "parity"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 3 and d["value"] > 0 and d["gpu_launches"] >= 9
    assert set(("bound", "achieved", "peak", "unit", "frac", "traffic")) <= set(d["roofline"])
    assert d["e2e"]["value"] > 0 and d["e2e"]["h2d_bytes_per_step"] == 2048 * 1024 * 4
    assert d["e2e"]["d2h_bytes_per_step"] == 2048 * 2048 * 4 and d["e2e"]["matches_device_run"] is True
    assert d["parity"]["mismatches"] == 0 and d["parity"]["checked"] >= 90
