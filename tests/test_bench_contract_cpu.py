"""The parts of bench.py's contract that can be checked without a GPU: the reference arm's JSON line,
the workload description, and that our own arm refuses to run (no CPU fallback) when there is no device."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=300):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=timeout)


def test_reference_arm_prints_the_contract_line(oracle):
    r = _run("--impl", "reference", "--steps", "2", "--warmup", "1")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["n_gpus"] == 1 and d["steps"] == 2 and d["higher_is_better"] is True
    assert d["unit"] == "GB/s" and d["value"] > 0 and d["ms_per_step"] > 0 and d["data"] == "synthetic" and d["vs_baseline"] is None
    assert d["config"]["workload"].startswith("cfg2 decode GEMV") and d["config"]["K"] == 4096 and d["config"]["N_per_gpu"] == 11008
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    e = d["e2e"]
    assert e["value"] == d["value"] and e["unit"] == d["unit"] and e["h2d_bytes_per_step"] == 0 and e["d2h_bytes_per_step"] == 0


def test_workload_description():
    sys.path.insert(0, ROOT)
    import bench

    one = bench.workload_config(4096, 11008, 1, 1)
    assert one["parallelism"] == "single GPU" and one["gather_message_bytes_per_rank"] == 0 and "model" not in one
    eight = bench.workload_config(8192, 3584, 1, 8, "cfg4")
    assert eight["N_total"] == 28672 and eight["gather_message_bytes_per_rank"] == 14336 and "x8" in eight["parallelism"]


def test_own_arm_needs_a_gpu():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    r = _run("--steps", "1", "--warmup", "1", "--no-extras", timeout=120)
    assert r.returncode != 0  # fails loudly: there is no CPU path to fall back to
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]


def test_reference_arm_under_a_launcher_runs_on_rank_zero_only():
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29577")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                       cwd=ROOT, capture_output=True, text=True, timeout=120, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")]  # the other ranks exit without work
