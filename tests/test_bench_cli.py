"""bench.py on a machine without a GPU: the reference arm runs the CPU path and prints the contract's line, the repo arm
refuses to run (there is no CPU fallback to time by accident)."""
import json
import subprocess
import sys

import pytest

from tests.conftest import ROOT

torch = pytest.importorskip("torch")


def run_bench(*args, timeout=600):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=timeout, cwd=str(ROOT))


def test_reference_arm_prints_the_contract_line():
    res = run_bench("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads([l for l in res.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["metric"] == "moe_decode_us_per_token" and line["unit"] == "us/token"
    assert line["higher_is_better"] is False and line["n_gpus"] == 1 and line["steps"] == 1 and line["vs_baseline"] is None
    assert line["value"] > 0 and line["gpu_launches"] == 0
    assert line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["cpu_baseline"]["value"] == line["value"] == line["e2e"]["value"]
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "11 stacked MoE layers" in line["config"]["workload"]


def test_reference_arm_of_a_path_the_reference_has_no_cpu_code_for():
    res = run_bench("--impl", "reference", "--workload", "lm_head")
    assert res.returncode == 0
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "no CPU function" in line["unavailable"]


def test_repo_arm_refuses_to_run_without_a_device():
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    res = run_bench("--steps", "1", "--warmup", "1")
    assert res.returncode != 0
    assert "needs a CUDA device" in (res.stderr + res.stdout)


def test_reference_arm_on_a_rank_other_than_zero_does_nothing():
    import os
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"],
                         capture_output=True, text=True, timeout=120, cwd=str(ROOT), env=env)
    assert res.returncode == 0 and res.stdout.strip() == ""
