"""CPU-only checks of bench.py's contract: the reference arm prints one JSON line with the agreed
keys (it times the oracle port on the host cores), and the main arm refuses to run without a GPU
instead of falling back to anything."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def run_bench(*args, timeout=600):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout, cwd=str(ROOT))


def test_reference_arm_prints_the_contract_line():
    r = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "w8a8_linear_stack_int8_tops" and line["unit"] == "TOP/s"
    assert line["higher_is_better"] is True and line["value"] > 0 and line["steps"] == 1
    assert line["config"]["workload"].startswith("cfg1")
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # without a GPU the same-GPU comparator says so instead of failing the line
    if not torch.cuda.is_available():
        assert "unavailable" in line["reference_cuda_ops_same_gpu"]


def test_other_ranks_of_the_reference_arm_do_no_work(monkeypatch):
    monkeypatch.setenv("RANK", "1")
    r = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0", "--gpus", "2", timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_main_arm_has_no_cpu_fallback():
    r = run_bench("--steps", "1", "--warmup", "3", timeout=300)
    assert r.returncode != 0
    assert "no CPU path" in (r.stderr + r.stdout)
