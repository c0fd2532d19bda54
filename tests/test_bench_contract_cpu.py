"""CPU-only checks of bench.py's contract: the reference arm prints one JSON line with the agreed
keys (without a GPU it times the oracle port on the host cores and says why the reference's CUDA
operators were not used), both arms name the workload with the same words, and the main arm refuses
to run without a GPU instead of falling back to anything."""
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
    assert line["config"]["workload"].startswith("cfg3") and line["scaling"] == "strong"
    cb = line["cpu_baseline"]
    assert cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if not torch.cuda.is_available():
        # no GPU: the CPU port stands in and the line says why the reference's CUDA operators did not run
        assert cb["kind"] == "port" and "no CUDA device" in line["reference_cuda_unavailable"]


def test_both_arms_name_the_workload_identically():
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    s = bench.workload_string("cfg3", 24, 64)
    assert "64 independent worlds x 2048 rows = 131072" in s
    assert s == bench.workload_string("cfg3", 24)  # nothing rank- or GPU-count-dependent in it
    assert bench.layer_gemm_algorithmic_bytes(512) > bench.WEIGHT_BYTES_LAYER


def test_other_ranks_of_the_reference_arm_do_no_work(monkeypatch):
    monkeypatch.setenv("RANK", "1")
    r = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0", "--gpus", "2", timeout=120)
    assert r.returncode == 0 and r.stdout.strip() == ""


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_main_arm_has_no_cpu_fallback():
    r = run_bench("--steps", "1", "--warmup", "3", timeout=300)
    assert r.returncode != 0
    assert "no CPU path" in (r.stderr + r.stdout)
