"""bench.py's reference arm on CPU: one JSON line with the contract's keys (the same line the GPU arm prints,
with "impl": "reference" and a cpu_baseline that describes the run)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_one_contract_line():
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode == 0, run.stderr[-2000:]
    lines = [line for line in run.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "q8_dit_block_linear_tflops" and line["unit"] == "TFLOP/s"
    assert line["n_gpus"] == 1 and line["steps"] == 1 and line["warmup"] == 0 and line["higher_is_better"] is True
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["vs_baseline"] is None and line["data"] == "synthetic"
    assert "workload" in line["config"] and "model" not in line["config"]
    baseline = line["cpu_baseline"]
    assert baseline["kind"] in ("port", "reference") and baseline["cores"] >= 1 and baseline["value"] == line["value"]
    assert baseline["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["unit"] == line["unit"]
    assert e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        import pytest
        pytest.skip("a GPU is present")
    run = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert run.returncode != 0                       # no CPU fallback: the product arm needs the CUDA path
    assert not [line for line in run.stdout.splitlines() if line.strip().startswith("{")]
