"""The benchmark's reference arm (the CPU oracle's layer step, no GPU needed) prints one JSON
line with the keys the harness reads; the GPU arm refuses to run without a CUDA device."""
import json
import subprocess
import sys
from pathlib import Path

REPO = Path(__file__).resolve().parent.parent


def run_bench(*args):
    return subprocess.run([sys.executable, str(REPO / "bench.py"), *args], capture_output=True, text=True,
                          timeout=900, cwd=str(REPO))


def test_reference_arm_prints_the_contract_line():
    r = run_bench("--impl", "reference", "--steps", "2", "--warmup", "3", "--cpu-seqs", "2")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "moe_decode_layer_latency" and d["unit"] == "us"
    assert d["higher_is_better"] is False and d["n_gpus"] == 1 and d["vs_baseline"] is None
    assert d["steps"] == 2 and d["warmup"] == 3 and d["value"] > 0
    assert abs(d["ms_per_step"] * 1e3 - d["value"]) < 1.0
    assert "workload" in d["config"] and "model" not in d["config"]
    base = d["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == d["value"] and "2 of 256" in base["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        import pytest

        pytest.skip("a CUDA device is present")
    r = run_bench("--steps", "1", "--warmup", "3", "--ops", "none", "--no-cpu")
    assert r.returncode != 0
    assert "no CPU path" in r.stderr or "CUDA" in r.stderr
