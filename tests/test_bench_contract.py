"""bench.py prints one JSON line with the keys its callers read: the reference arm (CPU, runs
everywhere) and the CUDA arm (GPU)."""
import json
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
COMMON = ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
          "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e")


def run_bench(*arguments, timeout):
    completed = subprocess.run([sys.executable, str(ROOT / "bench.py"), *arguments], cwd=ROOT,
                               capture_output=True, text=True, timeout=timeout)
    assert completed.returncode == 0, completed.stderr[-2000:]
    lines = [line for line in completed.stdout.splitlines() if line.startswith("{")]
    assert len(lines) == 1, completed.stdout[-2000:]
    return json.loads(lines[0])


def check_common(record, steps, warmup):
    for key in COMMON:
        assert key in record, key
    assert record["metric"] == "mxfp8_prefill_gemm_tflops" and record["unit"] == "TFLOP/s"
    assert record["steps"] == steps and record["warmup"] == warmup and record["n_gpus"] == 1
    assert record["higher_is_better"] is True and record["vs_baseline"] is None
    assert record["value"] > 0 and record["ms_per_step"] > 0
    assert "workload" in record["config"] and "model" not in record["config"]
    baseline = record["cpu_baseline"]
    assert baseline["kind"] in ("port", "reference") and baseline["cores"] >= 1 and baseline["sample"]
    for key in ("value", "unit", "h2d_bytes_per_step", "d2h_bytes_per_step"):
        assert key in record["e2e"], key


def test_reference_arm_line():
    record = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0", timeout=600)
    check_common(record, 1, 0)
    assert record["impl"] == "reference"
    assert record["cpu_baseline"]["value"] == record["value"]
    assert record["e2e"]["value"] == record["value"]
    assert record["e2e"]["h2d_bytes_per_step"] == 0 and record["e2e"]["d2h_bytes_per_step"] == 0


@pytest.mark.gpu
def test_cuda_arm_line():
    record = run_bench("--steps", "3", "--warmup", "3", "--repeats", "5", timeout=900)
    check_common(record, 3, 3)
    assert record["repeats"] == 5
    assert record["ms_per_step_min"] <= record["ms_per_step"] <= record["ms_per_step_max"]
    assert "impl" not in record or record["impl"] != "reference"
    roofline = record["roofline"]
    for key in ("bound", "achieved", "peak", "unit", "frac", "traffic"):
        assert key in roofline, key
    assert roofline["bound"] == "tensor" and 0.0 < roofline["frac"] < 1.5
    assert abs(roofline["frac"] - roofline["achieved"] / roofline["peak"]) < 1e-6
    assert record["gpu_launches"] > 0
    assert record["e2e"]["h2d_bytes_per_step"] > 0 and record["e2e"]["d2h_bytes_per_step"] > 0
    assert record["e2e"]["value"] < record["value"]          # host copies are inside its timed region
    for key in ("sm_mhz", "sm_max_mhz", "reasons"):
        assert key in record["clocks"], key
    assert record["clocks"]["samples"] >= 1
    # the other half of the headline metric: decode GEMV bandwidth, 4 shapes x M in {1, 4, 8}
    decode = record["decode"]
    assert len(decode["results"]) == 12 and 0.0 < decode["min_frac"] <= decode["mean_frac"] < 1.2
    assert {entry["m"] for entry in decode["results"]} == {1, 4, 8}
    assert len(decode["fp4_vector_results"]) == 4 and len(decode["marlin_results"]) == 12
    assert {entry["m"] for entry in decode["w4a16_results"]} == {1, 16, 256}
    assert len(decode["nvfp4_gemm_results"]) == 4 and all(entry["tflops"] > 0 for entry in decode["nvfp4_gemm_results"])
    assert {(entry["shape"], entry["m"]) for entry in decode["mxfp8_weight_only_results"]} == {
        (shape, m) for shape in ("qkv", "o", "gate_up", "down") for m in (1, 4, 8)}
    # the reference's own kernels beside this library's (present when oracle/_ref was built)
    for entry in record["reference_kernels"]["results"]:
        assert entry["us"] > 0 and entry["reference_us"] > 0
