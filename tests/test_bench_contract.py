"""bench.py's output contract: one JSON line per run with the keys the two arms share. The reference arm runs on the CPU
(the oracle's softmax on all host cores); the GPU arm is checked on a short run."""
import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

BENCH = os.path.join(ROOT, "bench.py")


def run_bench(*args, timeout=600):
    out = subprocess.run([sys.executable, BENCH, *args], check=True, capture_output=True, text=True, timeout=timeout, cwd=ROOT).stdout
    lines = [ln for ln in out.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, out
    return json.loads(lines[0])


def test_reference_arm_prints_the_shared_contract():
    sys.path.insert(0, ROOT)
    import bench

    line = run_bench("--impl", "reference", "--steps", "1", "--warmup", "0")
    assert line["impl"] == "reference"
    assert line["metric"] == "softmax_hbm_gbs" and line["unit"] == "GB/s" and line["higher_is_better"] is True
    assert line["config"] == bench.headline_config()  # the very object the GPU arm prints
    assert line["value"] > 0 and line["n_gpus"] == 1
    cb = line["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_traffic_table_names_only_known_workloads():
    sys.path.insert(0, ROOT)
    import bench

    known = {"softmax", "gemm_f64", "gemm_bf16", "gemm_f32", "gemm_f32_exact", "conv_f32", "conv_bf16", "attention", "attention_causal",
             "block_f32", "block_bf16"}
    assert set(bench.NCU_TRAFFIC_BYTES) <= known
    assert bench.FP64_TFLOPS_BUILDER_MEASURED == 35.5


@pytest.mark.gpu
def test_gpu_arm_prints_the_contract(rt):
    sys.path.insert(0, ROOT)
    import bench

    line = run_bench("--steps", "3", "--warmup", "3", "--no-extras")
    assert line["metric"] == "softmax_hbm_gbs" and line["n_gpus"] == 1 and line["steps"] == 3 and line["warmup"] == 3
    assert line["config"] == bench.headline_config()
    assert line["scaling"] == "weak" and line["vs_baseline"] is None and line["dtype"] == "f32" and line["data"] == "synthetic"
    roof = line["roofline"]
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s" and roof["peak"] > 0
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9 and roof["traffic"] > 0
    assert line["gpu_launches"] == 3  # one kernel per step
    assert set(line["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}
    e2e = line["e2e"]
    assert e2e["h2d_bytes_per_step"] == 8192 * 4096 * 4 and e2e["d2h_bytes_per_step"] == 8192 * 4096 * 4
    assert 0 < e2e["value"] < line["value"]  # host buffers over PCIe cannot beat the HBM-resident number
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["value"] > 0
