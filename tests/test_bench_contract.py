"""bench.py's reference arm (the CPU restatement timed on host cores) runs without a GPU: check the JSON line it
prints carries the contract's keys, and that the GPU arm refuses loudly when there is no device."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=300):
    env = dict(os.environ, OMP_NUM_THREADS=str(min(os.cpu_count() or 1, 8)))
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py")] + args, capture_output=True, text=True,
                          timeout=timeout, env=env, cwd=ROOT)


def test_reference_arm_prints_one_contract_line():
    res = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "vgg16_conv_images_per_s" and line["unit"] == "images/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == line["value"] and cb["sample"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0
    assert line["gpu_launches"] == 0 and line["data"] == "synthetic"


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_gpu_arm_fails_loudly_without_a_device():
    res = _run(["--steps", "1", "--warmup", "0", "--skip-cpu-baseline"], timeout=120)
    assert res.returncode != 0
    assert "no CPU path" in (res.stderr + res.stdout)


@pytest.mark.gpu
def test_gpu_arm_line_carries_both_roofline_fractions_and_the_error_columns():
    res = _run(["--workload", "cfg2", "--steps", "3", "--warmup", "3", "--skip-cpu-baseline"], timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = json.loads(res.stdout.strip().splitlines()[-1])
    assert line["metric"] == "conv_images_per_s" and line["scaling"] == "strong" and line["gpu_launches"] > 0
    rf = line["roofline"]
    for key in ("bound", "achieved", "peak", "unit", "frac", "frac_contract", "traffic", "kernel"):
        assert key in rf
    assert 0 < rf["frac_contract"] <= 1.5 and 0 < line["step_roofline_frac_contract"] <= 1.5
    layer = line["layers"][0]
    assert layer["contract"] == "F(4x4,3x3)" and layer["roof_frac_contract"] > 0 and layer["algo"] in ("staged", "row", "fused")
    err = line["errors"]["layers"][0]
    for who in ("engine", "reference_algebra"):
        assert set(err[who]) == {"E_B", "E_A", "E_C", "P999"}
    assert err["engine"]["E_B"] <= line["errors"]["tolerance_E_B"]
    e2e = line["e2e"]
    assert e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0 and e2e["value"] > 0
    assert "F(4x4,3x3) staged" in line["config"]["winograd"]
