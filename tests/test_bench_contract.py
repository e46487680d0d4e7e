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
