"""The bench script's contract, as far as it can be checked without a GPU: the CPU arm (`--impl reference`:
the C port of the reference's SIMD kernels, gemm.rs:211-260,483-550, the one place besides the tests where
`oracle/` is executed) prints one JSON line with the agreed keys, and the product arm refuses to run without
a CUDA device instead of falling back to anything."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def _run(*args, env_extra=None, timeout=600):
    import os

    env = dict(os.environ)
    env.update(env_extra or {})
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], cwd=ROOT, env=env, timeout=timeout,
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)


def test_reference_arm_prints_the_agreed_line():
    res = _run("--impl", "reference", "--steps", "1", "--warmup", "3")
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1, res.stdout
    d = json.loads(lines[0])
    assert d["impl"] == "reference"
    assert d["metric"].startswith("decode tok/s") and d["unit"] == "tok/s" and d["higher_is_better"] is True
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] >= 3
    assert d["value"] > 0 and d["ms_per_step"] > 0
    # tok/s of a whole sweep = 1000 / ms per sweep
    assert abs(d["value"] * d["ms_per_step"] / 1000.0 - 1.0) < 1e-6
    assert d["vs_baseline"] is None and d["data"] == "synthetic" and d["gpu_launches"] == 0
    cfg = d["config"]
    assert cfg["workload"] == "bitnet2b_decode_sweep" and "model" not in cfg
    # 30 layers of q/k/v + o + gate/up + down at 2560 / 6912, four weights a byte
    per_layer = (2560 + 2 * 640 + 2560 + 2 * 6912) * 2560 // 4 + 2560 * 6912 // 4
    assert cfg["packed_weight_bytes"] == 30 * per_layer
    cb = d["cpu_baseline"]
    assert cb["kind"] == "port" and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["unit"] == "tok/s"
    assert "sample" in cb and "layers" in cb["sample"]
    e2e = d["e2e"]
    assert e2e == {"value": d["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_other_ranks_do_no_work():
    """Under a multi-process launch only rank 0 runs the CPU arm; the others leave with status 0 and print
    nothing."""
    res = _run("--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "3",
               env_extra={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29533"})
    assert res.returncode == 0, res.stderr[-2000:]
    assert not [l for l in res.stdout.splitlines() if l.startswith("{")]


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the refusal on a machine without a GPU")
def test_product_arm_refuses_to_run_without_a_gpu():
    res = _run("--steps", "1", "--warmup", "3", timeout=300)
    assert res.returncode != 0
    assert "no CPU fallback" in (res.stdout + res.stderr)
    assert not [l for l in res.stdout.splitlines() if l.startswith("{")]
