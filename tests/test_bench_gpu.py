"""The benchmark entry point on one GPU with the tiny model: the JSON line a driver parses, for the
engine arm and for the arm that goes through torch DistributedDataParallel."""

import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*flags):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"):
        env.pop(k, None)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--model", "tiny", "--steps", "3", "--warmup", "3", *flags],
                         capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-3000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, out.stdout
    return json.loads(lines[0])


@pytest.mark.parametrize("flags", [(), ("--ddp",)], ids=["engine", "ddp"])
def test_bench_prints_one_json_line(flags):
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    line = _run(*flags)
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "gpu_launches", "e2e"):
        assert key in line, key
    assert line["n_gpus"] == 1 and line["steps"] == 3 and line["warmup"] == 3 and line["dtype"] == "bf16"
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["gpu_launches"] > 0
    assert line["committed_steps"] >= 6 and line["final_loss"] == line["final_loss"]  # every step committed, finite loss
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] == 4
    assert ("ddp" in line["config"]["parallelism"]) == bool(flags)
