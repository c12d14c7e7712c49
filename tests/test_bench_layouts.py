"""``bench.py --plan-only`` walks the benchmark's own code path up to the compiled plan on virtual
devices (meta tensors, mock runtime: nothing is allocated, no CUDA device is touched): the default
layouts for 1, 2, 4 and 8 GPUs and the Llama-3 / Mixtral configurations compile for the full model
shapes, with the layouts and schedules the documentation names."""
import json
import pathlib
import subprocess
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent


def _plan(*flags):
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--plan-only", *flags], stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, text=True, timeout=600, cwd=str(ROOT))
    assert proc.returncode == 0, proc.stderr[-3000:]
    return json.loads([l for l in proc.stdout.splitlines() if l.startswith("{")][-1])


@pytest.mark.parametrize("n,parallelism,schedule,microbatches", [
    (1, "pp1xdp1xtp1", "1f1b", 2), (2, "pp1xdp1xtp2", "1f1b", 4), (4, "pp4xdp1xtp1", "zero-bubble-h2", 8),
    (8, "pp4xdp1xtp2", "1f1b", 16)])
def test_default_layouts_compile_for_the_full_llama2_shape(n, parallelism, schedule, microbatches):
    p = _plan("--gpus", str(n))
    assert (p["parallelism"], p["schedule"], p["microbatches"]) == (parallelism, schedule, microbatches)
    stages = int(parallelism[2])
    if stages > 1:
        assert p["reshards"] >= 2 * (stages - 1) * microbatches
        assert p["stats"]["schedule"] == schedule
    assert p["layers_per_stage"] == ([8, 9, 8, 7] if n == 8 else None)
    # temporaries must leave room for parameters and optimizer state on a 180 GB part
    assert 0 < p["temp_gb_per_device"] < 100


def test_llama3_fsdp_tp_forced_reshard_and_mixtral_expert_parallel_plans():
    l3 = _plan("--gpus", "8", "--model", "llama3_8b", "--seq", "8192", "--per-gpu-batch", "4", "--microbatch", "1",
               "--pp", "2", "--dp", "2", "--tp", "2", "--fsdp", "--force-reshard")
    assert l3["parallelism"] == "pp2xdp2xtp2" and l3["layers_per_stage"] == [16, 16] and l3["microbatches"] == 16
    moe = _plan("--gpus", "8", "--model", "mixtral_8x7b", "--seq", "4096", "--per-gpu-batch", "2", "--microbatch", "1",
                "--pp", "2", "--dp", "4", "--tp", "1")
    assert moe["parallelism"] == "pp2xdp4xtp1" and moe["microbatches"] == 4 and moe["reshards"] > 0


def test_reference_arm_reports_why_it_is_unavailable():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1"],
                          stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300, cwd=str(ROOT))
    assert proc.returncode == 0
    line = json.loads(proc.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 10
