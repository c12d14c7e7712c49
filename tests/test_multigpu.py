"""Multi-GPU tests (need >= 2 CUDA devices): each launches one process per GPU with torchrun.
NVLS is switched off for NCCL so that a failing rank cannot fault its peers."""
import os
import subprocess
import sys

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script, nproc, *args, timeout=240, port=29531):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), script, *args]
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_fused_gemm_allreduce_matches_nccl():
    r = _torchrun(os.path.join(ROOT, "tests", "multigpu", "fused_tp_worker.py"), 2)
    assert "FUSED_TP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def _step(nproc, *args, port):
    import json
    r = _torchrun(os.path.join(ROOT, "tests", "multigpu", "step_worker.py"), nproc, *map(str, args), port=port)
    line = next((l for l in r.stdout.splitlines() if "STEP_OK" in l), None)
    assert line is not None, r.stdout[-2000:] + r.stderr[-3000:]
    return json.loads(line)


def test_pipeline_step_uses_the_peer_reshard_kernel_and_matches_eager():
    out = _step(2, 2, 1, 1, port=29532)
    assert out["STEP_OK"], out
    assert out["peer_reshard_uses"] > 0          # stage-boundary tiles were pulled from peer memory
    # the stage tasks wrote their boundary outputs straight into the peer-mapped tiles; only step
    # arguments that cross a boundary (token ids, labels: nothing produces them) are copied in
    assert out["reshard_sources_written_in_place"] >= 0.8 * out["peer_reshard_uses"], out
    assert out["reshard_sources_copied"] <= 0.2 * out["peer_reshard_uses"], out


def test_tensor_parallel_step_with_fused_all_reduce_matches_eager():
    out = _step(2, 1, 1, 2, port=29533)
    assert out["STEP_OK"], out


def test_data_parallel_fsdp_step_matches_eager():
    out = _step(2, 1, 2, 1, "fsdp", port=29534)
    assert out["STEP_OK"], out
    assert out["peer_collective_calls"] > 0      # parameter gathers / gradient reductions ran on the pull kernels


def test_expert_parallel_step_with_fused_dispatch_matches_eager():
    out = _step(2, 1, 2, 1, "moe", port=29535)
    assert out["STEP_OK"], out
    assert out["peer_moe_calls"] > 0             # router + dispatch and combine ran on the peer-memory kernels


def test_sequence_parallel_step_with_fused_reduce_scatter_and_all_gather_matches_eager():
    out = _step(2, 1, 1, 2, "sp", port=29536)
    assert out["STEP_OK"], out
    # the projections ran on the GEMM + reduce-scatter and all-gather + GEMM kernels, none on the all-reduce one
    assert out["fused_calls"].get("rs", 0) > 0 and out["fused_calls"].get("ag", 0) > 0, out
    assert out["fused_calls"].get("ar", 0) == 0, out
