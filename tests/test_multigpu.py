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
