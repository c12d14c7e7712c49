"""The one-process-per-device ("dist") topology on CPU: gloo ranks started by torchrun run the
compiled pipeline x tensor parallel step and compare their tiles with the eager step; a rank
that leaves between steps is detected by the others on the host (an error status within the
process-group timeout), with no device involved."""
import json
import os
import socket
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "multiproc", "dist_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(nproc, *args, timeout=420):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), WORKER, *map(str, args)]
    env = dict(os.environ, OMP_NUM_THREADS="1", GLOO_SOCKET_IFNAME="lo", CUDA_VISIBLE_DEVICES="")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


@pytest.mark.parametrize("pp,tp,dp", [(2, 1, 1), (2, 2, 1), (1, 1, 2), (2, 1, 2)])
def test_dist_topology_step_matches_eager(pp, tp, dp):
    r = _run(pp * tp * dp, "step", pp, tp, dp)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = next(l for l in r.stdout.splitlines() if "DIST_STEP_OK" in l)
    assert json.loads(line)["DIST_STEP_OK"] is True


def test_task_that_moves_between_stages_runs_on_ranks_its_template_was_not_compiled_for():
    r = _run(4, "moving", 2, 2)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = next(l for l in r.stdout.splitlines() if "DIST_MOVING_OK" in l)
    assert json.loads(line)["DIST_MOVING_OK"] is True


def test_rank_leaving_between_steps_is_reported_on_the_host():
    r = _run(2, "leave", 2, 1, timeout=240)
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert any(l.get("left") for l in lines), r.stdout[-2000:] + r.stderr[-2000:]
    survivors = [l for l in lines if "outcome" in l]
    assert survivors and all(l["outcome"].startswith("error") for l in survivors), lines
    assert all(l["seconds"] < 60 for l in survivors)


def test_two_ranks_save_and_reload_a_checkpoint(tmp_path):
    r = _run(2, "ckpt", 2, 1, str(tmp_path / "ckpt"), timeout=240)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    line = next(l for l in r.stdout.splitlines() if "DIST_CKPT_OK" in l)
    assert json.loads(line)["DIST_CKPT_OK"] is True
