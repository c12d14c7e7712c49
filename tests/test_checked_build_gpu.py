"""The checked kernel build: the same kernels compiled with index checks that record a status
code instead of trapping. Runs in a child process because the library is chosen at first load."""
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu

CHILD = textwrap.dedent(
    """
    import json, torch
    from multimesh_jax_b200.ops import _lib, kernels as K
    assert _lib.lib_path().name == "_mm_kernels_checked.so", _lib.lib_path()
    torch.manual_seed(0)
    dev = "cuda:0"
    out = {}
    # GEMM, normalisation and attention agree with fp32 PyTorch under the checked build too
    a = torch.randn(384, 512, device=dev, dtype=torch.bfloat16)
    w = torch.randn(256, 512, device=dev, dtype=torch.bfloat16)
    y = K.linear_fwd(a, w)
    ref = a.float() @ w.float().t()
    out["gemm_rel"] = float((y.float() - ref).norm() / ref.norm())
    x = torch.randn(300, 1024, device=dev, dtype=torch.bfloat16)
    g = torch.randn(1024, device=dev, dtype=torch.bfloat16)
    yn, rstd = K.rmsnorm_fwd(x, g, 1e-5)
    refn = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * g.float()
    out["norm_rel"] = float((yn.float() - refn).norm() / refn.norm())
    table = torch.randn(64, 256, device=dev, dtype=torch.bfloat16)
    ids = torch.randint(0, 64, (40,), device=dev)
    e = K.embedding_fwd(table, ids)
    out["emb_exact"] = bool(torch.equal(e, table[ids]))
    torch.cuda.synchronize()
    out["status_clean"] = K.read_status(clear=True)
    # a negative token id is masked in every build (the row reads as zeros); the checked build
    # also reports it
    bad = ids.clone(); bad[3] = -7
    e2 = K.embedding_fwd(table, bad)
    torch.cuda.synchronize()
    out["bad_row_zero"] = bool((e2[3] == 0).all())
    out["status_bad"] = K.read_status(clear=True)
    out["status_after_clear"] = K.read_status(clear=False)
    print("RESULT " + json.dumps(out))
    """
)


def test_checked_build_matches_and_reports_a_bad_index_without_a_fault():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    env = dict(os.environ, MM_CHECKED="1")
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT ")][-1]
    out = json.loads(line[len("RESULT "):])
    assert out["gemm_rel"] < 1e-2 and out["norm_rel"] < 1e-2 and out["emb_exact"]
    assert out["status_clean"] == 0
    assert out["bad_row_zero"]
    assert out["status_bad"] == 6          # MM_ERR_BOUNDS
    assert out["status_after_clear"] == 0
