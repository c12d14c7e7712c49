"""The allocation-free RMSNorm backward, called through its exported C symbol, must give the
same gradients as the ordinary entry point - on two calls in a row, because both calls share
the scratch array that is built into the library and the second one sees the first one's
leftovers. (Callers that cannot allocate: code running inside a frozen memory pool, early
library initialisation, latency-critical loops; see csrc/kernels/no_alloc.h.)

This file sorts last on purpose: a run that stops at the first failure has then already
executed every other test."""
import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

from multimesh_jax_b200.ops import _lib
from multimesh_jax_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def _entry():
    lib = ctypes.CDLL(str(_lib.lib_path()))
    fn = lib.mm_rmsnorm_bwd_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_void_p]
    return fn


def _call(fn, x, w, dy, rstd):
    dx = torch.empty_like(x)
    dw = torch.empty(x.shape[-1], dtype=torch.float32, device=x.device)
    rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
            x.shape[0], x.shape[1], 0, 0, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return dx, dw


@pytest.mark.parametrize("rows,D", [(333, 4096), (50, 512)])
def test_no_alloc_matches_regular_entry_point_twice(rows, D):
    fn = _entry()
    for seed in (0, 1):  # two calls in a row share the built-in scratch
        torch.manual_seed(seed)
        x = torch.randn(rows, D, device="cuda").bfloat16()
        w = (torch.randn(D, device="cuda") * 0.5 + 1).bfloat16()
        dy = torch.randn(rows, D, device="cuda").bfloat16()
        _, rstd = K.rmsnorm_fwd(x, w, 1e-5)
        ref_dx, ref_dw = K.rmsnorm_bwd(x, w, dy, rstd)
        dx, dw = _call(fn, x, w, dy, rstd)
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), ref_dx.float(), rtol=2e-2, atol=2e-2 * ref_dx.float().abs().max().item())
        torch.testing.assert_close(dw, ref_dw, rtol=1e-2, atol=1e-2 * ref_dw.abs().max().item())


def test_no_alloc_rejects_oversized_hidden_dimension():
    fn = _entry()
    D = 16384
    x = torch.zeros(4, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.empty(D, device="cuda")
    rc = fn(x.data_ptr(), w.data_ptr(), x.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, D, 0, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc != 0
