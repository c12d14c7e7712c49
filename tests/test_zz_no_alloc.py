"""The allocation-free RMSNorm backward, called through its exported C symbol, must give the
same gradients as the ordinary entry point and as PyTorch's fp32 autograd - on two calls in a
row, because both calls share the scratch array that is built into the library and the second
one sees the first one's leftovers. (Callers that cannot allocate: code running inside a frozen
memory pool, early library initialisation, latency-critical loops; see csrc/kernels/no_alloc.h.)

This file sorts last on purpose: a run that stops at the first failure has then already
executed every other test."""
import ctypes
from ctypes import c_int, c_int64, c_void_p

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


def _call(fn, x, w, dy, rstd, dx=None, dw=None):
    add_to_dx, accumulate_dw = int(dx is not None), int(dw is not None)
    dx = torch.empty_like(x) if dx is None else dx
    dw = torch.empty(x.shape[-1], dtype=torch.float32, device=x.device) if dw is None else dw
    rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(),
            x.shape[0], x.shape[1], accumulate_dw, add_to_dx, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    return dx, dw


def _autograd_reference(x, w, dy, eps):
    """RMSNorm gradients by PyTorch autograd in fp32 (from the same bf16-rounded inputs)."""
    xf = x.float().requires_grad_(True)
    wf = w.float().requires_grad_(True)
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * wf
    y.backward(dy.float())
    return xf.grad, wf.grad


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


# one case per kernel instantiation of the entry point: D <= 1024, <= 2048, <= 4096, <= 8192
@pytest.mark.parametrize("rows,D", [(50, 512), (129, 2048), (333, 4096), (200, 8192)])
def test_no_alloc_matches_regular_entry_point_and_autograd_twice(rows, D):
    fn = _entry()
    eps = 1e-5
    for seed in (0, 1):  # two calls in a row share the built-in scratch
        torch.manual_seed(seed)
        x = torch.randn(rows, D, device="cuda").bfloat16()
        w = (torch.randn(D, device="cuda") * 0.5 + 1).bfloat16()
        dy = torch.randn(rows, D, device="cuda").bfloat16()
        _, rstd = K.rmsnorm_fwd(x, w, eps)
        ref_dx, ref_dw = K.rmsnorm_bwd(x, w, dy, rstd)
        dx, dw = _call(fn, x, w, dy, rstd)
        torch.cuda.synchronize()
        # against the ordinary entry point (same arithmetic, other block shapes)
        torch.testing.assert_close(dx.float(), ref_dx.float(), rtol=2e-2, atol=2e-2 * ref_dx.float().abs().max().item())
        torch.testing.assert_close(dw, ref_dw, rtol=1e-2, atol=1e-2 * ref_dw.abs().max().item())
        # against fp32 autograd: dx is rounded to bf16 once, dw stays fp32
        ag_dx, ag_dw = _autograd_reference(x, w, dy, eps)
        assert _rel(dx, ag_dx) < 1e-2, (rows, D, seed, _rel(dx, ag_dx))
        assert _rel(dw, ag_dw) < 1e-3, (rows, D, seed, _rel(dw, ag_dw))


@pytest.mark.parametrize("rows,D", [(77, 1024), (260, 4096)])
def test_no_alloc_accumulates_into_existing_gradients_twice(rows, D):
    """``accumulate_dw`` adds the weight gradient to what ``dw_out`` holds and ``add_to_dx`` adds
    the input gradient into ``dx`` (the residual-stream add of a transformer block)."""
    fn = _entry()
    eps = 1e-5
    for seed in (2, 3):
        torch.manual_seed(seed)
        x = torch.randn(rows, D, device="cuda").bfloat16()
        w = (torch.randn(D, device="cuda") * 0.5 + 1).bfloat16()
        dy = torch.randn(rows, D, device="cuda").bfloat16()
        dx0 = torch.randn(rows, D, device="cuda").bfloat16()
        dw0 = torch.randn(D, device="cuda")
        _, rstd = K.rmsnorm_fwd(x, w, eps)
        dx, dw = _call(fn, x, w, dy, rstd, dx=dx0.clone(), dw=dw0.clone())
        torch.cuda.synchronize()
        ag_dx, ag_dw = _autograd_reference(x, w, dy, eps)
        assert _rel(dx, dx0.float() + ag_dx) < 1e-2
        assert _rel(dw, dw0 + ag_dw) < 1e-3
        # and the ordinary entry point agrees on the same request
        ref_dx, ref_dw = K.rmsnorm_bwd(x, w, dy, rstd, dw_out=dw0.clone(), accumulate_dw=True, dx_inout=dx0.clone())
        torch.cuda.synchronize()
        torch.testing.assert_close(dx.float(), ref_dx.float(), rtol=2e-2, atol=2e-2 * ref_dx.float().abs().max().item())
        torch.testing.assert_close(dw, ref_dw, rtol=1e-2, atol=1e-2 * ref_dw.abs().max().item())


def test_no_alloc_rejects_sizes_beyond_its_limits():
    fn = _entry()
    D = 16384
    x = torch.zeros(4, D, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dx = torch.empty_like(x)
    dw = torch.empty(D, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # hidden size beyond the built-in scratch
    assert fn(x.data_ptr(), w.data_ptr(), x.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, D, 0, 0,
              stream) != 0
    # hidden size that is not a multiple of 8, and a row count beyond the kernel's index range:
    # both are refused before anything is launched
    assert fn(x.data_ptr(), w.data_ptr(), x.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, 1020, 0, 0,
              stream) != 0
    assert fn(x.data_ptr(), w.data_ptr(), x.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 1 << 31, 1024,
              0, 0, stream) != 0
    torch.cuda.synchronize()
