"""Causal self-attention forward / backward on strided [B, S, H, D] views.

``q`` has ``hq`` heads, ``k`` / ``v`` have ``hkv`` heads (``hq % hkv == 0``, grouped-query
attention); all are views into one packed projection buffer, so only the last dimension
is contiguous. The softmax scale is ``1/sqrt(D)``.

The packed entry points (``attention_fwd_packed`` / ``attention_bwd_packed``) run the
tcgen05 flash-attention kernels of ``_mm_kernels.so`` (``mm_flash_attn_fwd`` /
``mm_flash_attn_bwd``) for bf16 CUDA tensors with head dimension 128 and a sequence length
that is a multiple of 128. Other CUDA shapes fall back to the fused scaled-dot-product
kernels that ship with PyTorch (a library path, counted as such in the benchmarks). CPU
tensors use an fp32 restatement.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Tuple

import torch

from . import _lib
from . import kernels as K

_aten = torch.ops.aten


def have_native_kernels() -> bool:
    try:
        lib = _lib.load()
    except RuntimeError:
        return False
    return hasattr(lib, "mm_flash_attn_fwd") and hasattr(lib, "mm_flash_attn_bwd")


_lib.register("mm_flash_attn_supported", ctypes.c_int, [ctypes.c_int, ctypes.c_int])
_lib.register("mm_flash_attn_fwd", ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                                  ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p])
_lib.register("mm_flash_attn_bwd", ctypes.c_int, [ctypes.c_void_p] * 7 + [ctypes.c_int] * 5 + [ctypes.c_void_p])


def native_supported(qkv: torch.Tensor) -> bool:
    """True when the packed projection can go through the tcgen05 attention kernels: CUDA,
    bf16, contiguous, head dimension 128, sequence length a multiple of 128."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and qkv.dim() == 4):
        return False
    if os.environ.get("MM_NATIVE_ATTENTION", "1") == "0":
        return False
    return bool(_lib.load().mm_flash_attn_supported(qkv.shape[1], qkv.shape[3]))


def _split_packed(qkv, rep: int):
    B, S, H, D = qkv.shape
    g = qkv.view(B, S, H // (rep + 2), rep + 2, D)
    return g[:, :, :, :rep], g[:, :, :, rep], g[:, :, :, rep + 1]


def attention_fwd_packed(qkv: torch.Tensor, rep: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Causal attention over a packed group-major projection [B,S,hkv*(rep+2),D] (rotary
    embedding already applied). Returns (out [B,S,hq,D], lse [B,hq,S] fp32)."""
    if not native_supported(qkv):
        return attention_fwd(*_split_packed(qkv, rep))
    B, S, H, D = qkv.shape
    hkv = H // (rep + 2)
    out = torch.empty((B, S, hkv * rep, D), dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty((B, hkv * rep, S), dtype=torch.float32, device=qkv.device)
    rc = _lib.load().mm_flash_attn_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, S, hkv, rep, D,
                                       torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "mm_flash_attn_fwd")
    K._count()
    return out, lse


def attention_bwd_packed(dout: torch.Tensor, qkv: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                         rep: int) -> torch.Tensor:
    """Gradient of :func:`attention_fwd_packed` with respect to the packed projection."""
    dqkv = torch.empty_like(qkv)
    if not (native_supported(qkv) and dout.dtype == torch.bfloat16):
        q, k, v = _split_packed(qkv, rep)
        dq, dk, dv = _split_packed(dqkv, rep)
        attention_bwd(dout, q, k, v, out, lse, dq, dk, dv)
        return dqkv
    B, S, H, D = qkv.shape
    hkv = H // (rep + 2)
    hq = hkv * rep
    dout = dout.contiguous()
    out = out.contiguous()
    dq_acc = torch.empty((B, S, hq, D), dtype=torch.float32, device=qkv.device)
    delta = torch.empty((B, hq, S), dtype=torch.float32, device=qkv.device)
    rc = _lib.load().mm_flash_attn_bwd(qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), dqkv.data_ptr(),
                                       dq_acc.data_ptr(), delta.data_ptr(), B, S, hkv, rep, D,
                                       torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "mm_flash_attn_bwd")
    K._count(4)
    return dqkv


def _merge_q(q):
    """[B,S,hkv,rep,D] -> [B,S,hq,D] (a view for rep == 1, otherwise a copy)."""
    B, S, Hkv, rep, D = q.shape
    return q.squeeze(3) if rep == 1 else q.reshape(B, S, Hkv * rep, D)


def _ref_fwd(q, k, v):
    q = _merge_q(q)
    B, S, Hq, D = q.shape
    rep = Hq // k.shape[2]
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = (p @ vf).permute(0, 2, 1, 3).contiguous()
    return o.to(q.dtype), lse, (qf, kf, vf, p)


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,S,hkv,rep,D], k/v [B,S,hkv,D] (strided views). Returns (out [B,S,hq,D]
    contiguous with hq = hkv*rep in group-major order, lse [B,hq,S] fp32)."""
    if not q.is_cuda:
        o, lse, _ = _ref_fwd(q, k, v)
        return o, lse
    q = _merge_q(q)
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if rep > 1:
        kt = kt.repeat_interleave(rep, dim=1)
        vt = vt.repeat_interleave(rep, dim=1)
    K.count_library_call()
    out, lse, _, _, _, _, _, _, _ = _aten._scaled_dot_product_flash_attention(
        qt, kt, vt, 0.0, True, False, scale=1.0 / math.sqrt(D))
    return out.transpose(1, 2).contiguous(), lse


def attention_bwd(dout, q, k, v, out, lse, dq, dk, dv) -> None:
    """Writes the gradients into the (strided) views ``dq`` [B,S,hkv,rep,D], ``dk``, ``dv``."""
    B, S, Hkv, rep, D = q.shape
    Hq = Hkv * rep
    dq5 = dq
    if not q.is_cuda:
        _, _, (qf, kf, vf, p) = _ref_fwd(q, k, v)
        dof = dout.float().permute(0, 2, 1, 3)
        dvf = p.transpose(-1, -2) @ dof
        dp = dof @ vf.transpose(-1, -2)
        delta = (dof * out.float().permute(0, 2, 1, 3)).sum(-1, keepdim=True)
        ds = p * (dp - delta) / math.sqrt(D)
        dqf = ds @ kf
        dkf = ds.transpose(-1, -2) @ qf
        dq5.copy_(dqf.permute(0, 2, 1, 3).reshape(B, S, Hkv, rep, D).to(dq.dtype))
        dk.copy_(dkf.view(B, Hkv, rep, S, D).sum(2).permute(0, 2, 1, 3).to(dk.dtype))
        dv.copy_(dvf.view(B, Hkv, rep, S, D).sum(2).permute(0, 2, 1, 3).to(dv.dtype))
        return
    qt, kt, vt = _merge_q(q).transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if rep > 1:
        kt = kt.repeat_interleave(rep, dim=1)
        vt = vt.repeat_interleave(rep, dim=1)
    ot, dot = out.transpose(1, 2), dout.transpose(1, 2)
    K.count_library_call()
    zero = torch.zeros((), dtype=torch.int64, device=q.device)
    gq, gk, gv = _aten._scaled_dot_product_flash_attention_backward(
        dot, qt, kt, vt, ot, lse, None, None, S, S, 0.0, True, zero, zero, scale=1.0 / math.sqrt(D))
    dq5.copy_(gq.transpose(1, 2).reshape(B, S, Hkv, rep, D))
    if rep > 1:
        gk = gk.view(B, Hkv, rep, S, D).sum(2)
        gv = gv.view(B, Hkv, rep, S, D).sum(2)
    dk.copy_(gk.transpose(1, 2))
    dv.copy_(gv.transpose(1, 2))
