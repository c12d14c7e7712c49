"""Functional layer over the CUDA kernel library.

Every function takes ``torch.Tensor`` arguments. CUDA tensors are handed to
the hand-written sm_100a kernels on the current stream; CPU tensors run an
equivalent PyTorch implementation so the framework can be exercised (and the
kernels' numerics checked) without a GPU. A CUDA tensor never falls back to a
PyTorch op silently: if the kernel library is missing, loading raises.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch

from . import _lib

bf16 = torch.bfloat16

# Number of kernel launches issued through this module (for benchmarks), and the number of
# calls that went to a vendor-library kernel instead of one of ours.
launch_count = 0
library_call_count = 0


def count_library_call(n: int = 1) -> None:
    global library_call_count
    library_call_count += n


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def read_status(clear: bool = True) -> int:
    """Device status word: 0 when no kernel has recorded a bounded-wait expiry."""
    return _lib.load().mm_read_status(1 if clear else 0)


STATUS_NAMES = {1: "a GEMM consumer gave up waiting for a TMA stage", 2: "a TMA producer gave up waiting for a free stage",
                3: "an epilogue gave up waiting for its accumulator", 4: "an MMA lane gave up waiting for a drained accumulator",
                5: "a wait for a peer GPU's flag ran out of time", 6: "a checked index was out of range",
                9: "a token overflowed the capacity of an expert's receive region"}


class StatusProbe:
    """Non-blocking view of one device's kernel status word.

    ``record()`` queues, on the current stream, a 4-byte copy of the word into pinned host
    memory followed by an event; ``poll()`` looks at the copies whose event has fired (all of
    them after a synchronisation when ``block``) and returns the first non-zero code it finds,
    clearing the device word so that the next step starts clean. The host thus learns of an
    expired bounded wait or a capacity overflow without ever stalling the stream."""

    SLOTS = 16

    def __init__(self, device: torch.device):
        from ..parallel.symm import tensor_from_ptr
        self.device = device
        with torch.cuda.device(device):
            ptr = _lib.load().mm_status_ptr()
        if not ptr:
            raise RuntimeError("the kernel library has no status block on this device")
        self.word = tensor_from_ptr(ptr, (1,), torch.int32, device)
        self.host = torch.zeros(self.SLOTS, dtype=torch.int32).pin_memory()
        self.events = [None] * self.SLOTS
        self.next = 0
        self._pending_code = 0

    def record(self) -> None:
        i = self.next % self.SLOTS
        if self.events[i] is not None and not self.events[i].query():
            self.events[i].synchronize()      # the ring is full: only then wait for the oldest copy
            self._take(i)
        self.host[i:i + 1].copy_(self.word, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.events[i] = ev
        self.next += 1

    def _take(self, i: int) -> None:
        code = int(self.host[i])
        self.events[i] = None
        if code and not self._pending_code:
            self._pending_code = code

    def poll(self, block: bool = False) -> int:
        if block:
            torch.cuda.synchronize(self.device)
        for i, ev in enumerate(self.events):
            if ev is not None and ev.query():
                self._take(i)
        code = self._pending_code
        if code:
            self._pending_code = 0
            with torch.cuda.device(self.device):
                read_status(clear=True)
        return code


# --------------------------------------------------------------------- GEMM
_OUT_MODE = {(bf16, False): 0, (torch.float32, False): 1, (torch.float32, True): 2, (bf16, True): 3}


# CTA-pair GEMM (tcgen05 cta_group::2, 256x256 tile per pair of SMs) for problems with at least
# this many rows: 9-11 % faster than the single-CTA kernel on 8192x4096x4096 in all three layouts.
# 0 switches it off. Environment: MM_GEMM_PAIR_MIN_M.
PAIR_MIN_M = int(os.environ.get("MM_GEMM_PAIR_MIN_M", "256"))


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         accumulate: bool = False, pair: Optional[bool] = None, m_dev: Optional[torch.Tensor] = None,
         k_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``C[M,N] (+)= A[M,K] @ B[N,K]^T`` with bf16 inputs and fp32 accumulation.

    ``a_mn`` / ``b_mn`` say that the operand is stored transposed (``[K, M]`` /
    ``[K, N]`` in memory, i.e. contiguous along M / N). Operands must be 2-D
    with unit stride in the last dimension. ``pair`` selects the CTA-pair kernel
    (None: by ``PAIR_MIN_M``).

    ``m_dev`` / ``k_dev``: one-element int32 device tensors with the number of rows / of
    contraction elements that actually hold data; the shapes of the operands are then upper
    bounds and the kernel reads the extents when it starts, so the host never needs to know
    them (rows of ``out`` beyond ``m_dev`` are left alone; with ``k_dev`` the operands' rows up
    to the next multiple of 64 must be zero, see :func:`zero_row_tail`).
    """
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    else:
        assert out.shape == (M, N) and out.stride(1) == 1
    if not a.is_cuda:
        af = (a.t() if a_mn else a).float()
        bf = (b.t() if b_mn else b).float()
        rows = min(M, max(0, int(m_dev[0]))) if m_dev is not None else M
        depth = min(K, max(0, int(k_dev[0]))) if k_dev is not None else K
        if depth == 0:
            return out
        res = af[:rows, :depth] @ bf[:, :depth].t()
        if accumulate:
            out[:rows].add_(res.to(out.dtype))
        else:
            out[:rows].copy_(res.to(out.dtype))
        return out
    assert a.dtype == bf16 and b.dtype == bf16
    mode = _OUT_MODE[(out.dtype, accumulate)]
    lib = _lib.load()
    if m_dev is not None or k_dev is not None:
        for t in (m_dev, k_dev):
            assert t is None or (t.dtype == torch.int32 and t.is_cuda and t.numel() >= 1)
        rc = lib.mm_gemm_pair_dyn_bf16(a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn), b.stride(0),
                                       out.data_ptr(), mode, out.stride(0), M, N, K,
                                       m_dev.data_ptr() if m_dev is not None else None,
                                       k_dev.data_ptr() if k_dev is not None else None, _stream())
        _lib.check(rc, "mm_gemm_pair_dyn_bf16")
        _count()
        return out
    if pair is None:
        pair = PAIR_MIN_M > 0 and M >= PAIR_MIN_M
    fn = lib.mm_gemm_pair_bf16 if pair else lib.mm_gemm_bf16
    rc = fn(a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn),
            b.stride(0), out.data_ptr(), mode, out.stride(0), M, N, K, _stream())
    _lib.check(rc, "mm_gemm_pair_bf16" if pair else "mm_gemm_bf16")
    _count()
    return out


def linear_fwd(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
               rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[T, N] = x[T, K] @ w[N, K]^T. ``rows``: device-side count of the rows of x that hold data."""
    return gemm(x, w, out=out, m_dev=rows)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dx[T, K] = dy[T, N] @ w[N, K]."""
    return gemm(dy, w, b_mn=True, out=out, accumulate=accumulate, m_dev=rows)


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                 accumulate: bool = False, out_dtype: Optional[torch.dtype] = None,
                 rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dw[N, K] (+)= dy[T, N]^T @ x[T, K]. With ``rows`` (device-side count of the rows that hold
    data) the tails of dy and x up to the next multiple of 64 rows must be zero, and a count of
    zero leaves ``out`` as it is."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=accumulate, out_dtype=out_dtype, k_dev=rows)


def zero_row_tail(x: torch.Tensor, rows: torch.Tensor, multiple: int = 64) -> None:
    """Zeroes rows [rows, round_up(rows, multiple)) of the 2-D tensor ``x`` (``rows``: int32 on the device)."""
    assert x.dim() == 2 and x.is_contiguous() and rows.dtype == torch.int32
    if not x.is_cuda:
        c = int(rows[0])
        x[c:min(x.shape[0], -(-c // multiple) * multiple)] = 0
        return
    rc = _lib.load().mm_zero_row_tail(x.data_ptr(), x.shape[1] * x.element_size(), rows.data_ptr(), multiple, x.shape[0],
                                      _stream())
    _lib.check(rc, "mm_zero_row_tail")
    _count()


# ------------------------------------------------------------------ RMSNorm
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    D = x.shape[-1]
    rows = x.numel() // D
    if not x.is_cuda:
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        y = (xf * rstd * w.float()).to(x.dtype)
        return y, rstd.reshape(rows)
    x = x.contiguous()
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    rc = _lib.load().mm_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, D,
                                    eps, _stream())
    _lib.check(rc, "mm_rmsnorm_fwd")
    _count()
    return y, rstd


_scratch = {}


def _get_scratch(device, nfloats: int) -> torch.Tensor:
    buf = _scratch.get(device)
    if buf is None or buf.numel() < nfloats:
        buf = torch.empty(max(nfloats, 1 << 20), dtype=torch.float32, device=device)
        _scratch[device] = buf
    return buf


def rmsnorm_bwd(x: torch.Tensor, w: torch.Tensor, dy: torch.Tensor, rstd: torch.Tensor,
                dw_out: Optional[torch.Tensor] = None, accumulate_dw: bool = False,
                dx_inout: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns (dx, dw). ``dw`` is fp32. With ``dx_inout`` the input gradient is
    added into that tensor (fusing the residual-stream add)."""
    D = x.shape[-1]
    rows = x.numel() // D
    if not x.is_cuda:
        xf, gf, wf = x.float().reshape(rows, D), dy.float().reshape(rows, D), w.float()
        r = rstd.reshape(rows, 1)
        gw = gf * wf
        dx = gw * r - xf * (r ** 3) * (gw * xf).sum(-1, keepdim=True) / D
        dw = (gf * xf * r).sum(0)
        if dx_inout is not None:
            dx_inout.add_(dx.reshape(x.shape).to(x.dtype))
            dx_t = dx_inout
        else:
            dx_t = dx.reshape(x.shape).to(x.dtype)
        if dw_out is None:
            dw_out = dw
        elif accumulate_dw:
            dw_out.add_(dw)
        else:
            dw_out.copy_(dw)
        return dx_t, dw_out
    lib = _lib.load()
    x = x.contiguous()
    dy = dy.contiguous()
    dx = dx_inout if dx_inout is not None else torch.empty_like(x)
    if dw_out is None:
        dw_out = torch.empty(D, dtype=torch.float32, device=x.device)
        accumulate_dw = False
    parts = lib.mm_rmsnorm_bwd_parts(rows)
    scratch = _get_scratch(x.device, parts * D)
    rc = lib.mm_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                            dw_out.data_ptr(), scratch.data_ptr(), rows, D, int(accumulate_dw),
                            int(dx_inout is not None), _stream())
    _lib.check(rc, "mm_rmsnorm_bwd")
    _count(2)
    return dx, dw_out


# --------------------------------------------------------------------- RoPE
def rope_tables(seq_len: int, head_dim: int, theta: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv)
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


def rope_(qk: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, backward: bool = False,
          rot_per_group: int = 1, group_size: int = 1) -> torch.Tensor:
    """In-place rotate-half RoPE on ``qk`` of shape [T, H, Dh] (token stride may exceed
    H*Dh, e.g. a slice of a fused QKV buffer). Position = t % S. With ``group_size`` > 1
    the H heads are packed in groups and only the first ``rot_per_group`` heads of every
    group are rotated (H counts all heads, rotated or not)."""
    T, H, Dh = qk.shape
    S = cos.shape[0]
    assert qk.stride(2) == 1 and qk.stride(1) == Dh
    assert H % group_size == 0
    n_rot = H // group_size * rot_per_group
    if not qk.is_cuda:
        pos = torch.arange(T) % S
        c = cos[pos].unsqueeze(1)
        s = sin[pos].unsqueeze(1) * (-1.0 if backward else 1.0)
        view = qk.view(T, H // group_size, group_size, Dh)[:, :, :rot_per_group]
        a, b = view[..., : Dh // 2].float(), view[..., Dh // 2:].float()
        c, s = c.unsqueeze(1), s.unsqueeze(1)
        lo, hi = a * c - b * s, b * c + a * s
        view[..., : Dh // 2] = lo.to(qk.dtype)
        view[..., Dh // 2:] = hi.to(qk.dtype)
        return qk
    rc = _lib.load().mm_rope(qk.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, S, n_rot, Dh, qk.stride(0),
                             int(backward), rot_per_group, group_size, _stream())
    _lib.check(rc, "mm_rope")
    _count()
    return qk


# ------------------------------------------------------------------- SwiGLU
def swiglu_fwd(gu: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h = silu(gate) * up. ``rows`` (one int32 on the device): only that many leading rows hold
    data; the others are skipped and their part of the result stays uninitialised."""
    T, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda:
        g, u = gu[:, :F].float(), gu[:, F:].float()
        return (torch.nn.functional.silu(g) * u).to(gu.dtype)
    h = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    rc = _lib.load().mm_swiglu_fwd_rows(gu.data_ptr(), h.data_ptr(), T, F, rows.data_ptr() if rows is not None else None,
                                        _stream())
    _lib.check(rc, "mm_swiglu_fwd")
    _count()
    return h


def swiglu_bwd(gu: torch.Tensor, dh: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, F2 = gu.shape
    F = F2 // 2
    if not gu.is_cuda:
        g, u, d = gu[:, :F].float(), gu[:, F:].float(), dh.float()
        sg = torch.sigmoid(g)
        dg = d * u * sg * (1 + g * (1 - sg))
        du = d * g * sg
        return torch.cat([dg, du], dim=1).to(gu.dtype)
    dgu = torch.empty_like(gu)
    rc = _lib.load().mm_swiglu_bwd_rows(gu.data_ptr(), dh.contiguous().data_ptr(), dgu.data_ptr(), T, F,
                                        rows.data_ptr() if rows is not None else None, _stream())
    _lib.check(rc, "mm_swiglu_bwd")
    _count()
    return dgu


# ------------------------------------------------------------ cross-entropy
def cross_entropy_fwd_bwd(logits: torch.Tensor, targets: torch.Tensor, grad_scale: float,
                          write_grad: bool = True) -> torch.Tensor:
    """Per-row loss (fp32). When ``write_grad`` the logits buffer is overwritten
    with d(loss_sum * grad_scale)/dlogits. Rows whose target is negative are skipped."""
    rows, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        valid = targets >= 0
        tsafe = targets.clamp(min=0)
        loss = torch.where(valid, lse - lf.gather(1, tsafe[:, None]).squeeze(1), torch.zeros_like(lse))
        if write_grad:
            g = torch.softmax(lf, dim=-1)
            g.scatter_add_(1, tsafe[:, None], -torch.ones(rows, 1))
            g = g * grad_scale * valid[:, None]
            logits.copy_(g.to(logits.dtype))
        return loss
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    rc = _lib.load().mm_cross_entropy(logits.data_ptr(), targets.data_ptr(), loss.data_ptr(), None, None,
                                      rows, V, logits.stride(0), 0, grad_scale, int(write_grad), _stream())
    _lib.check(rc, "mm_cross_entropy")
    _count()
    return loss


def cross_entropy_stats(logits: torch.Tensor, targets: torch.Tensor, vocab_start: int) -> torch.Tensor:
    """First pass of a vocabulary-sharded cross-entropy: per row (max, sum-exp relative to that
    max, logit of the target if it lies in this shard else 0) of this shard's logits [rows, V_local]."""
    rows, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        mx = lf.max(dim=-1).values
        se = torch.exp(lf - mx[:, None]).sum(-1)
        local = targets - vocab_start
        has = (targets >= 0) & (local >= 0) & (local < V)
        tl = torch.where(has, lf.gather(1, local.clamp(0, V - 1)[:, None]).squeeze(1), torch.zeros_like(mx))
        return torch.stack([mx, se, tl], dim=1)
    stats = torch.empty((rows, 3), dtype=torch.float32, device=logits.device)
    rc = _lib.load().mm_cross_entropy(logits.data_ptr(), targets.data_ptr(), None, stats.data_ptr(), None, rows, V,
                                      logits.stride(0), vocab_start, 0.0, 0, _stream())
    _lib.check(rc, "mm_cross_entropy")
    _count()
    return stats


def cross_entropy_combine(all_stats, targets: torch.Tensor, stat_ptrs=None):
    """Global (max, sum-exp) per row [rows, 2] and the loss per row from the shards' statistics.
    ``all_stats``: list of [rows, 3] tensors (CPU path), or with ``stat_ptrs`` the device
    addresses of the shards' arrays - this GPU's and its peers' - read by one kernel."""
    rows = targets.numel()
    if stat_ptrs is None:
        st = torch.stack(list(all_stats), dim=0)                       # [g, rows, 3]
        mx = st[..., 0].max(dim=0).values
        se = (st[..., 1] * torch.exp(st[..., 0] - mx)).sum(0)
        tl = st[..., 2].sum(0)
        loss = torch.where(targets >= 0, torch.log(se) + mx - tl, torch.zeros_like(mx))
        return torch.stack([mx, se], dim=1).contiguous(), loss
    import ctypes
    dev = targets.device
    stats2 = torch.empty((rows, 2), dtype=torch.float32, device=dev)
    loss = torch.empty(rows, dtype=torch.float32, device=dev)
    arr = (ctypes.c_int64 * len(stat_ptrs))(*stat_ptrs)
    rc = _lib.load().mm_ce_combine(arr, len(stat_ptrs), targets.data_ptr(), stats2.data_ptr(), loss.data_ptr(), rows,
                                   _stream())
    _lib.check(rc, "mm_ce_combine")
    _count()
    return stats2, loss


def cross_entropy_apply(logits: torch.Tensor, targets: torch.Tensor, stats2: torch.Tensor, vocab_start: int,
                        grad_scale: float) -> None:
    """Second pass: overwrites this shard's logits with d(loss * grad_scale)/dlogits given the
    global statistics."""
    rows, V = logits.shape
    if not logits.is_cuda:
        lf = logits.float()
        g = torch.exp(lf - stats2[:, :1]) / stats2[:, 1:2]
        local = targets - vocab_start
        has = (targets >= 0) & (local >= 0) & (local < V)
        g[has.nonzero().flatten(), local[has]] -= 1.0
        g = g * grad_scale * (targets >= 0)[:, None]
        logits.copy_(g.to(logits.dtype))
        return
    rc = _lib.load().mm_cross_entropy(logits.data_ptr(), targets.data_ptr(), None, None, stats2.data_ptr(), rows, V,
                                      logits.stride(0), vocab_start, grad_scale, 1, _stream())
    _lib.check(rc, "mm_cross_entropy")
    _count()


# ---------------------------------------------------------------- embedding
def embedding_fwd(table: torch.Tensor, ids: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    V, D = table.shape
    flat = ids.reshape(-1)
    if not table.is_cuda:
        local = flat - vocab_start
        ok = (local >= 0) & (local < V)
        out = table[local.clamp(0, V - 1)] * ok[:, None].to(table.dtype)
        return out
    out = torch.empty((flat.numel(), D), dtype=table.dtype, device=table.device)
    rc = _lib.load().mm_embedding_fwd(table.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.numel(), D,
                                      vocab_start, V, _stream())
    _lib.check(rc, "mm_embedding_fwd")
    _count()
    return out


def embedding_bwd(dout: torch.Tensor, ids: torch.Tensor, grad: torch.Tensor, vocab_start: int = 0) -> torch.Tensor:
    """grad[V, D] (fp32) += scatter-add of dout rows."""
    V, D = grad.shape
    flat = ids.reshape(-1)
    if not dout.is_cuda:
        local = flat - vocab_start
        ok = (local >= 0) & (local < V)
        grad.index_add_(0, local[ok], dout.reshape(-1, D)[ok].to(grad.dtype))
        return grad
    rc = _lib.load().mm_embedding_bwd(dout.contiguous().data_ptr(), flat.data_ptr(), grad.data_ptr(),
                                      flat.numel(), D, vocab_start, V, _stream())
    _lib.check(rc, "mm_embedding_bwd")
    _count()
    return grad


# -------------------------------------------------------------- misc adds
def add_(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a += b for contiguous bf16 tensors."""
    if not a.is_cuda or a.numel() % 8 or a.dtype != bf16 or not (a.is_contiguous() and b.is_contiguous()):
        return a.add_(b)
    rc = _lib.load().mm_add_bf16(a.data_ptr(), b.data_ptr(), a.data_ptr(), a.numel(), _stream())
    _lib.check(rc, "mm_add_bf16")
    _count()
    return a


def add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if not a.is_cuda or a.numel() % 8 or a.dtype != bf16 or not (a.is_contiguous() and b.is_contiguous()):
        return a + b
    out = torch.empty_like(a)
    rc = _lib.load().mm_add_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), _stream())
    _lib.check(rc, "mm_add_bf16")
    _count()
    return out


def accumulate_(acc: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """acc(fp32) += src(bf16)."""
    if not acc.is_cuda or acc.numel() % 8 or src.dtype != bf16 or acc.dtype != torch.float32:
        return acc.add_(src.to(acc.dtype))
    rc = _lib.load().mm_accumulate_f32_bf16(acc.data_ptr(), src.contiguous().data_ptr(), acc.numel(), _stream())
    _lib.check(rc, "mm_accumulate_f32_bf16")
    _count()
    return acc


# --------------------------------------------------------------------- AdamW
def adamw_step_(master: torch.Tensor, param: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
                grad: torch.Tensor, *, lr: float, beta1: float, beta2: float, eps: float,
                weight_decay: float, step, grad_scale: float = 1.0) -> None:
    """Fused AdamW on flat buffers (fp32 master/m/v/grad, bf16 working copy).
    ``step`` is an int, or a 1-element int64 tensor on the same device (read by the
    kernel, so no host synchronisation)."""
    n = master.numel()
    step_t = step if isinstance(step, torch.Tensor) else None
    if not master.is_cuda:
        step = int(step)
        g = grad * grad_scale
        m.mul_(beta1).add_(g, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        mh = m / (1 - beta1 ** step)
        vh = v / (1 - beta2 ** step)
        master.mul_(1 - lr * weight_decay).addcdiv_(mh, vh.sqrt() + eps, value=-lr)
        param.copy_(master.to(param.dtype))
        return
    assert n % 4 == 0
    rc = _lib.load().mm_adamw(master.data_ptr(), param.data_ptr(), m.data_ptr(), v.data_ptr(),
                              grad.data_ptr(), n, lr, beta1, beta2, eps, weight_decay,
                              1 if step_t is not None else int(step), grad_scale,
                              step_t.data_ptr() if step_t is not None else None, _stream())
    _lib.check(rc, "mm_adamw")
    _count()


def sumsq(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[0] += sum(x*x) for an fp32 buffer (gradient-norm clipping)."""
    if not x.is_cuda:
        out[0] += (x.double() ** 2).sum().float()
        return out
    rc = _lib.load().mm_sumsq_f32(x.data_ptr(), x.numel(), out.data_ptr(), _stream())
    _lib.check(rc, "mm_sumsq_f32")
    _count()
    return out


# ---------------------------------------------------------------- attention
def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """fp32 reference: q [B,S,Hq,D], k/v [B,S,Hkv,D] -> [B,S,Hq,D]."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ vf
    return o.permute(0, 2, 1, 3).contiguous()
