"""Sparse mixture-of-experts feed-forward layer (top-k softmax router, SwiGLU experts) with
expert parallelism.

The reference has no MoE or expert-parallel path (its only trace of all-to-all is an opcode
listed in ``src/pjrt_client/mm_computation.cc:379``); this layer exists because the
Mixtral-shaped benchmark configuration needs it.

Global view (what the captured graph contains)::

    y = moe_ffn(x[..., D], w_router[E, D], w_gu[E, 2, F, D], w_down[E, D, F], top_k)

Every token picks its ``top_k`` experts by router logit, the selected logits are soft-maxed into
gates, and ``y = sum_k gate_k * down_e(silu(gate_e(x)) * up_e(x))``. The backward pass is one
operator, ``moe_ffn_bwd``, that recomputes the routing and the expert activations.

Expert parallelism: the shard rule lets the *token* dimensions and the *expert* dimension use
the same mesh axis (``shares_axes``). A task whose experts are sharded runs the local forms
(:func:`moe_ffn_local`, :func:`moe_ffn_bwd_local`): route local tokens, send every (token, k)
row to the device that owns the expert (dispatch all-to-all), run the local experts on what
arrived, send results back (combine all-to-all) and reduce them with the gates. On CUDA the
expert projections run on the tcgen05 GEMM kernels; dispatch and combine go through
:meth:`DeviceCtx.all_to_all`.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import kernels as K
from .mm_ops import _cls, _define, register_shard_rule


# --------------------------------------------------------------------------- routing
def route(x2: torch.Tensor, wr: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Router logits (fp32), chosen experts [T, k] and gates [T, k] (softmax over the chosen logits)."""
    logits = x2.float() @ wr.float().t()
    topv, topi = logits.topk(top_k, dim=-1)
    gates = torch.softmax(topv, dim=-1)
    return logits, topi, gates


def select_experts(logits: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """The selection rule of ``moe_route_dispatch_kernel`` restated on tensors: per choice the
    largest logit not taken yet, ties to the lowest index; when no remaining logit compares
    greater than -inf (all NaN or -inf) the lowest free index with a neutral logit of 0. The
    result is always ``top_k`` distinct experts in ``[0, E)`` - the kernel stores rows into the
    owner's memory at offsets derived from them. Returns (experts [T, k], chosen logits [T, k])."""
    T, E = logits.shape
    work = logits.float().clone()
    work[torch.isnan(work)] = float("-inf")
    idx = torch.empty(T, top_k, dtype=torch.int64)
    val = torch.empty(T, top_k, dtype=torch.float32)
    taken = torch.zeros(T, E, dtype=torch.bool)
    for j in range(top_k):
        masked = torch.where(taken, torch.full_like(work, float("-inf")), work)
        best_v, best_i = masked.max(dim=-1)                    # max returns the first maximal index
        none = ~(best_v > float("-inf"))
        first_free = (~taken).float().argmax(dim=-1)
        best_i = torch.where(none, first_free, best_i)
        best_v = torch.where(none, torch.zeros_like(best_v), best_v)
        idx[:, j], val[:, j] = best_i, best_v
        taken[torch.arange(T), best_i] = True
    return idx, val


def _expert_fwd(rows: torch.Tensor, wgu_e: torch.Tensor, wdown_e: torch.Tensor, out=None, count=None):
    """rows [M, D] -> (gu [M, 2F] (gate | up), h [M, F], out [M, D]); ``out`` may be preallocated.
    ``count`` (one int32 on the device): only that many leading rows hold tokens - M is then the
    capacity of the expert's receive region; the GEMMs and the SwiGLU kernel read the count on
    the device and skip the rest (rows beyond the count hold whatever the buffers held before
    and are never read back)."""
    F = wgu_e.shape[1]
    gu = K.linear_fwd(rows, wgu_e.reshape(2 * F, -1), rows=count)
    h = K.swiglu_fwd(gu, rows=count)
    out = K.linear_fwd(h, wdown_e, out=out, rows=count)
    return gu, h, out


def _expert_bwd(rows, d_out, wgu_e, wdown_e, dx_out=None, out=None, count=None, dwgu_out=None, dwdown_out=None):
    """Gradients of one expert for the rows routed to it. Returns (dx_rows, dwgu_e, dwdown_e, out).
    With ``count`` (see :func:`_expert_fwd`) the weight gradients are written into the
    preallocated, zero-initialised ``dwgu_out`` [2, F, D] / ``dwdown_out`` [D, F] (fp32); an
    expert that received nothing leaves them zero."""
    F = wgu_e.shape[1]
    gu, h, out = _expert_fwd(rows, wgu_e, wdown_e, out=out, count=count)
    if count is None:
        dwdown = K.linear_wgrad(d_out, h, out_dtype=torch.float32)              # [D, F]
        dh = K.linear_dgrad(d_out, wdown_e)                                      # [M, F]
        dgu2 = K.swiglu_bwd(gu, dh)                                              # [M, 2F]
        dwgu = K.linear_wgrad(dgu2, rows, out_dtype=torch.float32).view(2, F, -1)
        dx = K.linear_dgrad(dgu2, wgu_e.reshape(2 * F, -1), out=dx_out)
        return dx, dwgu, dwdown, out
    # the contraction of a weight gradient runs over the rows: its last 64-row block must not
    # pick up what lies behind the count
    for t in (d_out, h, rows):
        K.zero_row_tail(t, count)
    dwdown = K.linear_wgrad(d_out, h, out=dwdown_out, rows=count)
    dh = K.linear_dgrad(d_out, wdown_e, rows=count)
    dgu2 = K.swiglu_bwd(gu, dh, rows=count)
    K.zero_row_tail(dgu2, count)
    dwgu = K.linear_wgrad(dgu2, rows, out=dwgu_out.view(2 * F, -1), rows=count).view(2, F, -1)
    dx = K.linear_dgrad(dgu2, wgu_e.reshape(2 * F, -1), out=dx_out, rows=count)
    return dx, dwgu, dwdown, out


# --------------------------------------------------------------------------- global view
def moe_ffn_impl(x, wr, wgu, wdown, top_k: int):
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    _, topi, gates = route(x2, wr, top_k)
    y = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
    for e in range(wgu.shape[0]):
        hit = topi == e
        tok = hit.any(-1).nonzero().flatten()
        if tok.numel() == 0:
            continue
        _, _, out = _expert_fwd(x2[tok].contiguous(), wgu[e], wdown[e])
        g = (gates * hit)[tok].sum(-1, keepdim=True)
        y.index_add_(0, tok, g * out.float())
    return y.to(x.dtype).view(x.shape)


def moe_ffn_bwd_impl(dy, x, wr, wgu, wdown, top_k: int):
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    _, topi, gates = route(x2, wr, top_k)
    dx = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
    dgates = torch.zeros_like(gates)
    dwgu = torch.zeros(wgu.shape, dtype=torch.float32, device=x.device)
    dwdown = torch.zeros(wdown.shape, dtype=torch.float32, device=x.device)
    for e in range(wgu.shape[0]):
        hit = topi == e
        tok, kpos = hit.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        g = gates[tok, kpos].unsqueeze(-1)
        rows, dyr = x2[tok].contiguous(), dy2[tok]
        d_out = (g * dyr.float()).to(x.dtype)
        dxr, dwgu_e, dwdown_e, out = _expert_bwd(rows, d_out, wgu[e], wdown[e])
        dx.index_add_(0, tok, dxr.float())
        dwgu[e] += dwgu_e
        dwdown[e] += dwdown_e
        dgates[tok, kpos] = (dyr.float() * out.float()).sum(-1)
    dx_r, dwr = _router_bwd(x2, wr, topi, gates, dgates)
    dx += dx_r
    return dx.to(x.dtype).view(x.shape), dwr.to(wr.dtype), dwgu.to(wgu.dtype), dwdown.to(wdown.dtype)


def _router_bwd(x2, wr, topi, gates, dgates):
    """Through the softmax over the chosen logits back to the router weights and the tokens."""
    dtopv = gates * (dgates - (gates * dgates).sum(-1, keepdim=True))
    dlogits = torch.zeros(x2.shape[0], wr.shape[0], dtype=torch.float32, device=x2.device)
    dlogits.scatter_(1, topi, dtopv)
    dwr = dlogits.t() @ x2.float()
    dx = dlogits @ wr.float()
    return dx, dwr


def _moe_backward(ctx, gy):
    x, wr, wgu, wdown = ctx.saved_tensors
    dx, dwr, dwgu, dwdown = torch.ops.mm_ops.moe_ffn_bwd(gy, x, wr, wgu, wdown, ctx.top_k)
    return dx, dwr, dwgu, dwdown, None


def _moe_setup(ctx, inputs, output):
    x, wr, wgu, wdown, top_k = inputs
    ctx.top_k = top_k
    ctx.save_for_backward(x, wr, wgu, wdown)


_define("moe_ffn(Tensor x, Tensor wr, Tensor wgu, Tensor wdown, int top_k) -> Tensor", moe_ffn_impl,
        lambda x, wr, wgu, wdown, top_k: torch.empty_like(x), backward=_moe_backward, setup=_moe_setup)
_define("moe_ffn_bwd(Tensor dy, Tensor x, Tensor wr, Tensor wgu, Tensor wdown, int top_k)"
        " -> (Tensor, Tensor, Tensor, Tensor)", moe_ffn_bwd_impl,
        lambda dy, x, wr, wgu, wdown, top_k: (torch.empty_like(x), torch.empty_like(wr), torch.empty_like(wgu),
                                              torch.empty_like(wdown)))


def moe_ffn(x, wr, wgu, wdown, top_k: int = 2):
    return torch.ops.mm_ops.moe_ffn(x, wr, wgu, wdown, top_k)


@register_shard_rule("mm_ops.moe_ffn.default")
def _rule_moe(node, ins, outs):
    # slots: 0 x, 1 wr, 2 wgu, 3 wdown | 4 y
    r = len(ins[0])
    classes = [_cls([(0, d), (4, d)]) for d in range(r - 1)]                     # tokens
    classes.append(_cls([(0, r - 1), (4, r - 1)], no_shard=True))               # model dimension
    experts = _cls([(2, 0), (3, 0)])
    experts["shares_axes"] = True
    classes.append(experts)
    classes.append(_cls([(1, 0)], no_shard=True))                               # router sees every expert
    return {"classes": classes}


@register_shard_rule("mm_ops.moe_ffn_bwd.default")
def _rule_moe_bwd(node, ins, outs):
    # slots: 0 dy, 1 x, 2 wr, 3 wgu, 4 wdown | 5 dx, 6 dwr, 7 dwgu, 8 dwdown
    r = len(ins[0])
    classes = [_cls([(0, d), (1, d), (5, d)], reduced=[1]) for d in range(r - 1)]   # dwr sums over tokens
    classes.append(_cls([(0, r - 1), (1, r - 1), (5, r - 1)], no_shard=True))
    experts = _cls([(3, 0), (4, 0), (7, 0), (8, 0)])
    experts["shares_axes"] = True
    classes.append(experts)
    classes.append(_cls([(2, 0), (6, 0)], no_shard=True))
    return {"classes": classes}


# --------------------------------------------------------------------------- expert parallel
def _plan_dispatch(topi: torch.Tensor, n: int, experts_per_rank: int):
    """For every destination rank: the (token, k) pairs it serves, as flat indices into [T*k]."""
    flat_e = topi.reshape(-1)
    dest = torch.div(flat_e, experts_per_rank, rounding_mode="floor")
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=n).tolist()
    return flat_e, order, counts


def _peer_moe(ctx, group, x2, n_experts: int):
    """The peer-memory implementation for this group, when the job has one (one process per
    GPU, bf16, a symmetric arena) - otherwise ``None`` and the all-to-all form runs."""
    reg = getattr(ctx, "peer_moe", None)
    if reg is None or not x2.is_cuda or x2.dtype != torch.bfloat16 or x2.shape[1] % 8:
        return None
    ranks = tuple(ctx.device_start + o for o in group)
    return reg.get(ranks, x2.shape[0], x2.shape[1], n_experts)


def moe_ffn_local(ctx, axes, key, x, wr, wgu, wdown, top_k: int):
    """This device's share of ``moe_ffn``: ``x`` holds its tokens, ``wgu`` / ``wdown`` its experts."""
    group, me = ctx.group_of(axes)
    n = len(group)
    if n == 1:
        return moe_ffn_impl(x, wr, wgu, wdown, top_k)
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    E_l = wgu.shape[0]
    peer = _peer_moe(ctx, group, x2, E_l * n)
    if peer is not None:
        return peer.forward(x2, wr, wgu, wdown, top_k).view(x.shape)
    _, topi, gates = route(x2, wr, top_k)
    flat_e, order, counts = _plan_dispatch(topi, n, E_l)
    tok = torch.div(order, top_k, rounding_mode="floor")
    rows_sorted = x2[tok]                                   # [T*k, D] grouped by destination
    eid_sorted = (flat_e[order] % E_l).to(torch.int32)
    recv_rows, recv_counts = ctx.all_to_all((key, "rows"), group, rows_sorted, counts)
    recv_eid, _ = ctx.all_to_all((key, "eid"), group, eid_sorted, counts)
    out_rows = torch.empty_like(recv_rows)
    for e in range(E_l):
        sel = (recv_eid == e).nonzero().flatten()
        if sel.numel():
            out_rows[sel] = _expert_fwd(recv_rows[sel].contiguous(), wgu[e], wdown[e])[2]
    back, _ = ctx.all_to_all((key, "back"), group, out_rows, recv_counts)   # same order as rows_sorted
    g = gates.reshape(-1)[order].unsqueeze(-1)
    y = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
    y.index_add_(0, tok, g * back.float())
    return y.to(x.dtype).view(x.shape)


def moe_ffn_bwd_local(ctx, axes, key, dy, x, wr, wgu, wdown, top_k: int):
    group, me = ctx.group_of(axes)
    n = len(group)
    if n == 1:
        return moe_ffn_bwd_impl(dy, x, wr, wgu, wdown, top_k)
    D = x.shape[-1]
    x2, dy2 = x.reshape(-1, D), dy.reshape(-1, D)
    E_l = wgu.shape[0]
    peer = _peer_moe(ctx, group, x2, E_l * n)
    if peer is not None:
        dx, dwr, dwgu, dwdown = peer.backward(dy2, x2, wr, wgu, wdown, top_k)
        return dx.view(x.shape), dwr, dwgu, dwdown
    _, topi, gates = route(x2, wr, top_k)
    flat_e, order, counts = _plan_dispatch(topi, n, E_l)
    tok = torch.div(order, top_k, rounding_mode="floor")
    g_sorted = gates.reshape(-1)[order].unsqueeze(-1)
    rows_sorted = x2[tok]
    dyr_sorted = dy2[tok]
    d_out_sorted = (g_sorted * dyr_sorted.float()).to(x.dtype)
    eid_sorted = (flat_e[order] % E_l).to(torch.int32)
    recv_rows, recv_counts = ctx.all_to_all((key, "rows"), group, rows_sorted, counts)
    recv_dout, _ = ctx.all_to_all((key, "dout"), group, d_out_sorted, counts)
    recv_eid, _ = ctx.all_to_all((key, "eid"), group, eid_sorted, counts)
    dx_rows = torch.empty_like(recv_rows)
    out_rows = torch.empty_like(recv_rows)
    dwgu = torch.zeros(wgu.shape, dtype=torch.float32, device=x.device)
    dwdown = torch.zeros(wdown.shape, dtype=torch.float32, device=x.device)
    for e in range(E_l):
        sel = (recv_eid == e).nonzero().flatten()
        if sel.numel() == 0:
            continue
        dxr, dwgu_e, dwdown_e, out = _expert_bwd(recv_rows[sel].contiguous(), recv_dout[sel].contiguous(), wgu[e], wdown[e])
        dx_rows[sel] = dxr
        out_rows[sel] = out
        dwgu[e] = dwgu_e
        dwdown[e] = dwdown_e
    back_dx, _ = ctx.all_to_all((key, "dx"), group, dx_rows, recv_counts)
    back_out, _ = ctx.all_to_all((key, "out"), group, out_rows, recv_counts)
    dx = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
    dx.index_add_(0, tok, back_dx.float())
    dgates = torch.zeros_like(gates).reshape(-1)
    dgates[order] = (dyr_sorted.float() * back_out.float()).sum(-1)
    dx_r, dwr = _router_bwd(x2, wr, topi, gates, dgates.view_as(gates))
    dx += dx_r
    return dx.to(x.dtype).view(x.shape), dwr.to(wr.dtype), dwgu.to(wgu.dtype), dwdown.to(wdown.dtype)


# operators whose per-device form talks to the other devices of the task: name -> (function,
# index of the tensor argument whose leading dimension tells over which mesh axes)
from .mm_ops import CTX_OPS  # noqa: E402  (the registry lives with the operator definitions)

CTX_OPS.update({
    "mm_ops.moe_ffn.default": (moe_ffn_local, 2),
    "mm_ops.moe_ffn_bwd.default": (moe_ffn_bwd_local, 3),
})
