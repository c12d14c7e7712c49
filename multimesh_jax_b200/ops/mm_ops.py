"""``torch.library`` operators over the hand-written kernels (namespace ``mm_ops``).

Each operator
* has a functional implementation (CUDA tensors -> our sm_100a kernels, CPU
  tensors -> the PyTorch restatement in :mod:`.kernels`),
* a fake implementation so that ``torch.fx`` captures it as a single node,
* an autograd formula whose backward is again made of ``mm_ops`` operators
  (so the backward graph is captured at kernel granularity too), and
* a sharding rule for the graph compiler (index classes: which dimensions of
  operands and results carry the same index, which must stay unsharded, which
  are summed away).

``FAST_OPS`` maps operator names to variants used inside compiled task
programs: they skip the dispatcher, may update dead inputs in place, and can
accumulate straight into a gradient accumulator (``acc=``) - e.g. the
weight-gradient GEMM adds into the fp32 accumulator in its epilogue.
"""
from __future__ import annotations

from typing import Dict

import torch

from . import kernels as K
from ..compiler.capture import register_shard_rule

lib = torch.library.Library("mm_ops", "DEF")


def _define(schema: str, impl, fake, *, backward=None, setup=None):
    name = schema.split("(")[0]
    lib.define(schema)
    torch.library.impl(lib, name, "CompositeExplicitAutograd")(impl)
    torch.library.register_fake(f"mm_ops::{name}")(fake)
    if backward is not None:
        torch.library.register_autograd(f"mm_ops::{name}", backward, setup_context=setup)


def _cls(members, no_shard=False, reduced=()):
    return {"members": [list(m) for m in members], "no_shard": no_shard, "reduced_outputs": list(reduced)}


def _flat2(x: torch.Tensor) -> torch.Tensor:
    return x.reshape(-1, x.shape[-1])


# ------------------------------------------------------------------------ linear
# x: [*B, K], w: [*N, K] -> y: [*B, *N].  Several "N" dimensions let a fused projection
# (gate|up, packed q|k|v heads) be sharded along the inner ones.
def linear_impl(x, w):
    K_ = x.shape[-1]
    return K.linear_fwd(x.reshape(-1, K_), w.reshape(-1, K_)).view(*x.shape[:-1], *w.shape[:-1])


def linear_dgrad_impl(dy, w):
    K_ = w.shape[-1]
    w2 = w.reshape(-1, K_)
    nb = dy.dim() - (w.dim() - 1)
    return K.linear_dgrad(dy.reshape(-1, w2.shape[0]), w2).view(*dy.shape[:nb], K_)


def linear_wgrad_impl(dy, x):
    K_ = x.shape[-1]
    nb = x.dim() - 1
    x2 = x.reshape(-1, K_)
    return K.linear_wgrad(dy.reshape(x2.shape[0], -1), x2).view(*dy.shape[nb:], K_)


_define("linear(Tensor x, Tensor w) -> Tensor", linear_impl,
        lambda x, w: x.new_empty(*x.shape[:-1], *w.shape[:-1]),
        backward=lambda ctx, g: (torch.ops.mm_ops.linear_dgrad(g, ctx.saved_tensors[1]),
                                 torch.ops.mm_ops.linear_wgrad(g, ctx.saved_tensors[0])),
        setup=lambda ctx, inputs, output: ctx.save_for_backward(*inputs))
_define("linear_dgrad(Tensor dy, Tensor w) -> Tensor", linear_dgrad_impl,
        lambda dy, w: dy.new_empty(*dy.shape[:dy.dim() - (w.dim() - 1)], w.shape[-1]))
_define("linear_wgrad(Tensor dy, Tensor x) -> Tensor", linear_wgrad_impl,
        lambda dy, x: dy.new_empty(*dy.shape[x.dim() - 1:], x.shape[-1]))


def linear_wgrad_fast(dy, x, acc=None):
    """Weight gradient; with ``acc`` = (buffer or None, dtype) the GEMM epilogue writes /
    accumulates straight into the gradient accumulator."""
    if acc is None:
        return linear_wgrad_impl(dy, x)
    buf, dtype = acc
    K_ = x.shape[-1]
    nb = x.dim() - 1
    x2 = x.reshape(-1, K_)
    dy2 = dy.reshape(x2.shape[0], -1)
    if buf is None:
        return K.linear_wgrad(dy2, x2, out_dtype=dtype).view(*dy.shape[nb:], K_)
    K.linear_wgrad(dy2, x2, out=buf.view(-1, K_), accumulate=True)
    return buf


@register_shard_rule("mm_ops.linear.default")
def _rule_linear(node, ins, outs):
    xb, wn = len(ins[0]) - 1, len(ins[1]) - 1
    classes = [_cls([(0, d), (2, d)]) for d in range(xb)]
    classes += [_cls([(1, d), (2, xb + d)]) for d in range(wn)]
    classes.append(_cls([(0, xb), (1, wn)], reduced=[0]))
    return {"classes": classes}


@register_shard_rule("mm_ops.linear_dgrad.default")
def _rule_linear_dgrad(node, ins, outs):
    wn = len(ins[1]) - 1
    nb = len(ins[0]) - wn
    classes = [_cls([(0, d), (2, d)]) for d in range(nb)]
    classes += [_cls([(0, nb + d), (1, d)], reduced=[0]) for d in range(wn)]
    classes.append(_cls([(1, wn), (2, nb)]))
    return {"classes": classes}


@register_shard_rule("mm_ops.linear_wgrad.default")
def _rule_linear_wgrad(node, ins, outs):
    nb = len(ins[1]) - 1
    wn = len(ins[0]) - nb
    classes = [_cls([(0, d), (1, d)], reduced=[0]) for d in range(nb)]
    classes += [_cls([(0, nb + d), (2, d)]) for d in range(wn)]
    classes.append(_cls([(1, nb), (2, wn)]))
    return {"classes": classes}


# ----------------------------------------------------------------------- rmsnorm
def rmsnorm_impl(x, w, eps):
    y, rstd = K.rmsnorm_fwd(x, w, eps)
    return y, rstd.view(x.shape[:-1])


def rmsnorm_bwd_impl(x, w, dy, rstd):
    dx, dw = K.rmsnorm_bwd(x, w, dy, rstd.reshape(-1))
    return dx, dw.to(w.dtype)


def _rmsnorm_backward(ctx, gy, grstd):
    x, w, rstd = ctx.saved_tensors
    dx, dw = torch.ops.mm_ops.rmsnorm_bwd(x, w, gy, rstd)
    return dx, dw, None


def _rmsnorm_setup(ctx, inputs, output):
    x, w, eps = inputs
    ctx.save_for_backward(x, w, output[1])


_define("rmsnorm(Tensor x, Tensor w, float eps) -> (Tensor, Tensor)", rmsnorm_impl,
        lambda x, w, eps: (torch.empty_like(x), x.new_empty(x.shape[:-1], dtype=torch.float32)),
        backward=_rmsnorm_backward, setup=_rmsnorm_setup)
_define("rmsnorm_bwd(Tensor x, Tensor w, Tensor dy, Tensor rstd) -> (Tensor, Tensor)", rmsnorm_bwd_impl,
        lambda x, w, dy, rstd: (torch.empty_like(x), torch.empty_like(w)))


def add_rmsnorm_impl(x, delta, w, eps):
    xn = K.add(x, delta)
    y, rstd = K.rmsnorm_fwd(xn, w, eps)
    return xn, y, rstd.view(x.shape[:-1])


def add_rmsnorm_bwd_impl(xn, w, dxn, dy, rstd):
    """d(sum) = dxn + rmsnorm_bwd(xn, w, dy): the add is fused into the kernel's epilogue."""
    acc = dxn.clone()
    _, dw = K.rmsnorm_bwd(xn, w, dy, rstd.reshape(-1), dx_inout=acc)
    return acc, dw.to(w.dtype)


def add_rmsnorm_bwd_fast(xn, w, dxn, dy, rstd):
    # dxn is dead after this operator inside a compiled task: accumulate in place
    _, dw = K.rmsnorm_bwd(xn, w, dy, rstd.reshape(-1), dx_inout=dxn)
    return dxn, dw.to(w.dtype)


def _add_rmsnorm_backward(ctx, gxn, gy, grstd):
    xn, w, rstd = ctx.saved_tensors
    if gxn is None:
        dsum, dw = torch.ops.mm_ops.rmsnorm_bwd(xn, w, gy, rstd)
    elif gy is None:
        return gxn, gxn, None, None
    else:
        dsum, dw = torch.ops.mm_ops.add_rmsnorm_bwd(xn, w, gxn, gy, rstd)
    return dsum, dsum, dw, None


def _add_rmsnorm_setup(ctx, inputs, output):
    ctx.save_for_backward(output[0], inputs[2], output[2])


_define("add_rmsnorm(Tensor x, Tensor delta, Tensor w, float eps) -> (Tensor, Tensor, Tensor)", add_rmsnorm_impl,
        lambda x, delta, w, eps: (torch.empty_like(x), torch.empty_like(x),
                                  x.new_empty(x.shape[:-1], dtype=torch.float32)),
        backward=_add_rmsnorm_backward, setup=_add_rmsnorm_setup)
_define("add_rmsnorm_bwd(Tensor xn, Tensor w, Tensor dxn, Tensor dy, Tensor rstd) -> (Tensor, Tensor)",
        add_rmsnorm_bwd_impl, lambda xn, w, dxn, dy, rstd: (torch.empty_like(xn), torch.empty_like(w)))


# ------------------------------------------------------------------------ swiglu
# gu: [..., 2, F] (gate = gu[..., 0, :], up = gu[..., 1, :]) -> [..., F]
def swiglu_impl(gu):
    F = gu.shape[-1]
    return K.swiglu_fwd(gu.reshape(-1, 2 * F)).view(*gu.shape[:-2], F)


def swiglu_bwd_impl(gu, dh):
    F = gu.shape[-1]
    return K.swiglu_bwd(gu.reshape(-1, 2 * F), dh.reshape(-1, F)).view(gu.shape)


_define("swiglu(Tensor gu) -> Tensor", swiglu_impl,
        lambda gu: gu.new_empty(*gu.shape[:-2], gu.shape[-1]),
        backward=lambda ctx, g: torch.ops.mm_ops.swiglu_bwd(ctx.saved_tensors[0], g),
        setup=lambda ctx, inputs, output: ctx.save_for_backward(inputs[0]))
_define("swiglu_bwd(Tensor gu, Tensor dh) -> Tensor", swiglu_bwd_impl, lambda gu, dh: torch.empty_like(gu))


# --------------------------------------------------------------------- attention
def _split_qkv(qkv, rep: int):
    """Views of a packed projection [B, S, hkv*(rep+2), D] whose heads are grouped per
    key/value head: ``rep`` query heads, then the key head, then the value head. A split of
    the packed dimension into equal contiguous parts therefore keeps whole groups together,
    which is what makes the layout tensor-parallel friendly. Returns q [B,S,hkv,rep,D] and
    k, v [B,S,hkv,D] (all strided views)."""
    B, S, H, D = qkv.shape
    g = qkv.view(B, S, H // (rep + 2), rep + 2, D)
    return g[:, :, :, :rep], g[:, :, :, rep], g[:, :, :, rep + 1]


def attention_impl(qkv, cos, sin, rep: int, inplace: bool = False):
    """Causal self-attention over a packed, group-major [B, S, hkv*(rep+2), D] projection
    with rotary embedding applied to the query and key heads first. Returns (out
    [B,S,hq,D], lse [B,hq,S], the rotated qkv saved for the backward pass). Head counts are
    derived from the tensor, so a head-sharded (tensor-parallel) slice works unchanged."""
    from .attention import attention_fwd_packed
    B, S, H, D = qkv.shape
    qkv_r = qkv if inplace else qkv.clone()
    K.rope_(qkv_r.view(B * S, H, D), cos, sin, rot_per_group=rep + 1, group_size=rep + 2)
    out, lse = attention_fwd_packed(qkv_r, rep)
    return out, lse, qkv_r


def attention_bwd_impl(dout, qkv_r, out, lse, cos, sin, rep: int):
    from .attention import attention_bwd_packed
    B, S, H, D = qkv_r.shape
    dqkv = attention_bwd_packed(dout, qkv_r, out, lse, rep)
    K.rope_(dqkv.view(B * S, H, D), cos, sin, backward=True, rot_per_group=rep + 1, group_size=rep + 2)
    return dqkv


def _attention_backward(ctx, gout, glse, gqkv):
    qkv_r, out, lse, cos, sin = ctx.saved_tensors
    dqkv = torch.ops.mm_ops.attention_bwd(gout, qkv_r, out, lse, cos, sin, ctx.rep)
    return dqkv, None, None, None


def _attention_setup(ctx, inputs, output):
    qkv, cos, sin, rep = inputs
    ctx.rep = rep
    ctx.save_for_backward(output[2], output[0], output[1], cos, sin)


def _attention_fake(qkv, cos, sin, rep):
    hq = rep * (qkv.shape[2] // (rep + 2))
    return (qkv.new_empty(qkv.shape[0], qkv.shape[1], hq, qkv.shape[3]),
            qkv.new_empty(qkv.shape[0], hq, qkv.shape[1], dtype=torch.float32), torch.empty_like(qkv))


_define("attention(Tensor qkv, Tensor cos, Tensor sin, int rep) -> (Tensor, Tensor, Tensor)",
        lambda qkv, cos, sin, rep: attention_impl(qkv, cos, sin, rep, False), _attention_fake,
        backward=_attention_backward, setup=_attention_setup)
_define("attention_bwd(Tensor dout, Tensor qkv_r, Tensor out, Tensor lse, Tensor cos, Tensor sin, int rep)"
        " -> Tensor", attention_bwd_impl,
        lambda dout, qkv_r, out, lse, cos, sin, rep: torch.empty_like(qkv_r))


# ----------------------------------------------------------------- cross entropy
def cross_entropy_impl(logits, targets, scale: float, inplace: bool = False):
    """Sum over tokens of the token cross-entropy times ``scale``; also returns
    d(loss)/d(logits) (computed in the same pass, written over the logits when
    ``inplace``)."""
    buf = logits if inplace else logits.clone()
    flat = _flat2(buf)
    loss_rows = K.cross_entropy_fwd_bwd(flat, targets.reshape(-1), scale, write_grad=True)
    return loss_rows.sum() * scale, buf


def _ce_backward(ctx, gloss, gdlogits):
    (dlogits,) = ctx.saved_tensors
    return dlogits * gloss.to(dlogits.dtype), None, None


_define("cross_entropy(Tensor logits, Tensor targets, float scale) -> (Tensor, Tensor)",
        lambda logits, targets, scale: cross_entropy_impl(logits, targets, scale, False),
        lambda logits, targets, scale: (logits.new_empty((), dtype=torch.float32), torch.empty_like(logits)),
        backward=_ce_backward, setup=lambda ctx, inputs, output: ctx.save_for_backward(output[1]))


# --------------------------------------------------------------------- embedding
def embedding_impl(table, ids):
    return K.embedding_fwd(table, ids).view(*ids.shape, table.shape[1])


def embedding_bwd_impl(dout, ids, vocab: int):
    grad = torch.zeros(vocab, dout.shape[-1], dtype=torch.float32, device=dout.device)
    K.embedding_bwd(_flat2(dout), ids, grad)
    return grad.to(dout.dtype)


def embedding_bwd_fast(dout, ids, vocab: int, acc=None):
    if acc is None:
        return embedding_bwd_impl(dout, ids, vocab)
    buf, dtype = acc
    if buf is None:
        buf = torch.zeros(vocab, dout.shape[-1], dtype=dtype, device=dout.device)
    if buf.dtype == torch.float32:
        K.embedding_bwd(_flat2(dout), ids, buf)
    else:
        buf.add_(embedding_bwd_impl(dout, ids, vocab))
    return buf


def _embedding_setup(ctx, inputs, output):
    ctx.save_for_backward(inputs[1])
    ctx.vocab = inputs[0].shape[0]


_define("embedding(Tensor table, Tensor ids) -> Tensor", embedding_impl,
        lambda table, ids: table.new_empty(*ids.shape, table.shape[1]),
        backward=lambda ctx, g: (torch.ops.mm_ops.embedding_bwd(g, ctx.saved_tensors[0], ctx.vocab), None),
        setup=_embedding_setup)
_define("embedding_bwd(Tensor dout, Tensor ids, int vocab) -> Tensor", embedding_bwd_impl,
        lambda dout, ids, vocab: dout.new_empty(vocab, dout.shape[-1]))


# ------------------------------------------------------------------------- adamw
def adamw_impl(param, master, m, v, grad, step, lr: float, beta1: float, beta2: float, eps: float, wd: float,
               grad_scale: float, inplace: bool = False):
    """One AdamW update. Returns (working copy, master, m, v). ``param`` is the current
    working copy (its buffer is reused when ``inplace``); ``step`` is a 1-element int64
    tensor on the same device holding the step count *after* this update (the kernel
    reads it, so the update never synchronises with the host)."""
    if not inplace:
        param, master, m, v = torch.empty_like(param), master.clone(), m.clone(), v.clone()
    g = grad.reshape(-1)
    if g.dtype != torch.float32:
        g = g.float()
    if param.is_cuda and param.dtype != torch.bfloat16:
        raise TypeError("the CUDA AdamW kernel keeps a bf16 working copy")
    K.adamw_step_(master.view(-1), param.view(-1), m.view(-1), v.view(-1), g, lr=lr, beta1=beta1, beta2=beta2,
                  eps=eps, weight_decay=wd, step=step.reshape(-1), grad_scale=grad_scale)
    return param, master, m, v


_define("adamw(Tensor param, Tensor master, Tensor m, Tensor v, Tensor grad, Tensor step, float lr, float beta1,"
        " float beta2, float eps, float wd, float grad_scale) -> (Tensor, Tensor, Tensor, Tensor)",
        lambda param, master, m, v, grad, step, lr, beta1, beta2, eps, wd, gs: adamw_impl(
            param, master, m, v, grad, step, lr, beta1, beta2, eps, wd, gs, False),
        lambda param, master, m, v, grad, step, lr, beta1, beta2, eps, wd, gs: (
            torch.empty_like(param), torch.empty_like(master), torch.empty_like(m), torch.empty_like(v)))


# -------------------------------------------------------------------- shard rules
def _leading(nin, x_slot, out_slots, rank_minus_1, extra_in=()):
    """Index classes tying leading dims of operand `x_slot` to the same dims of outputs."""
    classes = []
    for d in range(rank_minus_1):
        members = [(x_slot, d)] + [(s, d) for s in extra_in] + [(nin + o, d) for o in out_slots]
        classes.append(_cls(members))
    return classes


@register_shard_rule("mm_ops.rmsnorm.default")
def _rule_rmsnorm(node, ins, outs):
    r = len(ins[0])
    classes = _leading(2, 0, [0, 1], r - 1)
    classes.append(_cls([(0, r - 1), (1, 0), (2, r - 1)], no_shard=True))
    return {"classes": classes}


@register_shard_rule("mm_ops.rmsnorm_bwd.default")
def _rule_rmsnorm_bwd(node, ins, outs):
    r = len(ins[0])
    classes = []
    for d in range(r - 1):
        classes.append(_cls([(0, d), (2, d), (3, d), (4, d)], reduced=[1]))
    classes.append(_cls([(0, r - 1), (1, 0), (2, r - 1), (4, r - 1), (5, 0)], no_shard=True))
    return {"classes": classes}


@register_shard_rule("mm_ops.add_rmsnorm.default")
def _rule_add_rmsnorm(node, ins, outs):
    r = len(ins[0])
    classes = []
    for d in range(r - 1):
        classes.append(_cls([(0, d), (1, d), (3, d), (4, d), (5, d)]))
    classes.append(_cls([(0, r - 1), (1, r - 1), (2, 0), (3, r - 1), (4, r - 1)], no_shard=True))
    return {"classes": classes}


@register_shard_rule("mm_ops.add_rmsnorm_bwd.default")
def _rule_add_rmsnorm_bwd(node, ins, outs):
    r = len(ins[0])
    classes = []
    for d in range(r - 1):
        classes.append(_cls([(0, d), (2, d), (3, d), (4, d), (5, d)], reduced=[1]))
    classes.append(_cls([(0, r - 1), (1, 0), (2, r - 1), (3, r - 1), (5, r - 1), (6, 0)], no_shard=True))
    return {"classes": classes}


@register_shard_rule("mm_ops.swiglu.default")
def _rule_swiglu(node, ins, outs):
    r = len(ins[0])
    classes = [_cls([(0, d), (1, d)]) for d in range(r - 2)]
    classes.append(_cls([(0, r - 2)], no_shard=True))
    classes.append(_cls([(0, r - 1), (1, r - 2)]))
    return {"classes": classes}


@register_shard_rule("mm_ops.swiglu_bwd.default")
def _rule_swiglu_bwd(node, ins, outs):
    r = len(ins[0])
    classes = [_cls([(0, d), (1, d), (2, d)]) for d in range(r - 2)]
    classes.append(_cls([(0, r - 2), (2, r - 2)], no_shard=True))
    classes.append(_cls([(0, r - 1), (1, r - 2), (2, r - 1)]))
    return {"classes": classes}


@register_shard_rule("mm_ops.attention.default")
def _rule_attention(node, ins, outs):
    # qkv [B,S,H,D], cos, sin -> out [B,S,hq,D], lse [B,hq,S], qkv_r [B,S,H,D]
    return {"classes": [
        _cls([(0, 0), (3, 0), (4, 0), (5, 0)]),                     # batch
        _cls([(0, 2), (3, 2), (4, 1), (5, 2)]),                     # heads (packed groups shard together)
        _cls([(0, 1), (3, 1), (4, 2), (5, 1)], no_shard=True),      # sequence
        _cls([(0, 3), (3, 3), (5, 3)], no_shard=True),              # head dim
    ]}


@register_shard_rule("mm_ops.attention_bwd.default")
def _rule_attention_bwd(node, ins, outs):
    # dout, qkv_r, out, lse, cos, sin -> dqkv
    return {"classes": [
        _cls([(0, 0), (1, 0), (2, 0), (3, 0), (6, 0)]),
        _cls([(0, 2), (1, 2), (2, 2), (3, 1), (6, 2)]),
        _cls([(0, 1), (1, 1), (2, 1), (3, 2), (6, 1)], no_shard=True),
        _cls([(0, 3), (1, 3), (2, 3), (6, 3)], no_shard=True),
    ]}


@register_shard_rule("mm_ops.cross_entropy.default")
def _rule_cross_entropy(node, ins, outs):
    # slots: 0 logits, 1 targets | 2 loss, 3 dlogits. The vocabulary dimension may be sharded: the
    # per-device form of the operator (``cross_entropy_local``) then exchanges the softmax
    # statistics with the other shards itself, so the loss is not a partial sum over that axis.
    r = len(ins[0])
    classes = []
    for d in range(r - 1):
        classes.append(_cls([(0, d), (1, d), (3, d)], reduced=[0]))
    vocab = _cls([(0, r - 1), (3, r - 1)])
    vocab["shares_axes"] = True
    classes.append(vocab)
    return {"classes": classes}


def cross_entropy_local(ctx, axes, key, logits, targets, scale: float):
    """This device's share of a cross-entropy whose vocabulary is sharded over the mesh axes
    ``axes``: local statistics (max, sum-exp, target logit), exchange with the other shards
    (peer memory on GPUs: every rank's combine kernel reads the others' statistics directly),
    then the gradient of the local slice from the global statistics. Returns (loss summed over
    the local rows times ``scale`` - the same on every shard -, d loss / d logits slice)."""
    group, me = ctx.group_of(axes)
    if len(group) == 1:
        return cross_entropy_impl(logits, targets, scale, False)
    V_local = logits.shape[-1]
    buf = logits.clone()
    flat = buf.view(-1, V_local)
    tflat = targets.reshape(-1)
    stats = K.cross_entropy_stats(flat, tflat, me * V_local)
    stats2, loss_rows = ctx.combine_softmax_stats(stats, tflat, group, key)
    K.cross_entropy_apply(flat, tflat, stats2, me * V_local, scale)
    return loss_rows.sum() * scale, buf


# Operators whose per-device form talks to the other devices of the task over the mesh axes of the
# index class marked ``shares_axes``: operator name -> (function(ctx, axes, key, *args), slot of the
# tensor argument that carries that class). Other modules add their own entries.
CTX_OPS: Dict[str, tuple] = {
    "mm_ops.cross_entropy.default": (cross_entropy_local, 0),
}


@register_shard_rule("mm_ops.embedding.default")
def _rule_embedding(node, ins, outs):
    r = len(ins[1])
    classes = [_cls([(1, d), (2, d)]) for d in range(r)]
    classes.append(_cls([(0, 1), (2, r)]))
    classes.append(_cls([(0, 0)], no_shard=True))
    return {"classes": classes}


@register_shard_rule("mm_ops.embedding_bwd.default")
def _rule_embedding_bwd(node, ins, outs):
    r = len(ins[1])
    classes = [_cls([(0, d), (1, d)], reduced=[0]) for d in range(r)]
    classes.append(_cls([(0, r), (2, 1)]))
    classes.append(_cls([(2, 0)], no_shard=True))
    return {"classes": classes}


@register_shard_rule("mm_ops.adamw.default")
def _rule_adamw(node, ins, outs):
    r = len(ins[0])
    return {"classes": [_cls([(0, d), (1, d), (2, d), (3, d), (4, d), (6, d), (7, d), (8, d), (9, d)])
                        for d in range(r)]}


# ----------------------------------------------------------------------- fast ops
def _attention_fast(qkv, cos, sin, rep):
    return attention_impl(qkv, cos, sin, rep, inplace=True)


def _cross_entropy_fast(logits, targets, scale):
    return cross_entropy_impl(logits, targets, scale, inplace=True)


def _adamw_fast(param, master, m, v, grad, step, lr, beta1, beta2, eps, wd, gs):
    return adamw_impl(param, master, m, v, grad, step, lr, beta1, beta2, eps, wd, gs, inplace=True)


FAST_OPS: Dict[str, object] = {
    "mm_ops.linear.default": linear_impl,
    "mm_ops.linear_dgrad.default": linear_dgrad_impl,
    "mm_ops.linear_wgrad.default": linear_wgrad_fast,
    "mm_ops.rmsnorm.default": rmsnorm_impl,
    "mm_ops.rmsnorm_bwd.default": rmsnorm_bwd_impl,
    "mm_ops.add_rmsnorm.default": add_rmsnorm_impl,
    "mm_ops.add_rmsnorm_bwd.default": add_rmsnorm_bwd_fast,
    "mm_ops.swiglu.default": swiglu_impl,
    "mm_ops.swiglu_bwd.default": swiglu_bwd_impl,
    "mm_ops.attention.default": _attention_fast,
    "mm_ops.attention_bwd.default": attention_bwd_impl,
    "mm_ops.cross_entropy.default": _cross_entropy_fast,
    "mm_ops.embedding.default": embedding_impl,
    "mm_ops.embedding_bwd.default": embedding_bwd_fast,
    "mm_ops.adamw.default": _adamw_fast,
}
# tensor operands (by position among the tensor arguments) that the fast variant overwrites
INPLACE_OPERANDS: Dict[str, tuple] = {
    "mm_ops.add_rmsnorm_bwd.default": (2,),
    "mm_ops.attention.default": (0,),
    "mm_ops.cross_entropy.default": (0,),
}
# operators whose fast variant can write into a gradient accumulator (acc=(buffer|None, dtype))
ACC_FUSABLE = {"mm_ops.linear_wgrad.default", "mm_ops.embedding_bwd.default"}
