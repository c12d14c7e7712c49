"""Llama-family decoder (Llama-2 MHA and Llama-3 GQA shapes) written against ``mm_ops``.

The model is a pure function of a parameter pytree, so the same code runs
eagerly on one device (reference for differential tests) and is captured by
``torch.fx`` and partitioned into pipeline stages / tensor-parallel shards by
the MPMD compiler. Parameter layouts are chosen so that tensor-parallel
sharding is a plain dimension split:

* ``wqkv``  [H_total, Dh, D]   packed heads: ``hq`` query heads, then ``hkv`` key heads,
                               then ``hkv`` value heads (per tensor-parallel shard)
* ``wo``    [D, hq*Dh]
* ``wgu``   [2, F, D]          gate (index 0) and up (index 1) projections
* ``wdown`` [D, F]

Every layer is wrapped in ``named_scope("layers.<i>")`` so that regex task
registrations can place layers on pipeline stages.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch

from .. import lib as mm_lib
from ..ops import kernels as K
from ..ops import mm_ops  # noqa: F401  (registers the operators)
from ..ops import moe as _moe  # noqa: F401  (registers the mixture-of-experts operators)
from ..task import MultiMesh, Task, microbatch, named_scope, value_and_grad

ops = torch.ops.mm_ops


@dataclass
class LlamaConfig:
    vocab: int = 32000
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 32
    d_ff: int = 11008
    rope_theta: float = 1e4
    eps: float = 1e-5
    dtype: torch.dtype = torch.bfloat16
    # layers after which the residual stream leaves its task sharded on the hidden dimension
    # (logical axis "boundary_hidden") instead of on the batch: with the next layer on another
    # pipeline stage, every microbatch then crosses the stage boundary through a reshard that
    # changes the layout (hidden-sharded on the sender, batch-sharded on the receiver)
    hidden_sharded_after: Tuple[int, ...] = ()
    n_experts: int = 0      # > 0: every feed-forward block is a sparse mixture of SwiGLU experts
    top_k: int = 2          # experts per token (softmax over the chosen router logits)
    # Megatron-style sequence parallelism: between the tensor-parallel projections the residual
    # stream, the norms and their gradients are sharded on the sequence dimension over the
    # tensor-parallel mesh axis (logical axis "seq"). The layout changes in front of the
    # column-parallel projections (an all-gather, fused into the GEMM that reads the activation)
    # and behind the row-parallel ones (a reduce-scatter, fused into the GEMM that produces the
    # partial sums) instead of an all-reduce of replicated activations.
    sequence_parallel: bool = False
    # output projection and loss sharded on the vocabulary over the tensor-parallel axis (logical
    # axis "vocab"): every rank computes its slice of the logits; the softmax statistics are
    # exchanged between the ranks inside the loss operator
    vocab_parallel: bool = False

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @staticmethod
    def llama2_7b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig(vocab=128256, n_kv_heads=8, d_ff=14336, rope_theta=5e5)

    @staticmethod
    def mixtral_8x7b() -> "LlamaConfig":
        return LlamaConfig(vocab=32000, n_kv_heads=8, d_ff=14336, rope_theta=1e6, n_experts=8, top_k=2)

    @staticmethod
    def tiny(n_layers: int = 2, d_model: int = 256, n_heads: int = 2, n_kv_heads: int = 2, d_ff: int = 512,
             vocab: int = 512, n_experts: int = 0, top_k: int = 2) -> "LlamaConfig":
        return LlamaConfig(vocab=vocab, d_model=d_model, n_layers=n_layers, n_heads=n_heads, n_kv_heads=n_kv_heads,
                           d_ff=d_ff, n_experts=n_experts, top_k=top_k)

    def num_params(self) -> int:
        ffn = 3 * self.d_ff * self.d_model
        if self.n_experts:
            ffn = self.n_experts * ffn + self.n_experts * self.d_model
        per_layer = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim * self.d_model + self.d_model * self.d_model \
            + ffn + 2 * self.d_model
        return self.n_layers * per_layer + 2 * self.vocab * self.d_model + self.d_model

    def active_params(self) -> int:
        """Parameters a token actually multiplies with (``top_k`` of the experts)."""
        if not self.n_experts:
            return self.num_params()
        idle = (self.n_experts - self.top_k) * 3 * self.d_ff * self.d_model
        return self.num_params() - self.n_layers * idle

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token (forward + backward = 3x forward), causal attention counted at half."""
        dense = 2 * (self.active_params() - self.vocab * self.d_model)
        attn = 2 * 2 * seq_len * self.d_model * self.n_layers / 2
        return 3.0 * (dense + attn)


def init_params(cfg: LlamaConfig, device="cpu", seed: int = 0) -> Dict[str, Any]:
    g = torch.Generator(device="cpu").manual_seed(seed)
    dt = cfg.dtype
    D, Dh, F = cfg.d_model, cfg.head_dim, cfg.d_ff
    H = cfg.n_heads + 2 * cfg.n_kv_heads
    dev = torch.device(device)
    meta = dev.type == "meta"

    def normal(*shape, std=0.02):
        if meta:
            return torch.empty(*shape, dtype=dt, device=dev)
        if dev.type == "cuda":
            return (torch.randn(*shape, device=dev, dtype=torch.float32) * std).to(dt)
        return (torch.randn(*shape, generator=g) * std).to(dt).to(dev)

    def ones(*shape):
        return torch.ones(*shape, dtype=dt, device=dev)

    layers = []
    for _ in range(cfg.n_layers):
        layers.append({
            "attn_norm": ones(D),
            "wqkv": normal(H, Dh, D),
            "wo": normal(D, cfg.n_heads * Dh, std=0.02 / math.sqrt(2 * cfg.n_layers)),
            "ffn_norm": ones(D),
            **({"wgu": normal(2, F, D),
                "wdown": normal(D, F, std=0.02 / math.sqrt(2 * cfg.n_layers))} if not cfg.n_experts else
               {"router": normal(cfg.n_experts, D),
                "wgu": normal(cfg.n_experts, 2, F, D),
                "wdown": normal(cfg.n_experts, D, F, std=0.02 / math.sqrt(2 * cfg.n_layers))}),
        })
    return {"embed": normal(cfg.vocab, D), "layers": layers, "final_norm": ones(D), "lm_head": normal(cfg.vocab, D)}


def rope_tables(cfg: LlamaConfig, seq_len: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    return K.rope_tables(seq_len, cfg.head_dim, cfg.rope_theta, device)


def sp_enter(cfg: LlamaConfig, h: torch.Tensor) -> torch.Tensor:
    """Sequence-sharded activation -> full sequence, in front of a tensor-parallel projection.
    The cotangent takes the opposite way (full -> sequence-sharded: a reduce-scatter of the
    projection's partial input gradients)."""
    if not cfg.sequence_parallel:
        return h
    return mm_lib.relayout(h, ("batch", None, None), grad_spec=("batch", "seq", None))


def sp_leave(cfg: LlamaConfig, y: torch.Tensor) -> torch.Tensor:
    """Output of a row-parallel projection (partial sums over the tensor-parallel ranks) ->
    sequence-sharded; its cotangent is gathered back to the full sequence."""
    if not cfg.sequence_parallel:
        return y
    return mm_lib.relayout(y, ("batch", "seq", None), grad_spec=("batch", None, None))


def attention_block(cfg: LlamaConfig, p: Dict[str, torch.Tensor], h: torch.Tensor, cos, sin) -> torch.Tensor:
    """h: normalised activations [B, S, D] -> attention branch output [B, S, D]."""
    B, S, D = h.shape
    qkv = ops.linear(sp_enter(cfg, h), p["wqkv"])        # [B, S, H_total, Dh]
    qkv = mm_lib.with_sharding_constraint(qkv, ("batch", None, "heads", None))
    out, _, _ = ops.attention(qkv, cos, sin, cfg.n_heads // cfg.n_kv_heads)
    return sp_leave(cfg, ops.linear(out.flatten(2), p["wo"]))


def mlp_block(cfg: LlamaConfig, p: Dict[str, torch.Tensor], h: torch.Tensor) -> torch.Tensor:
    if cfg.n_experts:
        # experts live on the devices of the `expert` logical axis; tokens stay where they are and
        # travel to their experts and back inside the operator
        wgu = mm_lib.with_sharding_constraint(p["wgu"], ("expert", None, None, None))
        wdown = mm_lib.with_sharding_constraint(p["wdown"], ("expert", None, None))
        return ops.moe_ffn(h, p["router"], wgu, wdown, cfg.top_k)
    gu = ops.linear(sp_enter(cfg, h), p["wgu"])           # [B, S, 2, F]
    gu = mm_lib.with_sharding_constraint(gu, ("batch", None, None, "mlp"))
    return sp_leave(cfg, ops.linear(ops.swiglu(gu), p["wdown"]))


def forward_layers(cfg: LlamaConfig, layers: Sequence[Dict[str, torch.Tensor]], x: torch.Tensor, h: torch.Tensor,
                   cos, sin, next_norms: Sequence[torch.Tensor], first_index: int = 0):
    """Runs a run of layers. ``x`` is the residual stream, ``h`` its normalised copy for the
    first layer; ``next_norms[i]`` is the norm weight applied after layer i (the next
    layer's attention norm, or the final norm). Returns the new (x, h)."""
    for i, p in enumerate(layers):
        with named_scope(f"layers.{first_index + i}"):
            if (first_index + i - 1) in cfg.hidden_sharded_after:
                # receiving side of a forced boundary: batch-sharded again
                x = mm_lib.relayout(x, ("batch", None, None))
                h = mm_lib.relayout(h, ("batch", None, None))
            a = attention_block(cfg, p, h, cos, sin)
            x, h, _ = ops.add_rmsnorm(x, a, p["ffn_norm"], cfg.eps)
            m = mlp_block(cfg, p, h)
            x, h, _ = ops.add_rmsnorm(x, m, next_norms[i], cfg.eps)
            if (first_index + i) in cfg.hidden_sharded_after:
                x = mm_lib.relayout(x, (None, None, "boundary_hidden"))
                h = mm_lib.relayout(h, (None, None, "boundary_hidden"))
            elif cfg.sequence_parallel and not cfg.n_experts:
                x = mm_lib.with_sharding_constraint(x, ("batch", "seq", None))
                h = mm_lib.with_sharding_constraint(h, ("batch", "seq", None))
            else:
                x = mm_lib.with_sharding_constraint(x, ("batch", None, None))
    return x, h


def loss_fn(cfg: LlamaConfig, params: Dict[str, Any], tokens: torch.Tensor, labels: torch.Tensor, cos, sin,
            loss_scale: float) -> torch.Tensor:
    """Sum over tokens of the next-token cross-entropy, times ``loss_scale``."""
    layers = params["layers"]
    sp = cfg.sequence_parallel and not cfg.n_experts
    with named_scope("embed"):
        x = ops.embedding(params["embed"], tokens)         # [B, S, D]
        if sp:
            x = mm_lib.with_sharding_constraint(x, ("batch", "seq", None))
        h, _ = ops.rmsnorm(x, layers[0]["attn_norm"], cfg.eps)
    next_norms = [l["attn_norm"] for l in layers[1:]] + [params["final_norm"]]
    x, h = forward_layers(cfg, layers, x, h, cos, sin, next_norms)
    with named_scope("head"):
        w_out = params["lm_head"]
        if cfg.vocab_parallel:
            w_out = mm_lib.with_sharding_constraint(w_out, ("vocab", None))
        logits = ops.linear(sp_enter(cfg, h) if sp else h, w_out)   # [B, S, V]
        if cfg.vocab_parallel:
            logits = mm_lib.with_sharding_constraint(logits, ("batch", None, "vocab"))
        loss, _ = ops.cross_entropy(logits, labels, loss_scale)
    return loss


# ---------------------------------------------------------------------------
# Optimiser state and the training step
# ---------------------------------------------------------------------------
@dataclass
class AdamWConfig:
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1


def init_opt_state(params: Dict[str, Any]) -> Dict[str, Any]:
    from torch.utils import _pytree as pytree
    leaves, spec = pytree.tree_flatten(params)
    master = [l.float() for l in leaves]
    m = [torch.zeros_like(x) for x in master]
    v = [torch.zeros_like(x) for x in master]
    step = torch.zeros(1, dtype=torch.int64, device=leaves[0].device)
    return {"master": pytree.tree_unflatten(master, spec), "m": pytree.tree_unflatten(m, spec),
            "v": pytree.tree_unflatten(v, spec), "step": step}


def annotate_fsdp(params: Dict[str, Any]) -> Dict[str, Any]:
    """Gives every weight matrix the logical axis ``fsdp`` on a dimension that tensor
    parallelism leaves alone (and keeps ``heads`` / ``mlp`` on the dimension it shards). Mapped
    to the data axis of the mesh (``("fsdp", "data")`` after ``("batch", "data")``) this stores
    parameters, gradients' final form and optimizer state sharded over the data-parallel
    ranks: weights are gathered for use and gradients reduced back to the owner's shard."""
    wsc = mm_lib.with_sharding_constraint
    layers = []
    for p in params["layers"]:
        layers.append({**p,
                       "wqkv": wsc(p["wqkv"], ("heads", None, "fsdp")),
                       "wo": wsc(p["wo"], ("fsdp", "heads")),
                       "wgu": wsc(p["wgu"], (None, "mlp", "fsdp")),
                       "wdown": wsc(p["wdown"], ("fsdp", "mlp"))})
    return {**params, "embed": wsc(params["embed"], ("fsdp", None)), "lm_head": wsc(params["lm_head"], ("fsdp", None)),
            "layers": layers}


def gather_fsdp(params: Dict[str, Any]) -> Dict[str, Any]:
    """The layout the layers compute with: the ``fsdp`` axis gathered, tensor-parallel axes kept.
    Called once per step, outside the microbatch loop, so the all-gather of the weights and
    the reduction of their gradients each happen once per step."""
    rl = mm_lib.relayout
    layers = []
    for p in params["layers"]:
        layers.append({**p,
                       "wqkv": rl(p["wqkv"], ("heads", None, None)),
                       "wo": rl(p["wo"], (None, "heads")),
                       "wgu": rl(p["wgu"], (None, "mlp", None)),
                       "wdown": rl(p["wdown"], (None, "mlp"))})
    return {**params, "embed": rl(params["embed"], (None, None)), "lm_head": rl(params["lm_head"], (None, None)),
            "layers": layers}


def make_train_step(cfg: LlamaConfig, opt: AdamWConfig, *, seq_len: int, global_batch: int, microbatch_size: int,
                    schedule: Optional[str] = "1f1b", grad_dtype: torch.dtype = torch.float32,
                    fsdp: bool = False) -> Callable:
    """Builds ``step(params, opt_state, tokens, labels, cos, sin) -> (loss, params, opt_state)``.

    The loss is the mean token cross-entropy over the global batch; gradients are summed
    over microbatches in ``grad_dtype`` accumulators; AdamW keeps fp32 master weights."""
    from torch.utils import _pytree as pytree
    loss_scale = 1.0 / float(global_batch * seq_len)

    def step(params, opt_state, tokens, labels, cos, sin):
        used = params
        if fsdp:
            params = annotate_fsdp(params)
            used = gather_fsdp(params)

        def mb_loss(p, batch):
            tok, lab = batch
            return loss_fn(cfg, p, tok, lab, cos, sin, loss_scale)

        vg = value_and_grad(mb_loss)
        if microbatch_size < global_batch:
            vg = microbatch(vg, dim=0, size=microbatch_size, argnum=1, schedule=schedule,
                            accumulate_dtype=grad_dtype)
        loss, grads = vg(used, (tokens, labels))
        with named_scope("optimizer"):
            new_step = opt_state["step"] + 1
            g_leaves, spec = pytree.tree_flatten(grads)
            p_leaves = pytree.tree_leaves(params)
            ma, mm_, vv = (pytree.tree_leaves(opt_state[k]) for k in ("master", "m", "v"))
            new_p, new_master, new_m, new_v = [], [], [], []
            for p0, g, a, b, c in zip(p_leaves, g_leaves, ma, mm_, vv):
                p2, a2, b2, c2 = ops.adamw(p0, a, b, c, g, new_step, opt.lr, opt.beta1, opt.beta2, opt.eps,
                                           opt.weight_decay, 1.0)
                new_p.append(p2)
                new_master.append(a2)
                new_m.append(b2)
                new_v.append(c2)
        new_params = pytree.tree_unflatten(new_p, spec)
        new_state = {"master": pytree.tree_unflatten(new_master, spec), "m": pytree.tree_unflatten(new_m, spec),
                     "v": pytree.tree_unflatten(new_v, spec), "step": new_step}
        return loss, new_params, new_state

    return step


def register_pipeline_tasks(cfg: LlamaConfig, mesh: MultiMesh, num_stages: int,
                            logical_axes: Sequence[Tuple[str, str]] = (("batch", "data"), ("heads", "model"),
                                                                       ("mlp", "model"), ("fsdp", "data"),
                                                                       ("expert", "data"),
                                                                       ("boundary_hidden", "model"),
                                                                       ("seq", "model"), ("vocab", "model")),
                            layers_per_stage: Optional[Sequence[int]] = None,
                            split_backprop: Optional[Tuple[str, str]] = None) -> None:
    """Places the layers on pipeline stages (mesh axis ``stage``): ``layers_per_stage[s]``
    consecutive layers on stage ``s`` (default: equal shares), the embedding on the first stage
    and the head / loss on the last one - which is why the last stage may be given fewer layers.
    The optimiser update of a parameter runs where its gradient lives. ``split_backprop``
    (two suffixes) splits every backward task into its activation-gradient and weight-gradient
    halves, which the zero-bubble schedule needs."""
    if layers_per_stage is None:
        per = cfg.n_layers // num_stages
        layers_per_stage = [per] * (num_stages - 1) + [cfg.n_layers - per * (num_stages - 1)]
    if len(layers_per_stage) != num_stages or sum(layers_per_stage) != cfg.n_layers:
        raise ValueError(f"layers_per_stage {list(layers_per_stage)} does not cover {cfg.n_layers} layers on {num_stages} stages")
    stage_of: List[int] = []
    for s_, cnt in enumerate(layers_per_stage):
        stage_of.extend([s_] * cnt)
    la = [(a, b) for a, b in logical_axes if b in mesh.axis_names]

    def layer_task(matched: str, backprop: bool) -> Task:
        idx = int(matched.split(".")[1])
        stage = stage_of[idx]
        return Task(name=f"stage{stage}" + ("_bwd" if backprop else ""), mesh_slice={"stage": stage}, logical_axes=la,
                    split_backprop=split_backprop)

    mesh.register_task(r"(layers\.\d+)", factory=layer_task)
    mesh.register_task("(embed)", factory=lambda m, b: Task(name="stage0" + ("_bwd" if b else ""),
                                                            mesh_slice={"stage": 0}, logical_axes=la,
                                                            split_backprop=split_backprop))
    last = num_stages - 1
    mesh.register_task("(head)", factory=lambda m, b: Task(name=f"stage{last}" + ("_bwd" if b else ""),
                                                           mesh_slice={"stage": last}, logical_axes=la,
                                                           split_backprop=split_backprop))
