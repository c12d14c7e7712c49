"""Tiny Llama on CPU: (1) the mm_ops model (forward + backward) against an independent plain
PyTorch implementation; (2) the MPMD-compiled training step (2 pipeline stages on 2 virtual
devices, microbatching, AdamW) against the eager single-device step."""
import math

import pytest
import torch
from torch.utils import _pytree as pytree

import multimesh_jax_b200 as mm
from multimesh_jax_b200.models import llama

torch.manual_seed(0)



LR = 1e-2      # learning rate of every AdamW step in this file


def _adam_close(got: torch.Tensor, want: torch.Tensor, lr: float):
    """Parameters after one AdamW step. Adam's first step is lr * sign(g) for every element, so an
    element whose gradient is zero up to rounding can land 2 * lr away when the summation order of
    the gradient differs; such elements must stay rare (< 0.2 %) and within 2.2 * lr, all others
    must agree to 1e-3."""
    diff = (got - want).abs()
    loose = diff > 1e-3 + 1e-3 * want.abs()
    assert float(diff.max()) <= 2.2 * lr + 1e-6, f"max difference {float(diff.max())}"
    assert int(loose.sum()) <= max(1, int(0.002 * diff.numel())), f"{int(loose.sum())} of {diff.numel()} elements differ"

def _cfg(**kw):
    cfg = llama.LlamaConfig.tiny(**kw)
    cfg.dtype = torch.float32
    return cfg


def _reference_loss(cfg, params, tokens, labels, scale):
    """Plain PyTorch restatement (HF-style rotate-half RoPE, SDPA attention)."""
    B, S = tokens.shape
    Dh = cfg.head_dim
    hq, hkv = cfg.n_heads, cfg.n_kv_heads
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, Dh, 2, dtype=torch.float64) / Dh))
    ang = torch.outer(torch.arange(S, dtype=torch.float64), inv)
    cos, sin = ang.cos().float(), ang.sin().float()

    def norm(x, w):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.eps) * w

    def rope(t):  # [B,S,H,Dh]
        a, b = t[..., : Dh // 2], t[..., Dh // 2:]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.cat([a * c - b * s, b * c + a * s], dim=-1)

    x = params["embed"][tokens]
    for p in params["layers"]:
        h = norm(x, p["attn_norm"])
        qkv = torch.einsum("bsd,hed->bshe", h, p["wqkv"])
        rep = hq // hkv
        grouped = qkv.view(B, S, hkv, rep + 2, Dh)  # per kv head: rep query heads, key, value
        q = grouped[:, :, :, :rep].reshape(B, S, hq, Dh)
        k, v = grouped[:, :, :, rep], grouped[:, :, :, rep + 1]
        q, k = rope(q), rope(k)
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                             is_causal=True).transpose(1, 2)
        x = x + o.reshape(B, S, -1) @ p["wo"].t()
        h = norm(x, p["ffn_norm"])
        gu = torch.einsum("bsd,gfd->bsgf", h, p["wgu"])
        x = x + (torch.nn.functional.silu(gu[:, :, 0]) * gu[:, :, 1]) @ p["wdown"].t()
    h = norm(x, params["final_norm"])
    logits = h @ params["lm_head"].t()
    return torch.nn.functional.cross_entropy(logits.view(B * S, -1), labels.view(-1), reduction="sum") * scale


@pytest.mark.parametrize("kv", [2, 1])
def test_ops_model_matches_plain_pytorch(kv):
    cfg = _cfg(n_heads=2, n_kv_heads=kv, d_model=64, d_ff=96, vocab=128)
    params = llama.init_params(cfg)
    B, S = 2, 16
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    scale = 1.0 / (B * S)
    vg = mm.value_and_grad(lambda p: llama.loss_fn(cfg, p, tokens, labels, cos, sin, scale))
    loss, grads = vg(params)
    ref_params = pytree.tree_map(lambda t: t.clone().requires_grad_(True), params)
    ref_loss = _reference_loss(cfg, ref_params, tokens, labels, scale)
    ref_grads = torch.autograd.grad(ref_loss, pytree.tree_leaves(ref_params))
    torch.testing.assert_close(loss, ref_loss.detach(), rtol=1e-4, atol=1e-5)
    for g, r in zip(pytree.tree_leaves(grads), ref_grads):
        torch.testing.assert_close(g, r, rtol=2e-3, atol=2e-5)


def _eager_step(step, params, opt_state, tokens, labels, cos, sin):
    with mm.ignore_transforms():
        return step(params, opt_state, tokens, labels, cos, sin)


@pytest.mark.parametrize("schedule", ["gpipe", "1f1b"])
def test_compiled_pipeline_step_matches_eager(schedule):
    cfg = _cfg(n_layers=4, n_heads=2, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    opt = llama.AdamWConfig(lr=1e-2)
    B, S, MB = 8, 16, 2
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, opt, seq_len=S, global_batch=B, microbatch_size=MB, schedule=schedule)
    mesh = mm.MultiMesh((2, 1), ("stage", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=2)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu",
                                  donate_argnums=(0, 1))
    names = {t["original_color"] for t in exe.plan["templates"]}
    assert {"stage0", "stage1", "stage0_bwd", "stage1_bwd"} <= names
    p_ref, s_ref = params, opt_state
    p_mm, s_mm = params, opt_state
    for it in range(3):
        loss_ref, p_ref, s_ref = _eager_step(step, p_ref, s_ref, tokens, labels, cos, sin)
        loss, p_mm, s_mm = exe(p_mm, s_mm, tokens, labels, cos, sin)
        torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
        for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
            # Adam divides by |g|: elements with a vanishing gradient amplify summation-order noise
            torch.testing.assert_close(a.full_tensor(), b, rtol=1e-3, atol=2e-4)
    # layers 0-1 live on device 0, layers 2-3 on device 1: weights never move
    for t in exe.plan["templates"]:
        if t["original_color"].startswith("stage0"):
            assert (t["device_start"], t["num_devices"]) == (0, 1)
        if t["original_color"].startswith("stage1"):
            assert (t["device_start"], t["num_devices"]) == (1, 1)
    exe.shutdown()


@pytest.mark.parametrize("pp,tp", [(1, 2), (2, 2)])
def test_tensor_parallel_step_matches_eager(pp, tp):
    """Heads and the FFN width are sharded over the `model` mesh axis of every stage (the
    compiler derives weight shardings, inserts the reductions of partial sums and hoists none
    of them out of the loop since no weight gradient is partial); results equal the eager step."""
    cfg = _cfg(n_layers=2 * pp, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    B, S, MB = 8, 16, 4
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB)
    mesh = mm.MultiMesh((pp, tp), ("stage", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, _ = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    keys = set()
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        torch.testing.assert_close(a.full_tensor(), b, rtol=1e-3, atol=2e-4)
        keys.add(a.sharding["key"].split("m(")[0])
    # projection weights really are sharded: packed heads, attention output, gate/up, down
    assert any(k.startswith("float32[8/0,16,64]") for k in keys)
    assert any(k.startswith("float32[64,64/0]") for k in keys)
    assert any(k.startswith("float32[2,96/0,64]") for k in keys)
    assert any(k.startswith("float32[64,96/0]") for k in keys)
    kinds = [exe.cap.graph.node(n)["op"] for t in exe.plan["templates"] for n in t["nodes"]]
    assert kinds.count("mm.all_reduce") >= 4 * pp
    exe.shutdown()


@pytest.mark.parametrize("axes,fsdp", [((1, 2, 1), False), ((1, 2, 2), False), ((1, 2, 2), True), ((2, 2, 2), True)])
def test_data_parallel_and_fsdp_steps_match_eager(axes, fsdp):
    """Data parallelism (batch over the `data` mesh axis, gradient reductions hoisted out of
    the microbatch loop) and its fully sharded form (parameters, gradients' final form and
    optimizer state stored sharded over `data`; weights gathered once per step before the loop,
    gradients reduced once after it), alone and combined with tensor and pipeline parallelism."""
    pp = axes[0]
    cfg = _cfg(n_layers=2 * pp, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    B, S, MB = 8, 16, 4
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB,
                                 fsdp=fsdp)
    mesh = mm.MultiMesh(axes, ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, s_ref = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, s_mm = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        _adam_close(a.full_tensor(), b, LR)
    for a, b in zip(pytree.tree_leaves(s_mm["m"]), pytree.tree_leaves(s_ref["m"])):
        torch.testing.assert_close(a.full_tensor(), b, rtol=1e-3, atol=1e-5)
    g = exe.cap.graph
    by_task = {}
    for t in exe.plan["templates"]:
        for n in t["nodes"]:
            op = g.node(n)["op"]
            if op in ("mm.all_reduce", "mm.reduce_scatter", "mm.spmd_reshard", "mm.relayout"):
                kind = "loop" if "_loop" in t["name"] else ("reduce" if t["name"].endswith("_reduce") else "other")
                by_task[(kind, op)] = by_task.get((kind, op), 0) + 1
    # every weight gradient is reduced over `data` once per step, after the loop
    hoisted = by_task.get(("reduce", "mm.all_reduce"), 0) + by_task.get(("reduce", "mm.reduce_scatter"), 0)
    assert hoisted >= 6 * cfg.n_layers
    if fsdp:
        # a rank only needs the gradient of the parameter shard it owns: the reductions of the
        # sharded weights are reduce-scatters (half the traffic of an all-reduce at two ranks)
        assert by_task.get(("reduce", "mm.reduce_scatter"), 0) >= 4 * cfg.n_layers
    else:
        assert by_task.get(("reduce", "mm.reduce_scatter"), 0) == 0
    w = p_mm["layers"][0]["wgu"]
    data_axis = 1 if axes[0] == 1 else 0   # index of `data` inside the stage's sub-mesh
    data_axis = list(mesh.slice(stage=0).axis_names).index("data")
    sharded_on_data = any(data_axis in ax for ax in w.sharding["dim_axes"])
    if fsdp:
        # stored sharded over data (ZeRO-3 style), as is the optimizer state; gathered before the loop
        assert sharded_on_data
        assert any(data_axis in ax for ax in s_mm["master"]["layers"][0]["wgu"].sharding["dim_axes"])
        assert by_task.get(("other", "mm.relayout"), 0) == 4 * cfg.n_layers + 2
        assert by_task.get(("loop", "mm.relayout"), 0) == 0
    else:
        assert not sharded_on_data
    exe.shutdown()


@pytest.mark.parametrize("fsdp", [False, True])
def test_optimizer_task_is_cut_into_pieces_behind_the_gradient_reductions(fsdp, monkeypatch):
    """With a bucket size below the gradient volume the post-loop update task becomes several
    `_update` tasks, each reading only the reductions of its own bucket (so that it can run
    while later reductions are still on the wire); the step still equals the eager one."""
    monkeypatch.setenv("MULTIMESH_UPDATE_BUCKET_BYTES", "40000")
    cfg = _cfg(n_layers=2, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    B, S, MB = 8, 16, 4
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB,
                                 fsdp=fsdp)
    mesh = mm.MultiMesh((1, 2, 1), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=1)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, s_ref = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, s_mm = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        _adam_close(a.full_tensor(), b, 1e-2)
    for a, b in zip(pytree.tree_leaves(s_mm["v"]), pytree.tree_leaves(s_ref["v"])):
        torch.testing.assert_close(a.full_tensor(), b, rtol=1e-3, atol=1e-6)
    g = exe.cap.graph
    updates = [t for t in exe.plan["templates"] if t["name"].endswith("_update")]
    reduces = {t["id"] for t in exe.plan["templates"] if t["name"].endswith("_reduce")}
    assert len(updates) >= 3
    producer_template = {}
    for t in exe.plan["templates"]:
        for v in t["outputs"]:
            producer_template[v] = t["id"]
    seen = set()
    for t in updates:
        fed_by = {producer_template[v] for v in t["inputs"] if producer_template.get(v) in reduces}
        assert fed_by and not (fed_by & seen)        # its own reductions, nobody else's
        seen |= fed_by
        assert all(g.node(n)["op"].startswith("mm_ops.adamw") for n in t["nodes"])
    # the pieces are submitted in the order of the reductions that feed them
    order = [op["template"] for op in exe.plan["ops"] if op["kind"] == "task"]
    first_reduce_of = {t["id"]: min(order.index(producer_template[v]) for v in t["inputs"] if producer_template.get(v) in reduces)
                       for t in updates}
    by_submission = sorted(updates, key=lambda t: order.index(t["id"]))
    assert [first_reduce_of[t["id"]] for t in by_submission] == sorted(first_reduce_of.values())
    exe.shutdown()


def test_forced_layout_change_at_the_stage_boundary():
    """Two stages of (data 2 x model 2) devices with parameters stored FSDP-style; the first
    stage hands its output over sharded on the hidden dimension, the second takes it sharded on
    the batch: every microbatch crosses the boundary through a reshard that changes the layout."""
    cfg = _cfg(n_layers=4, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    cfg.hidden_sharded_after = (1,)
    B, S, MB = 8, 16, 4
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB,
                                 fsdp=True)
    mesh = mm.MultiMesh((2, 2, 2), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=2)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, _ = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        _adam_close(a.full_tensor(), b, LR)
    plan = exe.plan
    crossings = []
    for op in plan["ops"]:
        if op["kind"] != "reshard":
            continue
        s_, d_ = plan["stores"][op["src_store"]]["shape"], plan["stores"][op["dst_store"]]["shape"]
        if s_["device_start"] == 0 and d_["device_start"] == 4 and s_["sizes"] == [MB, S, 64]:
            crossings.append((s_["dim_axes"], d_["dim_axes"]))
    # two values (residual stream and its normalised copy) per microbatch, hidden-sharded -> batch-sharded
    assert len(crossings) == 2 * (B // MB)
    assert all(src == [[], [], [1]] and dst == [[0], [], []] for src, dst in crossings)
    exe.shutdown()


def test_zero_bubble_schedule_on_four_llama_stages():
    """Both values that cross a stage boundary backwards (gradients of the residual stream and of
    its normalised copy) stay in the activation-gradient half of the split backward task; the
    weight-gradient halves are non-critical and results equal the eager step."""
    cfg = _cfg(n_layers=4, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128)
    B, S, MB = 16, 16, 2
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB,
                                 schedule="zero-bubble-h2")
    mesh = mm.MultiMesh((4, 1, 1), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=4, split_backprop=("_act", "_wgt"))
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, _ = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        _adam_close(a.full_tensor(), b, LR)
    loop = [t for t in exe.plan["templates"] if t["in_loop"]]
    producer = {v: t["name"] for t in loop for v in t["outputs"]}
    noncritical = {t["name"] for t in loop if t["noncritical"]}
    assert len(noncritical) == 3                  # stages 1..3; stage 0 has no activation gradient to hand on
    for t in loop:
        if not t["noncritical"]:                  # nothing on the critical path waits for a weight-gradient task
            assert not any(producer.get(v) in noncritical for v in t["inputs"])
    exe.shutdown()


@pytest.mark.parametrize("pp,dp,tp,vocab", [(1, 1, 2, False), (1, 1, 2, True), (2, 2, 2, True), (1, 1, 4, True)])
def test_sequence_parallel_tensor_parallel_step_matches_eager(pp, dp, tp, vocab):
    """Sequence-parallel layout of the tensor-parallel region: the residual stream and the norms
    are sharded on the sequence over the `model` axis; the compiler turns "partial projection ->
    all-reduce -> slice" into reduce-scatters and the layout changes in front of the column-
    parallel projections into all-gathers, and the lowering fuses each of them into the GEMM
    beside it. With a vocabulary-sharded output projection the loss exchanges its softmax
    statistics instead of gathering the logits. Results equal the eager step."""
    import collections
    cfg = _cfg(n_layers=2 * pp, n_heads=4, n_kv_heads=4 if tp > 2 else 2, d_model=64, d_ff=96, vocab=128)
    cfg.sequence_parallel = True
    cfg.vocab_parallel = vocab
    B, S, MB = 8, 16, 4
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=LR), seq_len=S, global_batch=B, microbatch_size=MB)
    mesh = mm.MultiMesh((pp, dp, tp), ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, _ = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        _adam_close(a.full_tensor(), b, LR)
    g = exe.cap.graph
    loop_ops, kinds = collections.Counter(), collections.Counter()
    for t in exe.plan["templates"]:
        if "_loop" in t["name"]:
            loop_ops.update(g.node(n)["op"] for n in t["nodes"])
            kinds.update(i.kind for i in exe.programs[t["id"]].instrs)
    layers = cfg.n_layers
    # per layer: attention-out and FFN-down forward, QKV and gate/up input gradients (+ the head's)
    assert loop_ops["mm.reduce_scatter"] >= 4 * layers
    assert loop_ops["mm.all_reduce"] == 0                  # no activation is all-reduced any more
    gathers = sum(1 for t in exe.plan["templates"] for n in t["nodes"] if "gather_dim" in g.node(n)["attrs"])
    assert gathers >= 4 * layers
    # the lowering fused them: kind 10 = GEMM + reduce-scatter, kind 11 = all-gather + GEMM
    assert kinds[10] >= 4 * layers and kinds[11] >= 4 * layers
    assert kinds[9] == 0
    if vocab:
        # the logits are never gathered: their only consumer is the loss operator in its exchanging form
        assert kinds[8] >= pp // pp
        head = [s_ for s_ in exe.output_shardings()][0]
        assert head is not None
    log = "\n".join(exe.plan.get("log", []))
    assert "collective folding" in log
    exe.shutdown()
