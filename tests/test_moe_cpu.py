"""Mixture-of-experts layer: the operator pair against autograd through a dense restatement,
and the compiled Mixtral-shaped step with expert parallelism (experts and tokens share the
`data` mesh axis; dispatch and combine run inside the task) against the eager step."""
import pytest
import torch
from torch.utils import _pytree as pytree

import multimesh_jax_b200 as mm
from multimesh_jax_b200.models import llama
from multimesh_jax_b200.ops import moe


def _dense_moe(x, wr, wgu, wdown, top_k):
    T, D = x.shape
    logits = x @ wr.t()
    topv, topi = logits.topk(top_k, dim=-1)
    gates = torch.softmax(topv, dim=-1)
    y = torch.zeros_like(x)
    for e in range(wgu.shape[0]):
        gu = torch.einsum("td,gfd->tgf", x, wgu[e])
        out = (torch.nn.functional.silu(gu[:, 0]) * gu[:, 1]) @ wdown[e].t()
        w = (gates * (topi == e)).sum(-1, keepdim=True)      # zero for tokens that did not pick e
        y = y + w * out
    return y


def test_moe_operator_matches_dense_autograd():
    torch.manual_seed(0)
    T, D, F, E, k = 24, 16, 20, 4, 2
    x = torch.randn(T, D, requires_grad=True)
    wr = torch.randn(E, D, requires_grad=True)
    wgu = (torch.randn(E, 2, F, D) * 0.3).requires_grad_(True)
    wdown = (torch.randn(E, D, F) * 0.3).requires_grad_(True)
    dy = torch.randn(T, D)
    y = moe.moe_ffn(x, wr, wgu, wdown, k)
    grads = torch.autograd.grad(y, (x, wr, wgu, wdown), dy)
    y_ref = _dense_moe(x, wr, wgu, wdown, k)
    grads_ref = torch.autograd.grad(y_ref, (x, wr, wgu, wdown), dy)
    torch.testing.assert_close(y, y_ref, rtol=1e-4, atol=1e-5)
    for g, r in zip(grads, grads_ref):
        torch.testing.assert_close(g, r, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("axes", [(1, 2, 1), (1, 4, 1), (2, 2, 2)])
def test_expert_parallel_step_matches_eager(axes):
    pp = axes[0]
    cfg = llama.LlamaConfig.tiny(n_layers=2 * pp, n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128,
                                 n_experts=4, top_k=2)
    cfg.dtype = torch.float32
    B, S, MB = 8, 16, 4
    torch.manual_seed(0)
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    labels = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB)
    mesh = mm.MultiMesh(axes, ("stage", "data", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp)
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, labels, cos, sin), mesh=mesh, backend="cpu")
    with mm.ignore_transforms():
        loss_ref, p_ref, _ = step(params, opt_state, tokens, labels, cos, sin)
    loss, p_mm, _ = exe(params, opt_state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), loss_ref, rtol=1e-4, atol=1e-5)
    for a, b in zip(pytree.tree_leaves(p_mm), pytree.tree_leaves(p_ref)):
        torch.testing.assert_close(a.full_tensor(), b, rtol=1e-3, atol=1e-3)
    # experts are spread over the data axis of every stage; the router is not
    data_axis = list(mesh.slice(stage=0).axis_names).index("data")
    assert p_mm["layers"][0]["wgu"].sharding["dim_axes"][0] == [data_axis]
    assert p_mm["layers"][0]["wdown"].sharding["dim_axes"][0] == [data_axis]
    assert p_mm["layers"][0]["router"].sharding["dim_axes"] == [[], []]
    g = exe.cap.graph
    shared = [g.node(n)["attrs"].get("shared_axes") for t in exe.plan["templates"] for n in t["nodes"]
              if g.node(n)["op"].startswith("mm_ops.moe_ffn")]
    assert shared and all(s == f"[{data_axis}]" for s in shared)
    exe.shutdown()


def test_mixtral_shape_parameter_count():
    cfg = llama.LlamaConfig.mixtral_8x7b()
    assert abs(cfg.num_params() / 1e9 - 46.7) < 0.5       # 8x7B has about 46.7 B parameters
    assert abs(cfg.active_params() / 1e9 - 12.9) < 0.5     # about 12.9 B of them touch each token


def test_expert_selection_is_total_for_nan_and_infinite_logits():
    """The dispatch kernel derives peer-memory offsets from the chosen experts, so the selection
    must yield valid, distinct experts whatever the logits are."""
    inf, nan = float("inf"), float("nan")
    logits = torch.tensor([[0.1, 0.7, 0.7, -0.2],          # tie: lowest index first
                           [nan, nan, nan, nan],           # nothing comparable
                           [-inf, -inf, -inf, -inf],
                           [nan, 0.3, -inf, nan],          # one finite logit only
                           [inf, 1.0, inf, 0.0]])
    idx, val = moe.select_experts(logits, 2)
    assert idx.tolist() == [[1, 2], [0, 1], [0, 1], [1, 0], [0, 2]]
    for row in idx.tolist():
        assert len(set(row)) == 2 and all(0 <= e < 4 for e in row)
    assert val[1].tolist() == [0.0, 0.0] and val[3].tolist() == [pytest.approx(0.3), 0.0]
    # on ordinary logits the rule is torch.topk
    torch.manual_seed(3)
    rnd = torch.randn(64, 8)
    idx, val = moe.select_experts(rnd, 2)
    topv, topi = rnd.topk(2, dim=-1)
    assert torch.equal(idx, topi) and torch.equal(val, topv)


@pytest.mark.parametrize("count", [0, 5, 64, 100])
def test_expert_functions_with_a_row_count_equal_the_exact_size_call(count):
    """The expert forward / backward over a receive region of fixed capacity with the number of
    live rows given as a tensor (the form the GPU path uses so that the host never reads the
    count) equals the same functions on exactly the live rows; rows behind the count may hold
    anything, including NaN."""
    from multimesh_jax_b200.ops.moe import _expert_bwd, _expert_fwd
    torch.manual_seed(count)
    cap, D, F = 128, 32, 48
    rows = torch.randn(cap, D)
    d_out = torch.randn(cap, D)
    wgu = torch.randn(2, F, D) * 0.2
    wdown = torch.randn(D, F) * 0.2
    rows[count:] = float("nan")
    d_out[count:] = float("nan")
    n = torch.tensor([count], dtype=torch.int32)
    out = torch.zeros(cap, D)
    _, _, out = _expert_fwd(rows.clone(), wgu, wdown, out=out, count=n)
    dwgu = torch.zeros(2, F, D)
    dwdown = torch.zeros(D, F)
    dx = torch.zeros(cap, D)
    _expert_bwd(rows.clone(), d_out.clone(), wgu, wdown, dx_out=dx, out=torch.zeros(cap, D), count=n, dwgu_out=dwgu,
                dwdown_out=dwdown)
    if count == 0:
        assert bool((dwgu == 0).all()) and bool((dwdown == 0).all())
        return
    _, _, ref_out = _expert_fwd(rows[:count].contiguous(), wgu, wdown)
    ref_dx, ref_dwgu, ref_dwdown, _ = _expert_bwd(rows[:count].contiguous(), d_out[:count].contiguous(), wgu, wdown)
    torch.testing.assert_close(out[:count], ref_out, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dx[:count], ref_dx, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dwgu, ref_dwgu, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(dwdown, ref_dwdown, rtol=1e-4, atol=1e-5)
