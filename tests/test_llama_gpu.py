"""GPU: the mm_ops Llama (bf16, our CUDA kernels) against the fp32 CPU restatement, and the
compiled training step against the eager one."""
import pytest
import torch
from torch.utils import _pytree as pytree

import multimesh_jax_b200 as mm
from multimesh_jax_b200.models import llama
from multimesh_jax_b200.ops import kernels as K

pytestmark = pytest.mark.gpu


def test_model_grads_match_fp32_reference():
    torch.manual_seed(0)
    cfg = llama.LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=1, d_ff=512, vocab=512)
    B, S = 2, 256
    params = llama.init_params(cfg, device="cuda")
    tokens = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    labels = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    cos, sin = llama.rope_tables(cfg, S, "cuda")
    scale = 1.0 / (B * S)
    loss, grads = mm.value_and_grad(lambda p: llama.loss_fn(cfg, p, tokens, labels, cos, sin, scale))(params)
    cfg32 = llama.LlamaConfig(**{**cfg.__dict__, "dtype": torch.float32})
    p32 = pytree.tree_map(lambda t: t.float().cpu(), params)
    c32, s32 = llama.rope_tables(cfg32, S, "cpu")
    ref_loss, ref_grads = mm.value_and_grad(
        lambda p: llama.loss_fn(cfg32, p, tokens.cpu(), labels.cpu(), c32, s32, scale))(p32)
    assert K.read_status() == 0
    torch.testing.assert_close(loss.cpu(), ref_loss, rtol=2e-2, atol=2e-2)
    for g, r in zip(pytree.tree_leaves(grads), pytree.tree_leaves(ref_grads)):
        err = (g.float().cpu() - r).norm() / (r.norm() + 1e-12)
        assert err < 5e-2, f"relative gradient error {err}"


def test_compiled_step_matches_eager_on_gpu():
    torch.manual_seed(1)
    cfg = llama.LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=2, d_ff=512, vocab=512)
    B, S, MB = 4, 128, 2
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-3), seq_len=S, global_batch=B, microbatch_size=MB)
    params = llama.init_params(cfg, device="cuda")
    state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    labels = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    cos, sin = llama.rope_tables(cfg, S, "cuda")
    mesh = mm.MultiMesh((1, 1), ("stage", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=1)
    with mesh:
        exe = mm.compile_function(step, (params, state, tokens, labels, cos, sin), mesh=mesh, backend="cuda")
    with mm.ignore_transforms():
        ref_loss, ref_params, _ = step(params, state, tokens, labels, cos, sin)
    loss, new_params, _ = exe(params, state, tokens, labels, cos, sin)
    torch.testing.assert_close(loss.full_tensor(), ref_loss, rtol=2e-2, atol=2e-2)
    for a, b in zip(pytree.tree_leaves(new_params), pytree.tree_leaves(ref_params)):
        torch.testing.assert_close(a.full_tensor().float(), b.float(), rtol=2e-2, atol=2e-3)
    assert K.read_status() == 0
    exe.shutdown()


def test_expired_kernel_wait_fails_the_step_and_the_next_step_runs():
    """A bounded device wait that runs out during a step (here: a flag that nothing raises, with a
    300 ms limit, queued behind the step's kernels) is reported when the step is awaited -
    ``StepFailed`` naming the status code - and the status is cleared, so the next step is clean."""
    from multimesh_jax_b200.parallel import symm
    torch.manual_seed(2)
    cfg = llama.LlamaConfig.tiny(n_layers=1, d_model=256, n_heads=2, n_kv_heads=2, d_ff=512, vocab=512)
    B, S = 2, 128
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-3), seq_len=S, global_batch=B, microbatch_size=B)
    params = llama.init_params(cfg, device="cuda")
    state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    cos, sin = llama.rope_tables(cfg, S, "cuda")
    mesh = mm.MultiMesh((1, 1), ("stage", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=1)
    with mesh:
        exe = mm.compile_function(step, (params, state, tokens, tokens, cos, sin), mesh=mesh, backend="cuda")
    K.read_status()
    arena = symm.SymmetricArena(1 << 20, torch.device("cuda", 0))
    off = arena.alloc_flag()
    loss, p1, s1 = exe(params, state, tokens, tokens, cos, sin)
    symm.wait_flags(arena, [arena.flag_ptr(arena.rank, off)], 1, limit_ms=300)   # expires: nothing raises it
    with pytest.raises(mm.StepFailed, match="kernel status 5"):
        exe.wait()
    loss2, p2, s2 = exe(params, state, tokens, tokens, cos, sin)
    exe.wait()                                                                   # clean again
    assert torch.isfinite(loss2.full_tensor()).all()
    arena.close()
    exe.shutdown()


def test_transformer_tasks_run_as_native_kernel_programs_and_match_the_interpreted_path(monkeypatch):
    """On a CUDA device the forward, backward and optimizer tasks of the model are kernel programs
    replayed by the C++ launcher (one call per task, memory planned ahead); the results are those
    of the interpreted programs."""
    torch.manual_seed(3)
    cfg = llama.LlamaConfig.tiny(n_layers=2, d_model=256, n_heads=2, n_kv_heads=2, d_ff=512, vocab=512)
    B, S, MB = 4, 128, 2
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-3), seq_len=S, global_batch=B, microbatch_size=MB)
    params = llama.init_params(cfg, device="cuda")
    state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    labels = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    cos, sin = llama.rope_tables(cfg, S, "cuda")
    args = (params, state, tokens, labels, cos, sin)

    def run(native: bool):
        monkeypatch.setenv("MM_NATIVE_TASKS", "1" if native else "0")
        mesh = mm.MultiMesh((1, 1), ("stage", "model"))
        llama.register_pipeline_tasks(cfg, mesh, num_stages=1)
        with mesh:
            exe = mm.compile_function(step, args, mesh=mesh, backend="cuda")
        loss, p1, s1 = exe(*args)
        loss2, p2, s2 = exe(p1, s1, tokens, labels, cos, sin)       # second step: accumulators exist, tiles are re-bound
        out = (loss.full_tensor().clone(), loss2.full_tensor().clone(),
               [t.full_tensor().clone() for t in pytree.tree_leaves(p2)],
               [t.full_tensor().clone() for t in pytree.tree_leaves(s2["m"])])
        report, launches, scratch = exe.native_report(), exe.native_launches, getattr(exe, "native_scratch_bytes", 0)
        exe.wait()
        exe.shutdown()
        return out, report, launches, scratch

    nat, report, launches, scratch = run(True)
    assert all(v.startswith("native") for k, v in report.items()), report
    assert launches >= 2 * (2 * (B // MB) + 1) and scratch > 0
    ref, report0, launches0, _ = run(False)
    assert launches0 == 0 and all(v.startswith("interpreted") for v in report0.values())
    torch.testing.assert_close(nat[0], ref[0], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(nat[1], ref[1], rtol=1e-5, atol=1e-6)
    for a, b in zip(nat[2] + nat[3], ref[2] + ref[3]):
        torch.testing.assert_close(a.float(), b.float(), rtol=1e-3, atol=1e-5)
    assert K.read_status() == 0


def test_smoke_entry_point_runs():
    """The repository's smoke entry (one tiny training step through the MPMD compiler, native
    task programs and the CUDA runtime context) finishes with a finite loss and a clean status."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("graft_entry", os.path.join(root, "__graft_entry__.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.smoke()
