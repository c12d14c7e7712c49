"""Kernel programs of the native task launcher, built (not launched) on a machine without a GPU."""
import torch

import multimesh_jax_b200 as mm
from multimesh_jax_b200.compiler.native import build_native
from multimesh_jax_b200.models import llama


def _pp2_plan():
    cfg = llama.LlamaConfig.tiny(n_layers=4, n_heads=1, n_kv_heads=1, d_model=128, d_ff=256, vocab=256)
    cfg.dtype = torch.bfloat16
    B, S, MB = 8, 128, 2
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB,
                                 schedule="1f1b")
    mesh = mm.MultiMesh((2, 1), ("stage", "model"))
    llama.register_pipeline_tasks(cfg, mesh, num_stages=2)
    with mesh:
        return mm.compile_function(step, (params, opt_state, tokens, tokens, cos, sin), mesh=mesh, backend="cpu",
                                   donate_argnums=(0, 1))


def test_outputs_read_by_a_reshard_are_written_into_an_external_tile_without_a_copy():
    exe = _pp2_plan()
    plan = exe.plan
    sources = {op["src_store"] for op in plan["ops"] if op["kind"] == "reshard"}
    assert sources
    seen_ext = 0
    for t in plan["templates"]:
        if not t["name"].endswith("_loop"):
            continue
        ops = [op for op in plan["ops"] if op["kind"] == "task" and op["template"] == t["id"]]
        ext = None
        for op in ops:
            here = {k for k, (sid, m) in enumerate(zip(op["outputs"], op["accumulate"])) if m == 0 and sid in sources}
            ext = here if ext is None else ext & here
        protect = sorted({i for op in ops for i, sid in enumerate(op["inputs"]) if sid in sources})
        modes = tuple(1 if m else 0 for m in ops[0]["accumulate"])
        prog = exe.programs[t["id"]]
        plain = build_native(exe.cap, plan, t, prog, modes, False)
        direct = build_native(exe.cap, plan, t, prog, modes, False, sorted(ext), protect)
        assert direct.external == sorted(ext)
        # the producer writes into the tile: no kernel call is added, the output block shrinks
        # by exactly the bytes that moved out of it
        assert direct.num_calls == plain.num_calls
        moved = 0
        for k in ext:
            spec = direct.outputs[k]
            assert spec[0] == "ext"
            n = spec[3].itemsize
            for e in spec[2]:
                n *= e
            moved += (n + 255) // 256 * 256
            seen_ext += 1
        assert plain.out_block_bytes - direct.out_block_bytes == moved
        assert [o[0] for i, o in enumerate(direct.outputs) if i not in ext] == \
               [o[0] for i, o in enumerate(plain.outputs) if i not in ext]
    assert seen_ext >= 3          # x and h forward, their cotangents backward
    exe.shutdown()


def test_fresh_outputs_are_carved_from_bounded_chunks(monkeypatch):
    from multimesh_jax_b200.compiler import native
    exe = _pp2_plan()
    plan = exe.plan
    t = next(t for t in plan["templates"] if t["name"].endswith("stage0_loop"))
    ops = [op for op in plan["ops"] if op["kind"] == "task" and op["template"] == t["id"]]
    modes = tuple(1 if m else 0 for m in ops[0]["accumulate"])
    whole = build_native(exe.cap, plan, t, exe.programs[t["id"]], modes, False)
    assert len(whole.out_chunks) == 1 and whole.out_chunks[0] == whole.out_block_bytes
    monkeypatch.setattr(native._Builder, "OUT_CHUNK", 256 << 10)
    split = build_native(exe.cap, plan, t, exe.programs[t["id"]], modes, False)
    assert len(split.out_chunks) > 1 and sum(split.out_chunks) == split.out_block_bytes
    # every chunk respects the bound unless it holds a single larger output
    sizes = {}
    for spec in split.outputs:
        if spec[0] != "block":
            continue
        _, chunk, off, shape, dtype = spec
        n = dtype.itemsize
        for e in shape:
            n *= e
        assert 0 <= chunk < len(split.out_chunks) and off + n <= split.out_chunks[chunk]
        sizes.setdefault(chunk, []).append(n)
    for chunk, total in enumerate(split.out_chunks):
        assert total <= (256 << 10) or len(sizes.get(chunk, ())) <= 1
    assert split.num_calls == whole.num_calls
    exe.shutdown()
