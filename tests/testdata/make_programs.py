"""Writes the stored-program fixtures of this directory and their expected compile summaries.

    python tests/testdata/make_programs.py            # rewrite every fixture
    python tests/testdata/make_programs.py --check    # recompile the stored files and print the summaries

Each fixture is a training step of one of the in-tree model families captured on a small shape
under one parallel layout, stored before partitioning (``compile_function(save_program=...)``).
``tests/test_stored_programs.py`` compiles the files offline (no model code, no tensors, no
device) and compares the result with ``expected.json``: a change in the compiler that alters the
plan of a real-model graph shows up there, and this script regenerates the expectations once the
change is understood. The role of the 50 HLO text fixtures of the reference
(src/pjrt_client/testdata/*.txt).
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import multimesh_jax_b200 as mm  # noqa: E402
from multimesh_jax_b200 import _mm_C  # noqa: E402
from multimesh_jax_b200.models import llama  # noqa: E402
from multimesh_jax_b200.runtime.collectives import Topology  # noqa: E402

# name -> (pp, dp, tp), schedule, model options, step options
FIXTURES = {
    "llama_pp2_tp2_1f1b": ((2, 1, 2), "1f1b", {}, {}),
    "llama_pp4_zero_bubble": ((4, 1, 1), "zero-bubble-h2", {}, {}),
    "llama_dp2_fsdp": ((1, 2, 1), "1f1b", {}, {"fsdp": True}),
    "llama_tp2_sequence_parallel": ((1, 1, 2), "1f1b", {"sequence_parallel": True, "vocab_parallel": True}, {}),
    "llama_pp2_dp2_tp2_gpipe": ((2, 2, 2), "gpipe", {}, {}),
    "mixtral_ep2_pp2": ((2, 2, 1), "1f1b", {"n_experts": 4, "top_k": 2}, {}),
    "llama_tp2_all_reduce": ((1, 1, 2), "1f1b", {}, {}),
    "llama_pp2_dp2_fsdp_zero_bubble": ((2, 2, 1), "zero-bubble-h2", {}, {"fsdp": True}),
    "llama_pp4_uneven_stages_1f1b": ((4, 1, 1), "1f1b", {"n_layers": 6, "layers_per_stage": [2, 2, 1, 1]}, {}),
    "llama_one_device_microbatched": ((1, 1, 1), "1f1b", {}, {}),
}
SUMMARY_KEYS = ("status", "message", "hazards", "plan_hash", "templates", "template_names", "stores", "tasks", "reshards",
                "reshard_bytes", "temp_bytes_per_device_max", "device_high_water_max", "device_high_water", "stats")


def capture(name: str, path: str) -> None:
    (pp, dp, tp), schedule, model_opts, step_opts = FIXTURES[name]
    n = pp * dp * tp
    torch.manual_seed(0)
    moe = {k: model_opts[k] for k in ("n_experts", "top_k") if k in model_opts}
    cfg = llama.LlamaConfig.tiny(n_layers=model_opts.get("n_layers", 2 * pp), n_heads=4, n_kv_heads=2, d_model=64, d_ff=96, vocab=128, **moe)
    cfg.dtype = torch.float32
    cfg.sequence_parallel = model_opts.get("sequence_parallel", False)
    cfg.vocab_parallel = model_opts.get("vocab_parallel", False)
    B, S, MB = 8 * dp, 16, 2 * dp
    params = llama.init_params(cfg)
    opt_state = llama.init_opt_state(params)
    tokens = torch.randint(0, cfg.vocab, (B, S))
    cos, sin = llama.rope_tables(cfg, S, "cpu")
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-2), seq_len=S, global_batch=B, microbatch_size=MB,
                                 schedule=schedule, **step_opts)
    mesh = mm.MultiMesh((pp, dp, tp), ("stage", "data", "model"))
    split = ("_act", "_wgt") if schedule == "zero-bubble-h2" else None
    llama.register_pipeline_tasks(cfg, mesh, num_stages=pp, split_backprop=split,
                                  layers_per_stage=model_opts.get("layers_per_stage"))
    with mesh:
        exe = mm.compile_function(step, (params, opt_state, tokens, tokens, cos, sin), mesh=mesh,
                                  context=_mm_C.MockContext(n), topology=Topology("cpu", n), donate_argnums=(0, 1),
                                  save_program=path)
    exe.shutdown()


def summary(path: str) -> dict:
    r = mm.compile_program_file(path)
    return {k: r[k] for k in SUMMARY_KEYS}


def main() -> int:
    check = "--check" in sys.argv[1:]
    expected = {}
    for name in FIXTURES:
        path = os.path.join(HERE, name + ".mmprog.json")
        if not check:
            capture(name, path)
        expected[name] = summary(path)
        print(name, os.path.getsize(path) >> 10, "KiB", {k: expected[name][k] for k in ("templates", "tasks", "reshards", "device_high_water_max")})
    if not check:
        with open(os.path.join(HERE, "expected.json"), "w") as f:
            json.dump(expected, f, indent=1, sort_keys=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
