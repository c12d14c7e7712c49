"""Host cost of a training step: the native task launcher against the interpreted task bodies.

    python benchmarks/bench_host.py [--layers 4] [--microbatches 8] [--steps 20]

A small Llama-shaped model (d_model 256, sequence 128) makes the GPU work per task a few hundred
microseconds, so the wall-clock time of a step is what the host needs to submit it. The same
step is compiled twice - task bodies as native kernel programs (one call into the C++ launcher
per task) and as interpreted programs (one Python call per kernel) - and timed after warm-up
with a device synchronisation on both sides. One JSON line: host microseconds per step and per
task for both forms, kernel launches per step, and the ratio.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--steps", type=int, default=20)
    ns = ap.parse_args()
    import multimesh_jax_b200 as mm
    from multimesh_jax_b200.models import llama
    from multimesh_jax_b200.ops import kernels as K

    torch.manual_seed(0)
    cfg = llama.LlamaConfig.tiny(n_layers=ns.layers, d_model=256, n_heads=2, n_kv_heads=2, d_ff=512, vocab=512)
    MB, S = 2, 128
    B = MB * ns.microbatches
    step = llama.make_train_step(cfg, llama.AdamWConfig(lr=1e-3), seq_len=S, global_batch=B, microbatch_size=MB)
    tokens = torch.randint(0, cfg.vocab, (B, S), device="cuda")
    cos, sin = llama.rope_tables(cfg, S, "cuda")
    out = {"layers": ns.layers, "microbatches": ns.microbatches, "steps": ns.steps}
    for native in (True, False):
        os.environ["MM_NATIVE_TASKS"] = "1" if native else "0"
        params = llama.init_params(cfg, device="cuda")
        state = llama.init_opt_state(params)
        mesh = mm.MultiMesh((1, 1), ("stage", "model"))
        llama.register_pipeline_tasks(cfg, mesh, num_stages=1)
        with mesh:
            exe = mm.compile_function(step, (params, state, tokens, tokens, cos, sin), mesh=mesh, backend="cuda",
                                      donate_argnums=(0, 1))
        for _ in range(3):
            loss, params, state = exe(params, state, tokens, tokens, cos, sin)
        torch.cuda.synchronize()
        k0, l0 = K.launch_count, exe.launches
        t0 = time.perf_counter()
        for _ in range(ns.steps):
            loss, params, state = exe(params, state, tokens, tokens, cos, sin)
        host = time.perf_counter() - t0          # submission only: nothing waits for the GPU
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        tasks = (exe.launches - l0) / ns.steps
        key = "native" if native else "interpreted"
        out[key] = {"host_us_per_step": round(host / ns.steps * 1e6, 1), "wall_us_per_step": round(wall / ns.steps * 1e6, 1),
                    "tasks_per_step": tasks, "host_us_per_task": round(host / ns.steps / max(tasks, 1) * 1e6, 1),
                    "kernel_launches_per_step": (K.launch_count - k0) / ns.steps,
                    "native_task_launches_per_step": getattr(exe, "native_launches", 0) / (ns.steps + 3),
                    "loss": float(loss.full_tensor().item())}
        exe.wait()
        exe.shutdown()
    out["host_time_ratio_interpreted_over_native"] = round(out["interpreted"]["host_us_per_step"] / out["native"]["host_us_per_step"], 2)
    out["kernel_status"] = K.read_status()
    print(json.dumps(out), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
