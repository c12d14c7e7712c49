#!/usr/bin/env python
"""Headline benchmark: training tokens/s of a Llama-2-7B-shape decoder (bf16, seq 2048,
AdamW, random init, synthetic token ids) through the MPMD compiler and runtime.

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Weak scaling: 8 sequences of 2048 tokens per GPU and step (global batch 64 at N = 8, the
configuration named by the baseline), microbatches of 4 sequences per data-parallel rank.
Default layouts: N = 1 single device; N = 2 tensor parallel with sequence-sharded activations
(GEMM + reduce-scatter and all-gather + GEMM kernels; the fastest measured layout on 2 GPUs); N = 4 four pipeline stages with
the zero-bubble-H2 schedule (the fastest measured layout on 4 GPUs); N = 8 the layout the
baseline names, 4 pipeline stages x tensor parallel 2, 1F1B with 16 microbatches. --pp / --dp / --tp / --fsdp / --force-reshard / --model select the others
(Llama-3-8B with FSDP and a layout-changing stage boundary, Mixtral-8x7B with expert
parallelism over the data axis).

Prints ONE JSON line (rank 0). `value` is device-timed (CUDA events around exactly K steps,
barrier + synchronize on both sides, max over ranks); `e2e` repeats the measurement with the
per-step host->device copy of that step's token ids from pinned memory and a device->host
read of the loss inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

# one growing segment per stream instead of many fixed-size blocks: the step's large, short-lived
# activations would otherwise fragment the caching allocator at this model size
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import torch  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKENS_PER_S = None  # the reference publishes no number for this metric


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="llama2_7b", choices=["llama2_7b", "llama3_8b", "mixtral_8x7b", "tiny"])
    p.add_argument("--seq", type=int, default=2048)
    p.add_argument("--per-gpu-batch", type=int, default=8)
    p.add_argument("--microbatch", type=int, default=4)
    p.add_argument("--layers", type=int, default=0, help="override the number of layers (debugging only)")
    p.add_argument("--tp", type=int, default=0, help="tensor-parallel degree (0 = default for N)")
    p.add_argument("--dp", type=int, default=0, help="data-parallel degree (0 = default for N)")
    p.add_argument("--pp", type=int, default=0, help="pipeline stages (0 = N / (tp * dp))")
    p.add_argument("--fsdp", action="store_true", help="store parameters and optimizer state sharded over the data axis")
    p.add_argument("--sp", type=int, default=-1,
                   help="1: sequence-parallel layout of the tensor-parallel region (GEMM + reduce-scatter and "
                        "all-gather + GEMM kernels, vocabulary-sharded output projection and loss); 0: replicated "
                        "activations with GEMM + all-reduce; -1: on whenever the tensor-parallel degree is above 1")
    p.add_argument("--force-reshard", action="store_true",
                   help="stage outputs leave sharded on the hidden dimension and enter the next stage sharded on "
                        "the batch, so every microbatch crosses the boundary through a layout-changing reshard")
    p.add_argument("--layers-per-stage", default="",
                   help="comma-separated layer counts per pipeline stage (default: the last stage, which also "
                        "runs the LM head and the loss, gets two layers fewer when there are four stages)")
    p.add_argument("--schedule", default="",
                   help="microbatch schedule: 1f1b, gpipe, zero-bubble-h2 (split backward tasks) or auto (zero-bubble-h2 "
                        "when there are pipeline stages, with 1f1b as the fallback); empty = the default of the layout")
    p.add_argument("--plan-only", action="store_true",
                   help="compile the step for --gpus virtual devices on the mock runtime (no CUDA device is "
                        "touched, nothing is allocated), print the plan's statistics as one JSON line and exit")
    p.add_argument("--trace", default="", help="after the timed runs, profile one more step per rank and write "
                                               "its time breakdown to this directory (not a benchmark value)")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def default_layout(n: int):
    """(pipeline stages, data parallel, tensor parallel, schedule) used when no layout flag is given:
    the fastest measured layout per GPU count, except at 8 GPUs where the named layout and schedule
    are kept - 4 stages x TP2, 1F1B with 16 microbatches."""
    return {1: (1, 1, 1, "1f1b"), 2: (1, 1, 2, "1f1b"), 4: (4, 1, 1, "zero-bubble-h2"),
            8: (4, 1, 2, "1f1b")}.get(n, (1, n, 1, "1f1b"))


def default_layers_per_stage(n_layers: int, pp: int, schedule: str):
    """Measured on 4 GPUs (PP4, 8 microbatches, tokens/s): under 1F1B the last stage, which also owns
    the output projection and the loss, wants fewer layers and the extra layer sits best on an
    early stage - 8/9/8/7 77,288, 9/8/8/7 76,159, 8/9/9/6 74,606, 8/8/9/7 72,237, 8/8/8/8 71,804;
    zero-bubble runs 4.8 % faster with equal shares (None)."""
    if pp == 4 and n_layers % 4 == 0 and n_layers >= 16 and schedule == "1f1b":
        q = n_layers // 4
        return [q, q + 1, q, q - 1]
    return None


def main():
    args = parse_args()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return 0
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference cannot be installed offline: its build needs scikit-build, JAX/jaxlib patches, "
                          "Bazel and network fetches of OpenXLA, zuku and Legion (pip: ModuleNotFoundError: skbuild)"}))
        return 0

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    n = args.gpus
    if world != n and not (world == 1 and n == 1) and not args.plan_only:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n}")
    import multimesh_jax_b200 as mm
    from multimesh_jax_b200.models import llama
    from multimesh_jax_b200.ops import kernels as K
    if not args.plan_only:
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
        if n > 1:
            mm.init(gpus=n, distributed=True)
    import torch.distributed as dist

    cfg = {"llama2_7b": llama.LlamaConfig.llama2_7b, "llama3_8b": llama.LlamaConfig.llama3_8b,
           "mixtral_8x7b": llama.LlamaConfig.mixtral_8x7b, "tiny": llama.LlamaConfig.tiny}[args.model]()
    if args.layers:
        cfg.n_layers = args.layers
    if args.tp or args.dp or args.pp:
        tp, dp = args.tp or 1, args.dp or 1
        pp = args.pp or n // (tp * dp)
        default_schedule = "1f1b"
    else:
        pp, dp, tp, default_schedule = default_layout(n)
    args.schedule = args.schedule or default_schedule
    if pp * dp * tp != n:
        raise SystemExit(f"pp{pp} x dp{dp} x tp{tp} != {n} GPUs")
    sp = (tp > 1 and not cfg.n_experts and not args.force_reshard) if args.sp < 0 else bool(args.sp)
    cfg.sequence_parallel = cfg.vocab_parallel = sp
    if args.force_reshard and pp > 1:
        per_stage = cfg.n_layers // pp
        cfg.hidden_sharded_after = tuple(s * per_stage - 1 for s in range(1, pp))
        if not args.layers_per_stage:
            args.layers_per_stage = ",".join([str(per_stage)] * pp)   # boundaries above assume equal shares
    seq = args.seq
    global_batch = args.per_gpu_batch * n
    mb = min(args.microbatch * dp, global_batch)   # --microbatch counts sequences per data-parallel rank
    opt = llama.AdamWConfig()
    if args.layers_per_stage:
        lps = [int(v) for v in args.layers_per_stage.split(",")]
    else:
        lps = default_layers_per_stage(cfg.n_layers, pp, args.schedule)

    # abstract arguments for the capture; real tensors are created shard by shard below
    with torch.device("meta"):
        a_params = llama.init_params(cfg, device="meta")
        a_state = llama.init_opt_state(a_params)
    a_tok = torch.empty(global_batch, seq, dtype=torch.int64, device="meta")
    a_cos = torch.empty(seq, cfg.head_dim // 2, dtype=torch.float32, device="meta")

    def compile_with(schedule):
        step_fn = llama.make_train_step(cfg, opt, seq_len=seq, global_batch=global_batch, microbatch_size=mb,
                                        schedule=schedule, fsdp=args.fsdp)
        mesh = mm.MultiMesh((pp, dp, tp), ("stage", "data", "model"))
        split = ("_act", "_wgt") if schedule == "zero-bubble-h2" else None
        llama.register_pipeline_tasks(cfg, mesh, num_stages=pp, layers_per_stage=lps, split_backprop=split)
        with mesh:
            if args.plan_only:
                from multimesh_jax_b200 import _mm_C
                from multimesh_jax_b200.runtime.collectives import Topology
                return mm.compile_function(step_fn, (a_params, a_state, a_tok, a_tok, a_cos, a_cos), mesh=mesh,
                                           donate_argnums=(0, 1), context=_mm_C.MockContext(n),
                                           topology=Topology("cpu", n), name="train_step")
            return mm.compile_function(step_fn, (a_params, a_state, a_tok, a_tok, a_cos, a_cos), mesh=mesh,
                                       donate_argnums=(0, 1), backend="dist" if n > 1 else "cuda", name="train_step")

    t0 = time.time()
    if args.schedule == "auto":
        # the plan is a pure function of the program, so every rank takes the same branch
        args.schedule = "zero-bubble-h2" if pp > 1 else "1f1b"
        try:
            exe = compile_with(args.schedule)
        except Exception as e:  # noqa: BLE001 - fall back to the plain pipeline schedule
            if pp == 1:
                raise
            print(f"[bench] zero-bubble-h2 did not compile ({type(e).__name__}: {e}); using 1f1b", file=sys.stderr)
            args.schedule = "1f1b"
            exe = compile_with(args.schedule)
    else:
        exe = compile_with(args.schedule)
    compile_s = time.time() - t0
    if args.plan_only:
        plan = exe.plan
        print(json.dumps({"plan_only": True, "n_gpus": n, "parallelism": f"pp{pp}xdp{dp}xtp{tp}", "schedule": args.schedule,
                          "layers_per_stage": lps, "microbatches": global_batch // mb, "compile_s": round(compile_s, 2),
                          "tasks": sum(1 for op in plan["ops"] if op["kind"] == "task"),
                          "reshards": sum(1 for op in plan["ops"] if op["kind"] == "reshard"),
                          "temp_gb_per_device": round(plan["temp_bytes_per_device_max"] / 2 ** 30, 1),
                          "plan_hash": plan["hash"], "stats": plan["stats"], "compiler_notes": plan.get("log", [])}))
        exe.shutdown()
        return 0

    from multimesh_jax_b200.models.init_sharded import init_sharded_llama
    params, state = init_sharded_llama(cfg, exe, dev, seed=1234)
    cos, sin = llama.rope_tables(cfg, seq, dev)

    g = torch.Generator().manual_seed(1)   # every rank draws the same global batch and keeps its own slice
    pool = min(24, args.warmup + 2 * args.steps)   # a fresh batch every step
    host_tok = [torch.randint(0, cfg.vocab, (global_batch, seq), generator=g).pin_memory() for _ in range(pool)]
    host_lab = [torch.randint(0, cfg.vocab, (global_batch, seq), generator=g).pin_memory() for _ in range(pool)]
    dev_tok = [t.to(dev) for t in host_tok]
    dev_lab = [t.to(dev) for t in host_lab]

    counter = [0]
    host_s = [0.0]      # wall-clock seconds the host spends inside the step call (submission only: the call does not wait for the GPU)

    def run_step(_i, e2e: bool):
        nonlocal params, state
        i = counter[0]
        counter[0] += 1
        if e2e:
            tok = host_tok[i % pool].to(dev, non_blocking=True)
            lab = host_lab[i % pool].to(dev, non_blocking=True)
        else:
            tok, lab = dev_tok[i % pool], dev_lab[i % pool]
        t0 = time.perf_counter()
        loss, params, state = exe(params, state, tok, lab, cos, sin)
        host_s[0] += time.perf_counter() - t0
        if e2e:
            return float(loss.full_tensor().item())
        return loss

    def barrier():
        if n > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(steps: int, e2e: bool):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        last = None
        for i in range(steps):
            last = run_step(i, e2e)
        e.record()
        barrier()
        ms = s.elapsed_time(e)
        if n > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, last

    last = None
    for i in range(args.warmup):
        last = run_step(i, False)
    # The compiled program (captured graph, plan, per-task programs) is a large, long-lived object
    # graph: a full collection that walks it takes a few hundred milliseconds of host time, longer
    # than the launch queue can cover. Everything alive now is moved out of the collector's reach.
    import gc
    gc.collect()
    gc.freeze()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0, lib0 = K.launch_count, K.library_call_count
    host_s[0] = 0.0
    ms, last = timed(args.steps, False)
    host_ms = host_s[0] * 1e3 / args.steps
    launches = K.launch_count - launches0
    lib_calls = K.library_call_count - lib0
    clocks = sampler.stop()
    loss_val = float(last.full_tensor().item()) if hasattr(last, "full_tensor") else float(last)
    ms_e2e, _ = timed(args.steps, True)
    status = K.read_status()
    if args.trace:
        from multimesh_jax_b200.utils import timeline
        os.makedirs(args.trace, exist_ok=True)
        res = {}
        barrier()
        with timeline.profile(res, device=local_rank, context=getattr(exe, "context", None)):
            t_last = run_step(0, False)
            t_last.wait() if hasattr(t_last, "wait") else None
            torch.cuda.synchronize()
        with open(os.path.join(args.trace, f"breakdown_n{n}_rank{rank}.txt"), "w") as f:
            f.write(res["breakdown"].format() + "\n" + json.dumps(res["breakdown"].to_dict()) + "\n")
        barrier()

    tokens = global_batch * seq * args.steps
    value = tokens / (ms / 1e3)
    e2e_value = tokens / (ms_e2e / 1e3)
    flops = cfg.flops_per_token(seq) * global_batch * seq
    if rank == 0:
        out = {
            "metric": "train tokens/s (device-timed, max over ranks)",
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": n, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / BASELINE_TOKENS_PER_S) if BASELINE_TOKENS_PER_S else None,
            "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "config": {"model": f"{args.model} shape ({cfg.n_layers} layers, d_model {cfg.d_model}, "
                                f"{cfg.n_heads}q/{cfg.n_kv_heads}kv heads, ffn {cfg.d_ff}, vocab {cfg.vocab})",
                       "global_batch": global_batch, "seq_len": seq, "microbatch": mb,
                       "layers_per_stage": lps, "parallelism": f"pp{pp}xdp{dp}xtp{tp}" + ("+fsdp" if args.fsdp else "")
                                      + ("+forced-reshard" if args.force_reshard else "") + ("+sp" if sp else ""), "schedule": args.schedule, "optimizer": "AdamW (fp32 master)",
                       "l2": "working set (>= 13 GB of weights per step) far exceeds the 126 MB L2; no flush needed"},
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": 2 * global_batch * seq * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "library_kernel_calls": lib_calls,
            "host_ms_per_step": round(host_ms, 2),
            "native_task_launches": getattr(exe, "native_launches", 0),
            "tflops_per_gpu": round(flops / (ms / args.steps / 1e3) / n / 1e12, 1),
            "loss": round(loss_val, 4), "compile_s": round(compile_s, 1), "kernel_status": status,
            "reshard_sources_in_place_vs_copied": [getattr(getattr(exe, "_peer_reshard", None), "direct_uses", 0),
                                                   getattr(getattr(exe, "_peer_reshard", None), "copied_uses", 0)],
            "fused_gemm_collective_calls": sum(o.calls for o in getattr(getattr(exe, "_fused_tp", None), "_ops", {}).values()),
            "impl": "ours",
        }
        print(json.dumps(out), flush=True)
    if n > 1:
        dist.barrier()
    exe.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
