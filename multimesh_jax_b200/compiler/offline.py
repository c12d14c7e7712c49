"""Command-line offline compile of a stored program.

    python -m multimesh_jax_b200.compiler.offline step.mmprog.json [--device-memory-gb 180] [--dump-plan]

Prints one JSON summary (templates, tasks, reshards, per-device memory high-water marks, whether
the plan fits the given device memory, hazards of the submission order). Exit code 1 when the
plan does not fit, violates the runtime protocol or has an unordered conflicting pair. Needs no
GPU and none of the model code that produced the file
(the reference's `CompileHloModuleFromFile`, src/pjrt_client/mm_pjrt_client.cc:702-771, serves
its compiler tests the same way).
"""
from __future__ import annotations

import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="python -m multimesh_jax_b200.compiler.offline")
    p.add_argument("program")
    p.add_argument("--device-memory-gb", type=float, default=0.0, help="made-up device memory size; 0 = no limit")
    p.add_argument("--dump-plan", action="store_true", help="also print the plan's operation list")
    ns = p.parse_args(argv)
    from .api import compile_program_file
    r = compile_program_file(ns.program, int(ns.device_memory_gb * (1 << 30)), want_plan=ns.dump_plan)
    plan = r.pop("plan", None)
    r.pop("log", None)
    print(json.dumps(r))
    if plan is not None:
        for op in plan["ops"]:
            print(json.dumps(op))
    return 0 if (r["fits"] and r["status"] == 0 and not r["hazards"]) else 1


if __name__ == "__main__":
    sys.exit(main())
