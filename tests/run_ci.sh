#!/usr/bin/env bash
# Continuous-integration entry point: build, CPU tests, then - when a GPU is visible - the GPU
# tests and a short benchmark. Usage: tests/run_ci.sh [--gpus N] | tests/run_ci.sh --asan
#
# --asan: the CPU tests once more against an AddressSanitizer build of the C++ compiler / runtime
# module, made in a scratch copy of the tree (the in-tree module is not touched). libstdc++ is
# preloaded next to libasan so that the sanitizer can intercept C++ exceptions inside Python.
set -euo pipefail
cd "$(dirname "$0")/.."
gpus=0
if [[ "${1:-}" == "--gpus" ]]; then gpus="${2:-1}"; fi

if [[ "${1:-}" == "--asan" ]]; then
  scratch="$(mktemp -d)"
  cp -r multimesh_jax_b200 tests docs bench.py __graft_entry__.py pyproject.toml "$scratch"/
  cd "$scratch"
  MM_HOST_CXXFLAGS="-fsanitize=address -fno-omit-frame-pointer -O1 -g1" \
    python -c "from multimesh_jax_b200.csrc import build as b; b.build_host(force=True)"
  LD_PRELOAD="$(gcc -print-file-name=libasan.so) $(gcc -print-file-name=libstdc++.so.6)" \
    ASAN_OPTIONS=detect_leaks=0:halt_on_error=1 \
    python -m pytest tests -q -m "not gpu" -p no:cacheprovider \
      --deselect tests/test_sanitizers.py --deselect tests/test_bench_layouts.py --deselect tests/test_dist_gloo.py
  exit 0
fi

python -c "import __graft_entry__ as g; g.build()"
python -m pytest tests -q -m "not gpu"

if python -c "import torch, sys; sys.exit(0 if torch.cuda.is_available() else 1)"; then
  python -m pytest tests -q -m gpu
  python -c "import __graft_entry__ as g; g.smoke()"
  if [[ "$gpus" -gt 1 ]]; then
    NCCL_NVLS_ENABLE=0 python -m torch.distributed.run --nnodes=1 --nproc-per-node "$gpus" \
      --master-addr 127.0.0.1 --master-port 29555 bench.py --gpus "$gpus" --steps 2 --warmup 3
  else
    python bench.py --steps 2 --warmup 3
  fi
fi
