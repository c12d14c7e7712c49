#!/usr/bin/env bash
# Continuous-integration entry point: build, CPU tests, then - when a GPU is visible - the GPU
# tests and a short benchmark. Usage: tests/run_ci.sh [--gpus N]
set -euo pipefail
cd "$(dirname "$0")/.."
gpus=0
if [[ "${1:-}" == "--gpus" ]]; then gpus="${2:-1}"; fi

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
