#!/bin/bash
# Prepare a node for the experiment scripts (reference: scripts/setup.sh and scripts/setup_remote.sh, which
# provision the authors' rented machines over ssh; here everything is local and offline):
# build the two in-tree libraries, print what the runs will see, and run the CPU tests.
set -e
cd "$(dirname "$0")/.."
python __graft_entry__.py
python - <<'PY'
import torch, diloco_swarm_b200
print("torch", torch.__version__, "| cuda available:", torch.cuda.is_available(), "| GPUs:", torch.cuda.device_count())
PY
if command -v nvidia-smi > /dev/null; then
  nvidia-smi --query-gpu=index,name,memory.total,clocks.max.sm --format=csv     # read-only queries
  nvidia-smi topo -m || true
fi
if [ "${1:-}" = "--test" ]; then
  python -m pytest tests -q -m "not gpu"
fi
