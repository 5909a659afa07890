#!/usr/bin/env bash
# Undo what experiments/setup.sh and a few runs leave behind on this machine: the built native
# libraries and object files, run logs, test scratch and Python caches.  Sources and configs stay.
# (The reference's cleanup scripts remove its conda environment and dotfiles from a rented
# machine, scripts/cleanup.sh and scripts/cleanup_remote.sh; nothing of that kind is installed here.)
set -euo pipefail
cd "$(dirname "$0")/.."

rm -rf diloco_swarm_b200/build
rm -f diloco_swarm_b200/libdswarm_host.so diloco_swarm_b200/libdswarm_cuda.so
if [[ "${1:-}" == "--logs" ]]; then
  rm -rf logs
fi
rm -rf /tmp/dsw_tests /tmp/dswarm_bench /tmp/dswarm_ref_bench
find . -name __pycache__ -type d -not -path "./baseline/_ref/*" -prune -exec rm -rf {} +
rm -rf .pytest_cache .hypothesis
echo "cleaned (run experiments/setup.sh or python __graft_entry__.py to rebuild)"
