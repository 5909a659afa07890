#!/bin/bash
# Smoke run without a GPU: two data-parallel gloo ranks memorise one sentence (what the reference's
# experiments/test.sh does with its own launcher).  Pass a number of steps as the first argument.
set -euo pipefail
cd "$(dirname "$0")/.."

STEPS="${1:-40}"
MODEL=(--model @configs/model/gpt2-tiny.toml)
DATA=(--data @configs/data/memorize.toml --data.tokenize true --data.seq_length 128)
OPTIM=(--train.inner_optimizer @configs/optimizer/adamw.toml --train.inner_optimizer.lr 0.006
       --train.outer_optimizer @configs/optimizer/none.toml)
RUN=(--swarm.num_stages 1 --device cpu --amp.enable false --eval.enable false
     --train.max_steps "$STEPS" --train.batch_size 2 --train.micro_batch_size 1)

python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
  -m diloco_swarm_b200.train "${RUN[@]}" "${MODEL[@]}" "${DATA[@]}" "${OPTIM[@]}"
