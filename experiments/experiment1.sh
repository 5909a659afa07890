#!/bin/bash
# Main comparison: single GPU vs SWARM (gradient sync every step) vs DiLoCo-SWARM (H = 50),
# GPT-2 small, 2 stages x 4 replicas on one 8-GPU node.  Same flags as the reference's
# experiments/experiment1.sh; sizes there were tuned for 80 GB GPUs, a B200 takes them as is.
set -e
DATA=${DATA:-@configs/data/fineweb-edu-10bt.toml}     # offline: DATA=@configs/data/synthetic-zipf.toml
COMMON="--model @configs/model/gpt2-small.toml --data $DATA --train.inner_optimizer @configs/optimizer/adamw.toml \
  --train.inner_optimizer.lr 4e-4 --train.scheduler.enable true --train.scheduler.num_warmup_steps 50 \
  --train.max_steps 2000 --data.seq_length 1024 --eval.enable true --eval.every_n_steps 50 --eval.eval_size 0.001 \
  --sample.enable true --sample.every_n_steps 100"
RUN="python -m torch.distributed.run --nnodes=1 --master-addr 127.0.0.1"

# weak baseline: one GPU
$RUN --nproc-per-node 1 -m diloco_swarm_b200.train --swarm.num_stages 1 --swarm.sync_every_n_steps 1 $COMMON \
  --train.outer_optimizer @configs/optimizer/none.toml --train.batch_size 512 --train.micro_batch_size 64

# strong baseline: SWARM
$RUN --nproc-per-node 8 -m diloco_swarm_b200.train --swarm.num_stages 2 --swarm.sync_every_n_steps 1 $COMMON \
  --train.outer_optimizer @configs/optimizer/none.toml --train.batch_size 2048 --train.micro_batch_size 32 \
  --train.max_micro_batches 12

# DiLoCo-SWARM
$RUN --nproc-per-node 8 -m diloco_swarm_b200.train --swarm.num_stages 2 --swarm.sync_every_n_steps 50 $COMMON \
  --train.outer_optimizer @configs/optimizer/nesterov.toml --train.outer_optimizer.lr 0.7 \
  --train.batch_size 2048 --train.micro_batch_size 32 --train.max_micro_batches 12
