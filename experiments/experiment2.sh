#!/bin/bash
# Communication-frequency sweep: DiLoCo-SWARM with H in {1, 10, 20, 50, 100, 200, 500}
# (the reference sweeps 10..200 and reports that H = 1 did not converge).
set -e
DATA=${DATA:-@configs/data/fineweb-edu-10bt.toml}
for H in ${HS:-1 10 20 50 100 200 500}; do
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m diloco_swarm_b200.train \
  --swarm.num_stages 2 --swarm.sync_every_n_steps $H --model @configs/model/gpt2-small.toml --data $DATA \
  --train.inner_optimizer @configs/optimizer/adamw.toml --train.inner_optimizer.lr 4e-4 \
  --train.outer_optimizer @configs/optimizer/nesterov.toml --train.outer_optimizer.lr 0.7 \
  --train.scheduler.enable true --train.scheduler.num_warmup_steps 50 --train.max_steps 2000 \
  --train.batch_size 2048 --train.micro_batch_size 32 --train.max_micro_batches 12 --data.seq_length 1024 \
  --eval.enable true --eval.every_n_steps $H --eval.eval_size 0.001 --sample.enable false \
  --logging.run_id diloco-H$H
done
