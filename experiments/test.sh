#!/bin/bash
# Smoke run: 2-process data parallel on CPU with the memorisation set (reference: experiments/test.sh).
python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m diloco_swarm_b200.train \
  --swarm.num_stages 1 --device cpu --model @configs/model/gpt2-tiny.toml --data @configs/data/memorize.toml \
  --data.tokenize true --data.seq_length 128 --train.inner_optimizer @configs/optimizer/adamw.toml \
  --train.outer_optimizer @configs/optimizer/none.toml --train.inner_optimizer.lr 0.006 --train.max_steps 40 \
  --train.batch_size 2 --train.micro_batch_size 1 --amp.enable false --eval.enable false
