#!/bin/bash
# Model-size sweep: single GPU vs DiLoCo-SWARM for GPT-2 tiny / medium / large.  Micro-batch sizes follow the
# reference (medium 8, large 4).  MEDIUM_STAGES=4 gives the 4 stages x 2 replicas layout.
set -e
DATA=${DATA:-@configs/data/fineweb-edu-10bt.toml}
for SPEC in ${SPECS:-"tiny 64 16" "medium 8 16" "large 4 8"}; do
set -- $SPEC; MODEL=$1; MBS=$2; CAP=$3
STAGES=2; [ "$MODEL" = "medium" ] && STAGES=${MEDIUM_STAGES:-2}
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m diloco_swarm_b200.train \
  --swarm.num_stages $STAGES --swarm.sync_every_n_steps 50 --swarm.layer_split balanced \
  --model @configs/model/gpt2-$MODEL.toml --data $DATA \
  --train.inner_optimizer @configs/optimizer/adamw.toml --train.inner_optimizer.lr 4e-4 \
  --train.outer_optimizer @configs/optimizer/nesterov.toml --train.outer_optimizer.lr 0.7 \
  --train.scheduler.enable true --train.scheduler.num_warmup_steps 50 --train.max_steps 2000 \
  --train.batch_size 2048 --train.micro_batch_size $MBS --train.max_micro_batches $CAP --data.seq_length 1024 \
  --eval.enable true --eval.every_n_steps 50 --eval.eval_size 0.001 --sample.enable false \
  --logging.run_id diloco-$MODEL
done
