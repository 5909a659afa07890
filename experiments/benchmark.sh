#!/bin/bash
# Throughput of the four kinds of parallelism on one node: single GPU, data parallel, pipeline parallel
# and SWARM, over micro-batch sizes and in-flight limits, then one table from the runs' metric histories.
# This is the "Benchmark" section of the reference's results notebook (notebooks/3.0-results.ipynb, cells
# 33-48: GPT-2 small, five steps, batch 512 x 1024), which there reads the numbers from wandb.
# GPUS=8 (default) gives DP on 8, PP on 2 and 4, SWARM as 2 x 4; MBS and CAPS choose the sweep.
set -e
cd "$(dirname "$0")/.."
GPUS=${GPUS:-8}
OUT=${OUT:-logs/benchmark}
DATA=${DATA:-@configs/data/synthetic-zipf.toml}
COMMON="--model @configs/model/gpt2-small.toml --data $DATA --data.seq_length 1024 --train.batch_size 512 \
  --train.inner_optimizer @configs/optimizer/adamw.toml --train.outer_optimizer @configs/optimizer/none.toml \
  --train.max_steps 5 --eval.enable false --sample.enable false --logging.log_dir $OUT --logging.console.log_level ERROR"
RUNS=()
launch() {   # name, processes, stages, micro-batch size, in-flight limit
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$2" --master-addr 127.0.0.1 -m diloco_swarm_b200.train \
    --swarm.num_stages "$3" --swarm.layer_split balanced $COMMON --train.micro_batch_size "$4" \
    --train.max_micro_batches "$5" --logging.run_id "$1"
  RUNS+=("$1=$OUT/$1")
}
for MB in ${MBS:-8 16 32}; do
  launch "single-mbs$MB" 1 1 "$MB" 1
  launch "dp$GPUS-mbs$MB" "$GPUS" 1 "$MB" 1
  for CAP in ${CAPS:-4 8}; do
    launch "pp2-mbs$MB-cap$CAP" 2 2 "$MB" "$CAP"
    [ "$GPUS" -ge 4 ] && launch "pp4-mbs$MB-cap$CAP" 4 4 "$MB" "$CAP"
    [ "$GPUS" -ge 4 ] && launch "swarm$GPUS-mbs$MB-cap$CAP" "$GPUS" 2 "$MB" "$CAP"
  done
done
python -m diloco_swarm_b200.utils.results "${RUNS[@]}" --table throughput
