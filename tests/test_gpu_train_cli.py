"""The training entry point on one GPU with the b200 engine: the reference's memorisation test
(tests/test_memorize.py:76-84, `device = cuda`), end to end through the command line, the sm_100a
kernels (head size 32 attention included), the end-of-training sampling and the logs."""
import os
import re
import shutil
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOG = "/tmp/dsw_tests/gpu_cli"


def test_memorization_on_one_gpu():
    from diloco_swarm_b200.utils.data import MEMORIZE_SENTENCE
    shutil.rmtree(f"{LOG}/memorize", ignore_errors=True)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=1",
           "--master-addr", "127.0.0.1", "--master-port", "29790", "-m", "diloco_swarm_b200.train",
           "--swarm.num_stages", "1", "--engine", "b200", "--model", "@configs/model/gpt2-tiny.toml",
           "--data", "@configs/data/memorize.toml", "--data.tokenize", "true", "--data.seq_length", "128",
           "--train.inner_optimizer", "@configs/optimizer/adamw.toml", "--train.outer_optimizer",
           "@configs/optimizer/none.toml", "--train.inner_optimizer.lr", "0.006", "--train.max_steps", "220",
           "--train.batch_size", "4", "--train.micro_batch_size", "2", "--train.max_micro_batches", "2",
           "--sample.max_new_tokens", "64", "--sample.temperature", "0.1", "--eval.enable", "false",
           "--logging.log_dir", LOG, "--logging.run_id", "memorize", "--logging.console.log_level", "ERROR"]
    p = subprocess.run(cmd, cwd=ROOT, timeout=300, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    text = open(f"{LOG}/memorize/master.log").read()
    losses = [float(x) for x in re.findall(r"\[TRAIN\] Step: \d+ - Time: [\d.]+s - Loss: ([\d.]+)", text)]
    assert len(losses) == 220 and losses[-1] < 0.05, (len(losses), losses[-5:])      # one epoch holds 225 steps
    assert MEMORIZE_SENTENCE in text.split("Sample 1:")[-1], text[-1500:]
