"""Multi-GPU runs of the b200 engine (skipped on boxes with fewer GPUs).

Plain SWARM with a gradient sync every step yields the same weights whatever the
routing, so a 1 x 2 data-parallel run must reproduce the one-GPU loss curve, and a
2 x 2 swarm must reproduce the 2 x 1 pipeline (per-stage gradient clipping makes
pipelines differ slightly from the one-stage run).  Fused and library collectives
must agree for DiLoCo.
"""
import os
import re
import shutil
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOG = "/tmp/dsw_tests/gpu_multi"
_port = [29700]


def _run(run_id, nproc, stages, extra=(), engine="b200", timeout=300):
    shutil.rmtree(f"{LOG}/{run_id}", ignore_errors=True)
    _port[0] += 3
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_port[0]), "-m", "diloco_swarm_b200.train",
           "--swarm.num_stages", str(stages), "--engine", engine, "--model", "@configs/model/gpt2-tiny.toml",
           "--model.n_head", "2",                      # head size 64: the tcgen05 attention kernels
           "--data", "@configs/data/synthetic-zipf.toml", "--data.num_examples", "256", "--data.seq_length", "128",
           "--train.inner_optimizer", "@configs/optimizer/adamw.toml", "--train.inner_optimizer.lr", "0.003",
           "--train.outer_optimizer", "@configs/optimizer/none.toml", "--train.max_steps", "5",
           "--train.batch_size", "16", "--train.micro_batch_size", "2", "--train.max_micro_batches", "3",
           "--train.step_timeout", "30", "--eval.enable", "false", "--sample.enable", "false",
           "--logging.log_dir", LOG, "--logging.run_id", run_id, "--logging.console.log_level", "ERROR"] + list(extra)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run(cmd, cwd=ROOT, env=env, timeout=timeout, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    text = open(f"{LOG}/{run_id}/master.log").read()
    return [float(x) for x in re.findall(r"\[TRAIN\] Step: \d+ - Time: [\d.]+s - Loss: ([\d.]+)", text)]


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def test_data_parallel_fused_grad_sync_matches_single_gpu():
    _need(2)
    one = _run("one", 1, 1)
    two = _run("dp2", 2, 1)
    assert len(one) == len(two) == 5
    assert max(abs(a - b) for a, b in zip(one, two)) < 5e-3, (one, two)
    wire = _run("dp2_bf16", 2, 1, ["--swarm.grad_wire_dtype", "bfloat16"])
    assert max(abs(a - b) for a, b in zip(one, wire)) < 2e-2, (one, wire)


def test_diloco_fused_outer_sync_matches_library_twin():
    _need(2)
    extra = ["--train.outer_optimizer.type", "SGD", "--train.outer_optimizer.lr", "0.7",
             "--train.outer_optimizer.nesterov", "true", "--swarm.sync_every_n_steps", "2", "--train.max_steps", "6"]
    fused = _run("diloco_fused", 2, 1, extra)
    nccl = _run("diloco_nccl", 2, 1, extra + ["--swarm.collective", "nccl"])
    assert len(fused) == len(nccl) == 3
    assert max(abs(a - b) for a, b in zip(fused, nccl)) < 5e-3, (fused, nccl)


def test_swarm_2x2_matches_pipeline_2x1():
    _need(4)
    pipe = _run("pp2", 2, 2)
    swarm = _run("sw4", 4, 2)
    assert max(abs(a - b) for a, b in zip(pipe, swarm)) < 5e-3, (pipe, swarm)


def test_nvls_collectives_match_single_gpu():
    """The multimem variants of both stage-wide synchronisations (reduction and broadcast inside the NVSwitch)
    on two replicas: plain SWARM with fp32 and bf16 wire reproduces the one-GPU curve, DiLoCo agrees with the
    peer-load kernels.  On a box without NVLS the buffers come without a multicast address and the runs fall
    back to the peer-load kernels, so the comparison still holds."""
    _need(2)
    one = _run("one_b", 1, 1)
    two = _run("dp2_nvls", 2, 1, ["--swarm.collective", "nvls"])
    assert max(abs(a - b) for a, b in zip(one, two)) < 5e-3, (one, two)
    wire = _run("dp2_nvls_bf16", 2, 1, ["--swarm.collective", "nvls", "--swarm.grad_wire_dtype", "bfloat16"])
    assert max(abs(a - b) for a, b in zip(one, wire)) < 2e-2, (one, wire)
    extra = ["--train.outer_optimizer.type", "SGD", "--train.outer_optimizer.lr", "0.7",
             "--train.outer_optimizer.nesterov", "true", "--swarm.sync_every_n_steps", "2", "--train.max_steps", "6"]
    fused = _run("diloco_fused_b", 2, 1, extra)
    nvls = _run("diloco_nvls", 2, 1, extra + ["--swarm.collective", "nvls"])
    assert len(fused) == len(nvls) == 3
    assert max(abs(a - b) for a, b in zip(fused, nvls)) < 5e-3, (fused, nvls)


def test_copy_engine_transport_matches_nccl():
    """The two pipeline transports carry the same tensors in the same order: same loss curve."""
    _need(2)
    nccl = _run("pp2_nccl", 2, 2, ["--swarm.p2p", "nccl"])
    copy = _run("pp2_copy", 2, 2, ["--swarm.p2p", "copy", "--swarm.p2p_slots", "2"])     # 2 slots: rings wrap and fill
    assert len(nccl) == len(copy) == 5
    assert max(abs(a - b) for a, b in zip(nccl, copy)) < 2e-3, (nccl, copy)


def test_step_timeout_on_nccl_warns_then_drains():
    """A host-side straggler (a finite sleep per microbatch on rank 0, far below the process-group timeout)
    makes rank 1 wait longer than train.step_timeout: it must log the reference's warning, let everything
    posted drain, and the run must finish with the same losses as the undisturbed pipeline."""
    _need(2)
    calm = _run("pp2_calm", 2, 2, ["--train.max_steps", "3"])
    slow = _run("pp2_slow", 2, 2, ["--train.max_steps", "3", "--train.step_timeout", "1",
                                   "--swarm.straggler_rank", "0", "--swarm.straggler_ms", "200"])
    assert len(calm) == len(slow) == 3
    assert max(abs(a - b) for a, b in zip(calm, slow)) < 5e-3, (calm, slow)
    log1 = open(f"{LOG}/pp2_slow/1.log").read()
    assert "Train step 1 timed out" in log1 and "to drain" in log1
    assert "timed out" not in open(f"{LOG}/pp2_calm/1.log").read()


def test_replica_leaves_between_steps_on_gpus():
    """Membership change in the form that is safe on shared GPUs: a replica announces its leave, finishes its
    step and exits with nothing in flight; the survivor learns of it on the host before its next launch, shrinks
    the stage group and carries on (autograd engine on NCCL groups, one stage x two replicas, NVLS off, no
    multimem)."""
    _need(2)
    losses = _run("leave_gpu", 2, 1, ["--elastic.enable", "true", "--elastic.timeout", "20", "--elastic.leave_rank", "1",
                                      "--elastic.leave_after_step", "2", "--train.max_steps", "5",
                                      "--train.step_timeout", "5"], engine="torch", timeout=150)
    assert len(losses) == 5 and all(l == l for l in losses)
    assert losses[-1] < losses[0]
    text = open(f"{LOG}/leave_gpu/master.log").read() + open(f"{LOG}/leave_gpu/0.log").read()
    assert "ranks [1] are gone" in text
    assert "Rank 1 leaves after step 2" in open(f"{LOG}/leave_gpu/1.log").read()
