"""Multi-process topologies on CPU/gloo (the reference's test strategy, tests/test_memorize.py),
plus what the reference never tests: loss parity between topologies and with the virtual swarm,
DiLoCo, checkpoint/resume and the step timeout."""
import os
import re
import shutil
import subprocess
import sys

import pytest
import torch

from helpers import make_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LOG = "/tmp/dsw_tests/mp"
pytestmark = pytest.mark.slow
_port = [29600]


_done = {}


def launch(run_id, nproc, stages, extra=(), timeout=240, expect_ok=True, reuse=False):
    key = (run_id, nproc, stages, tuple(extra))
    if reuse and key in _done:
        return _done[key]
    _done[key] = None
    shutil.rmtree(f"{LOG}/{run_id}", ignore_errors=True)
    _port[0] += 3
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(_port[0]), "-m", "diloco_swarm_b200.train",
           "--swarm.num_stages", str(stages), "--device", "cpu",
           "--model", "@configs/model/gpt2-tiny.toml", "--model.n_layer", "2", "--model.vocab_size", "50257",
           "--data", "@configs/data/synthetic-zipf.toml", "--data.num_examples", "400", "--data.seq_length", "32",
           "--train.inner_optimizer", "@configs/optimizer/adamw.toml", "--train.inner_optimizer.lr", "4e-4",
           "--train.outer_optimizer", "@configs/optimizer/none.toml",
           "--train.max_steps", "6", "--train.batch_size", "16", "--train.micro_batch_size", "4",
           "--train.max_micro_batches", "2", "--train.seed", "0", "--train.step_timeout", "60",
           "--amp.enable", "false", "--eval.enable", "false", "--sample.enable", "false",
           "--logging.log_dir", LOG, "--logging.run_id", run_id, "--logging.console.log_level", "ERROR"] + list(extra)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    p = subprocess.run(cmd, cwd=ROOT, env=env, timeout=timeout, capture_output=True, text=True)
    if expect_ok:
        assert p.returncode == 0, p.stderr[-3000:]
    return p


def global_losses(run_id):
    text = open(f"{LOG}/{run_id}/master.log").read()
    return [float(x) for x in re.findall(r"\[TRAIN\] Step: \d+ - Time: [\d.]+s - Loss: ([\d.]+)", text)]


def virtual_losses(world_size, stages, steps=6, **over):
    from diloco_swarm_b200.parallel.simulator import VirtualSwarm
    from diloco_swarm_b200.utils import data as D
    base = dict(model={"n_layer": 2, "n_head": 4, "n_embd": 128, "vocab_size": 50257, "block_size": 1024},
                data={"path": "synthetic:zipf", "seq_length": 32, "num_examples": 400, "vocab_limit": 50257},
                train={"micro_batch_size": 4, "batch_size": 16, "max_steps": steps, "max_micro_batches": 2, "seed": 0,
                       "inner_optimizer": {"type": "AdamW", "lr": 4e-4}},
                swarm={"num_stages": stages})
    for k, v in over.items():
        base.setdefault(k, {}).update(v)
    cfg = make_config(**base)
    ds = D.get_dataset(cfg.data, D.ByteTokenizer(), seed=0)
    train, _ = ds.train_test_split(cfg.eval.eval_size, seed=0)
    vs = VirtualSwarm(cfg, world_size)
    vs.num_train_steps = steps
    out, it = [], iter(D.BatchLoader(train, 16))
    for step in range(1, steps + 1):
        r = vs.train_step(step, next(it))
        if r["do_sync"]:
            out.append(r["global"].loss)
    return out


def test_swarm_topologies_give_the_single_process_loss_curve():
    """Plain SWARM with a gradient sync every step is mathematically one process
    accumulating all microbatches, whatever the routing (src/train.py:168,217-218)."""
    launch("single", 1, 1)
    ref = global_losses("single")
    assert len(ref) == 6 and ref[-1] < ref[0]
    for name, nproc, stages in (("dp2", 2, 1), ("swarm4", 4, 2)):
        launch(name, nproc, stages, reuse=True)
        got = global_losses(name)
        assert len(got) == 6
        # the logged loss is the mean over the last-stage replicas of per-replica sums, so with
        # uneven routing it is not the single-process number; the weights are, hence the next steps'
        # losses stay on the single-process curve within routing noise
        assert abs(got[-1] - ref[-1]) < 0.05 * ref[-1], (name, got, ref)


def test_multiprocess_matches_virtual_swarm_plain():
    launch("swarm4", 4, 2, reuse=True)
    got = global_losses("swarm4")
    want = virtual_losses(4, 2)
    assert len(got) == len(want) == 6
    assert max(abs(a - b) for a, b in zip(got, want)) < 2e-3, (got, want)


def test_multiprocess_matches_virtual_swarm_diloco():
    extra = ["--train.outer_optimizer.type", "SGD", "--train.outer_optimizer.lr", "0.7",
             "--train.outer_optimizer.nesterov", "true", "--swarm.sync_every_n_steps", "3"]
    launch("diloco4", 4, 2, extra)
    got = global_losses("diloco4")
    want = virtual_losses(4, 2, train={"outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}},
                          swarm={"sync_every_n_steps": 3})
    assert len(got) == len(want) == 2                # global metrics exist on sync steps only
    assert max(abs(a - b) for a, b in zip(got, want)) < 2e-3, (got, want)


def test_memorization_on_a_swarm():
    """The reference's integration test (tests/test_memorize.py:76-84) on its SWARM topology, 4 processes
    in 2 stages: train the 4-layer model on one sentence and find the sentence in master.log, where the
    end-of-training samples are logged.  Offline the tokenizer is byte level (61 tokens instead of 14), so
    the run is 170 steps of 4 one-row microbatches (sequence length 64) instead of 40 steps of one."""
    from diloco_swarm_b200.utils.data import MEMORIZE_SENTENCE
    shutil.rmtree(f"{LOG}/memorize", ignore_errors=True)
    _port[0] += 3
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
           "--master-addr", "127.0.0.1", "--master-port", str(_port[0]), "-m", "diloco_swarm_b200.train",
           "--swarm.num_stages", "2", "--device", "cpu", "--model", "@configs/model/gpt2-tiny.toml",
           "--data", "@configs/data/memorize.toml", "--data.tokenize", "true", "--data.seq_length", "64",
           "--train.inner_optimizer", "@configs/optimizer/adamw.toml", "--train.outer_optimizer",
           "@configs/optimizer/none.toml", "--train.inner_optimizer.lr", "0.006", "--train.max_steps", "170",
           "--train.batch_size", "4", "--train.micro_batch_size", "1", "--train.max_micro_batches", "2",
           "--sample.max_new_tokens", "64", "--sample.temperature", "0.1", "--sample.num_samples", "2",
           "--logging.file.log_level", "INFO", "--amp.enable", "false", "--ckpt.enable", "true",
           "--eval.enable", "false", "--logging.log_dir", LOG, "--logging.run_id", "memorize",
           "--logging.console.log_level", "ERROR"]
    p = subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, OMP_NUM_THREADS="1"), timeout=600, capture_output=True, text=True)
    assert p.returncode == 0, p.stderr[-3000:]
    text = open(f"{LOG}/memorize/master.log").read()
    assert MEMORIZE_SENTENCE in text.split("Sample 1:")[-1], text[-1500:]
    # the swarm's final checkpoint, merged into one model, says the same in the one-process sampler
    from diloco_swarm_b200 import generate as G
    from diloco_swarm_b200.utils import data as D
    model = G.load_model(f"{LOG}/memorize/checkpoints/step_170")
    out = G.generate(model, D.get_tokenizer(), "I am", max_new_tokens=64, temperature=0.0, num_samples=1)
    assert MEMORIZE_SENTENCE in out[0], out


def test_three_stage_pipeline_with_eval_and_sampling():
    launch("pp3", 3, 3, ["--eval.enable", "true", "--eval.eval_size", "0.1", "--eval.every_n_steps", "3",
                         "--sample.enable", "true", "--sample.max_new_tokens", "4", "--sample.num_samples", "2"])
    text = open(f"{LOG}/pp3/master.log").read()
    assert "[TEST] Avg. Loss" in text and "Sample 2:" in text
    assert os.path.exists(f"{LOG}/pp3/samples/0.txt") and os.path.exists(f"{LOG}/pp3/samples/6.txt")


def test_checkpoint_and_resume():
    launch("ck", 2, 2, ["--ckpt.enable", "true", "--ckpt.every_n_steps", "3", "--train.max_steps", "6"])
    full = global_losses("ck")
    d = f"{LOG}/ck/checkpoints"
    assert sorted(os.listdir(d)) == ["step_3", "step_6"]
    assert sorted(os.listdir(f"{d}/step_3")) == ["meta.json", "model.0.pt", "model.1.pt", "optim.0.pt", "optim.1.pt"]
    sd = torch.load(f"{d}/step_3/model.1.pt", weights_only=True)
    assert "lm_head.weight" in sd and "transformer.h.0.ln_1.weight" in sd and "transformer.wte.weight" not in sd
    # resume from step 3 into the same run directory: steps 4..6 must reproduce the first run
    shutil.rmtree(f"{d}/step_6")
    os.remove(f"{LOG}/ck/master.log")
    cmd_extra = ["--ckpt.enable", "true", "--ckpt.resume", "true", "--ckpt.every_n_steps", "3", "--train.max_steps", "6"]
    # same launch line; Logger reuses <log_dir>/<run_id>, so the checkpoints are found
    launch_keep("ck", 2, 2, cmd_extra)
    resumed = global_losses("ck")
    assert len(resumed) == 3
    assert max(abs(a - b) for a, b in zip(resumed, full[3:])) < 1e-4, (resumed, full)


def test_checkpoint_moves_to_another_topology():
    """A 2 x 2 swarm's checkpoint, merged and re-cut by utils/ckpt.py, resumes as one process and as a
    plain 2-stage pipeline: the first step after the move sees the same weights and the same batch, so its loss
    is the loss the swarm itself reports for that step."""
    from diloco_swarm_b200.utils import ckpt as C
    # balanced routing: with the uniform draw a last-stage replica can end a step without a microbatch,
    # and the logged loss (a mean over the replicas that saw data, as in the reference) is then scaled
    launch("ckmove", 4, 2, ["--ckpt.enable", "true", "--ckpt.every_n_steps", "3", "--train.max_steps", "4",
                            "--swarm.routing", "balanced"])
    want = global_losses("ckmove")[3]
    src = f"{LOG}/ckmove/checkpoints/step_3"
    full = C.merge_model(src)
    assert "transformer.h.1.mlp.c_proj.weight" in full and "lm_head.weight" in full and len(full) == 2 + 2 * 12 + 2 + 1
    mean = C.merge_model(src, average_replicas=True)          # replicas agree right after a synchronisation
    assert all(torch.allclose(full[k], mean[k], atol=1e-6) for k in full)
    for run_id, nproc, stages in (("ckmove1", 1, 1), ("ckmove2", 2, 2)):
        shutil.rmtree(f"{LOG}/{run_id}", ignore_errors=True)
        meta = C.reshard(src, f"{LOG}/{run_id}/checkpoints/step_3", stages, nproc // stages)
        assert meta["world_size"] == nproc and meta["resharded_from"]["world_size"] == 4
        launch_keep(run_id, nproc, stages, ["--ckpt.resume", "true", "--train.max_steps", "4"])
        got = global_losses(run_id)
        assert len(got) == 1 and abs(got[0] - want) < 2e-4, (run_id, got, want)


def test_adaptive_routing_moves_work_away_from_a_slow_replica():
    """routing = adaptive on 2 x 2: last-stage replica 3 is slowed on the host (a sleep per microbatch op);
    every rank shares its compute time per microbatch after each step and the next steps draw replicas in
    proportion to the measured speeds, so the slow replica ends up with clearly less than its even share."""
    from diloco_swarm_b200.utils import results
    launch("adaptive", 4, 2, ["--swarm.routing", "adaptive", "--swarm.straggler_rank", "3", "--swarm.straggler_ms", "80",
                              "--train.batch_size", "32", "--train.micro_batch_size", "2", "--train.max_steps", "10",
                              "--train.max_micro_batches", "4"])
    key = "train/local/num_micro_batches/current"
    per_step = lambda total: [b - a for a, b in zip([0] + total[:-1], total)]      # the metric is a running count
    fast = per_step(results.load_history(f"{LOG}/adaptive", "1")[key].tolist())
    slow = per_step(results.load_history(f"{LOG}/adaptive", "3")[key].tolist())
    assert len(fast) == 10 and all(f + s == 16 for f, s in zip(fast, slow))       # every microbatch is served once
    assert sum(slow[2:]) < 0.6 * sum(fast[2:]), (fast, slow)
    assert len(global_losses("adaptive")) == 10


def test_step_timeline_of_a_swarm():
    """--logging.timeline_steps: every rank records its forwards and backwards of two steps; the merged
    trace has one lane per rank, spans that do not overlap within a lane, every microbatch once per stage,
    and a last stage that only starts after the first stage's first forward."""
    from diloco_swarm_b200.utils import timeline as T
    launch("timeline", 4, 2, ["--logging.timeline_steps", "2", "--logging.timeline_start", "2", "--train.max_steps", "4"])
    recs = T.load(f"{LOG}/timeline/timeline")
    assert sorted((r["rank"], r["step"]) for r in recs) == [(r, s) for r in range(4) for s in (2, 3)]
    for r in recs:
        spans = sorted((o["start_ms"], o["end_ms"]) for o in r["ops"])
        assert all(a[1] <= b[0] + 1e-6 for a, b in zip(spans, spans[1:])), r
        assert {"optimizer", "grad_sync"} <= {o["name"] for o in r["ops"]}
    step2 = [r for r in recs if r["step"] == 2]
    fwd_first = sorted(o["name"] for r in step2 if r["rank"] % 2 == 0 for o in r["ops"] if o["name"].startswith("F"))
    last = sorted(o["name"] for r in step2 if r["rank"] % 2 == 1 for o in r["ops"] if o["name"].startswith("FB"))
    assert fwd_first == sorted(f"F{m}" for m in range(4)) and last == sorted(f"FB{m}" for m in range(4))
    trace = T.chrome_trace(recs)
    assert {e["pid"] for e in trace["traceEvents"]} == {0, 1, 2, 3}
    origin = min(r["t0"] for r in step2)
    start = lambda r, prefix: min((r["t0"] - origin) * 1e3 + o["start_ms"] for o in r["ops"] if o["name"].startswith(prefix))
    first_fwd_end = min((r["t0"] - origin) * 1e3 + o["end_ms"] for r in step2 if r["rank"] % 2 == 0
                        for o in r["ops"] if o["name"].startswith("F"))
    assert all(start(r, "FB") >= first_fwd_end - 1.0 for r in step2 if r["rank"] % 2 == 1 and
               any(o["name"].startswith("FB") for o in r["ops"]))
    util = T.utilisation(recs)
    assert set(util) == {2, 3} and all(0 < v <= 1.0 + 1e-6 for k, v in util[2].items() if k.endswith("_busy"))


def launch_keep(run_id, nproc, stages, extra):
    """Like launch() but keeps the existing run directory."""
    real_rmtree = shutil.rmtree
    shutil.rmtree = lambda *a, **k: None
    try:
        return launch(run_id, nproc, stages, extra)
    finally:
        shutil.rmtree = real_rmtree


def replay_with_membership(gone, from_step, dropped_step, steps, **over):
    """Global losses of a single-process replay (VirtualSwarm) of the launch() configuration in which rank
    ``gone`` is out of the routing from ``from_step`` on and ``dropped_step`` (or None) is abandoned."""
    from diloco_swarm_b200.parallel.simulator import VirtualSwarm
    from diloco_swarm_b200.utils import data as D
    cfg = make_config(model={"n_layer": 2, "n_head": 4, "n_embd": 128, "vocab_size": 50257, "block_size": 1024},
                      data={"path": "synthetic:zipf", "seq_length": 32, "num_examples": 400, "vocab_limit": 50257},
                      train={"micro_batch_size": 4, "batch_size": 16, "max_steps": steps, "max_micro_batches": 2, "seed": 0,
                             "inner_optimizer": {"type": "AdamW", "lr": 4e-4}}, swarm={"num_stages": 2})
    base = cfg.model_dump()
    for k, v in over.items():
        base[k].update(v)
    cfg = make_config(**base)
    train, _ = D.get_dataset(cfg.data, D.ByteTokenizer(), seed=0).train_test_split(cfg.eval.eval_size, seed=0)
    vs = VirtualSwarm(cfg, 4)
    vs.num_train_steps = steps
    out, it = [], iter(D.BatchLoader(train, 16))
    for step in range(1, steps + 1):
        if step == from_step:
            vs.set_alive([r != gone for r in range(4)])
        res = vs.train_step(step, next(it), dropped=(step == dropped_step))
        if res["global"] is not None and res["do_sync"]:          # the trainer logs global metrics on sync steps
            out.append(res["global"].loss)
    return out


@pytest.mark.parametrize("leaver", [2])          # a first-stage replica; the DiLoCo test below takes a last-stage one
def test_rank_leaves_between_steps_and_the_swarm_reroutes(leaver):
    """Host-side failure: one replica announces a leave, finishes its step and exits; the others learn
    of it from the store before their next step, route around it and keep training."""
    name = f"leave{leaver}"
    launch(name, 4, 2, ["--elastic.enable", "true", "--elastic.timeout", "20", "--elastic.leave_rank", str(leaver),
                        "--elastic.leave_after_step", "2", "--train.max_steps", "5"])
    losses = global_losses(name)
    assert len(losses) == 5 and losses[-1] < losses[0]
    text = open(f"{LOG}/{name}/master.log").read() + open(f"{LOG}/{name}/0.log").read()
    assert f"ranks [{leaver}] are gone" in text
    assert f"Rank {leaver} leaves after step 2" in open(f"{LOG}/{name}/{leaver}.log").read()
    want = replay_with_membership(gone=leaver, from_step=3, dropped_step=None, steps=5)
    assert max(abs(a - b) for a, b in zip(losses, want)) < 2e-3, (losses, want)


def test_rank_leaves_under_diloco():
    """A last-stage replica leaves between two outer steps: the next pseudo-gradient average runs over the
    replicas that are left, and the losses on the outer steps equal the single-process replay."""
    outer = {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}
    launch("leave_diloco", 4, 2, ["--elastic.enable", "true", "--elastic.timeout", "20", "--elastic.leave_rank", "3",
                                  "--elastic.leave_after_step", "3", "--train.max_steps", "6",
                                  "--train.outer_optimizer.type", "SGD", "--train.outer_optimizer.lr", "0.7",
                                  "--train.outer_optimizer.nesterov", "true", "--swarm.sync_every_n_steps", "2"])
    losses = global_losses("leave_diloco")
    want = replay_with_membership(gone=3, from_step=4, dropped_step=None, steps=6,
                                  train={"outer_optimizer": outer}, swarm={"sync_every_n_steps": 2})
    assert len(losses) == len(want) == 3          # global metrics exist on the outer steps 2, 4, 6
    assert max(abs(a - b) for a, b in zip(losses, want)) < 2e-3, (losses, want)


@pytest.mark.parametrize("victim", [2])          # a first-stage replica: last-stage replicas wait for its activations
def test_rank_dies_silently_and_the_step_is_dropped(victim):
    """Host-side failure without notice: a replica exits at the start of step 3, after the step's routing
    was fixed with it in.  The others' transfers with it fail or time out, the common verdict drops the
    step on every live rank, the rank that did not vote is removed before step 4 and training goes on
    (fresh pipeline groups, re-formed stage group)."""
    name = f"die{victim}"
    launch(name, 4, 2, ["--elastic.enable", "true", "--elastic.timeout", "6", "--train.step_timeout", "6",
                        "--elastic.die_rank", str(victim), "--elastic.die_at_step", "3", "--train.max_steps", "6",
                        "--sample.enable", "true", "--sample.max_new_tokens", "3", "--sample.num_samples", "2"],
           timeout=300)
    losses = global_losses(name)
    assert len(losses) == 5 and losses[-1] < losses[0], losses          # steps 1, 2, 4, 5, 6
    logs = {r: open(f"{LOG}/{name}/{r}.log").read() for r in range(4)}
    assert f"Rank {victim} dies silently at step 3" in logs[victim]
    for r in range(4):
        if r != victim:
            assert "Step 3 is dropped" in logs[r], r
            assert f"Step 4: ranks [{victim}] are gone" in logs[r], r
    assert "Sample 2:" in open(f"{LOG}/{name}/master.log").read()      # end-of-training sampling among the survivors
    # the survivors' loss curve is the one a single process gets when it drops step 3 and takes the victim
    # out of the routing from step 4 on
    want = replay_with_membership(gone=victim, from_step=4, dropped_step=3, steps=6)
    assert max(abs(a - b) for a, b in zip(losses, want)) < 2e-3, (losses, want)


def test_tiny_diloco_swarm_2x2_matches_single_process_replay():
    """Tiny GPT-2 (2 layers, d 128, 4 heads, tied embeddings requested, vocab 50257, seq 128, fp32) as
    DiLoCo-SWARM on 2 stages x 2 replicas over gloo: microbatch 4, 4 microbatches per step, AdamW 4e-4
    (betas 0.9/0.95, wd 0.1), H = 10, outer Nesterov lr 0.7 momentum 0.9, 20 steps, Zipf(1.0) tokens from
    seed 0.  The loss must drop and the 4-process run must match the single-process replay of the same
    seeded routing."""
    extra = ["--model.parameter_sharing", "true", "--data.seq_length", "128", "--data.num_examples", "400",
             "--train.max_steps", "20", "--train.batch_size", "16", "--train.micro_batch_size", "4",
             "--train.outer_optimizer.type", "SGD", "--train.outer_optimizer.lr", "0.7",
             "--train.outer_optimizer.momentum", "0.9", "--train.outer_optimizer.nesterov", "true",
             "--swarm.sync_every_n_steps", "10"]
    launch("config1", 4, 2, extra, timeout=400)
    got = global_losses("config1")
    want = virtual_losses(4, 2, steps=20, model={"parameter_sharing": True},
                          data={"seq_length": 128},
                          train={"outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}},
                          swarm={"sync_every_n_steps": 10})
    assert len(got) == len(want) == 2                       # global metrics on the sync steps 10 and 20
    assert got[1] < got[0]
    assert max(abs(a - b) for a, b in zip(got, want)) < 5e-3, (got, want)
    local = open(f"{LOG}/config1/1.log").read()             # the master's own (local) curve, every step
    import re as _re
    curve = [float(x) for x in _re.findall(r"'train/local/loss/current': ([\d.]+)", local)]
    assert len(curve) == 20 and min(curve[-3:]) < curve[0]
