"""This framework's host-side components against the reference's own code, on CPU.

The unmodified reference is installed under ``baseline/_ref`` for the benchmark's reference arm.  Where it
is present, its classes serve as the oracle here: the same weights give the same logits, the same loss,
the same parameters after optimiser steps, the same DiLoCo outer step, the same layer split, the same
microbatch partition, learning-rate schedule and metric values.  Skipped when the install is missing.
"""
import math
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _import_reference():
    if not os.path.isdir(os.path.join(REF, "src")):
        pytest.skip("baseline/_ref is not installed")
    sys.modules.setdefault("autorootcwd", types.ModuleType("autorootcwd"))      # only changes directory
    try:
        import pydantic_config
        if not hasattr(pydantic_config, "parse_argv"):
            pydantic_config.parse_argv = lambda: {}                                # imported, never called here
        if REF not in sys.path:
            sys.path.insert(0, REF)
        import src.ckpt as rckpt
        import src.config as rc
        import src.metrics as rm
        import src.model as rmodel
        import src.sampler as rs
        import src.utils as ru
    except Exception as e:                                                         # missing optional packages
        pytest.skip(f"the reference does not import here: {type(e).__name__}: {e}")
    return types.SimpleNamespace(ckpt=rckpt, config=rc, metrics=rm, model=rmodel, sampler=rs, utils=ru)


@pytest.fixture(scope="module")
def ref():
    return _import_reference()


def _pair(ref, tied=False, n_layer=2):
    """The reference's model and ours holding the same weights."""
    from diloco_swarm_b200.models.gpt2 import GPT2Config, TorchStage
    kw = dict(block_size=64, vocab_size=512, n_layer=n_layer, n_head=4, n_embd=64, dropout=0.0, bias=True,
              parameter_sharing=tied)
    torch.manual_seed(0)
    theirs = ref.model.GPT2(ref.model.GPT2Config(**kw))
    ours = TorchStage(GPT2Config(**kw), 0, 1)
    assert set(ours.state_dict()) == set(theirs.state_dict())
    ours.load_state_dict(theirs.state_dict())
    return theirs, ours


@pytest.mark.parametrize("tied", [False, True])
def test_same_weights_same_logits(ref, tied):
    theirs, ours = _pair(ref, tied)
    ids = torch.randint(0, 512, (3, 33), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        a, b = theirs(ids), ours(input_ids=ids)
    assert a.shape == b.shape == (3, 33, 512) and torch.allclose(a, b, atol=1e-6, rtol=0)
    assert ours.num_parameters() == theirs.num_parameters()


@pytest.mark.parametrize("kind", ["AdamW", "SGD", "nesterov"])
def test_masked_loss_and_optimiser_steps(ref, kind):
    """Three steps of forward, masked loss, backward, clipping and the optimiser: AdamW (weight decay on
    every tensor), SGD with momentum, SGD-Nesterov (src/utils.py:59-65)."""
    from diloco_swarm_b200.config import OptimizerConfig
    from diloco_swarm_b200.optim import get_optimizer
    theirs, ours = _pair(ref)
    kw = dict(type="AdamW", lr=1e-2) if kind == "AdamW" else dict(type="SGD", lr=1e-2, nesterov=kind == "nesterov")
    opt_t = ref.utils.get_optimizer(theirs, ref.config.OptimizerConfig(**kw))
    opt_o = get_optimizer(ours, OptimizerConfig(**kw))
    if kind == "AdamW":
        assert opt_o.defaults["weight_decay"] == opt_t.defaults["weight_decay"] == 0.1
        assert tuple(opt_o.defaults["betas"]) == tuple(opt_t.defaults["betas"]) == (0.9, 0.95)
    else:
        assert {k: opt_o.defaults[k] for k in ("momentum", "nesterov", "weight_decay")} == \
            {k: opt_t.defaults[k] for k in ("momentum", "nesterov", "weight_decay")}
    g = torch.Generator().manual_seed(2)
    loss_fn = torch.nn.CrossEntropyLoss()
    for _ in range(3):
        ids = torch.randint(0, 512, (4, 17), generator=g)
        mask = (torch.rand(4, 16, generator=g) > 0.3).long()
        inp, tgt = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()      # as the reference's collate_batch
        la = loss_fn(*ref.utils.filter_logits_targets(theirs(inp), tgt, mask))
        logits = ours(input_ids=inp)
        keep = mask.reshape(-1).bool()
        lb = torch.nn.functional.cross_entropy(logits.reshape(-1, 512)[keep], tgt.reshape(-1)[keep])
        assert torch.allclose(la, lb, atol=1e-6)
        for model, loss, opt in ((theirs, la, opt_t), (ours, lb, opt_o)):
            opt.zero_grad()
            loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step()
    sa, sb = theirs.state_dict(), ours.state_dict()
    assert all(torch.allclose(sa[k], sb[k], atol=1e-6) for k in sa)


def test_diloco_outer_step_matches_the_reference_helpers(ref):
    """One replica: H inner steps, then pseudo-gradient, outer SGD-Nesterov and copy back, done with the
    reference's helpers (src/utils.py:213-226) and with this framework's autograd engine."""
    from helpers import make_config, single_world
    from diloco_swarm_b200.models.engine_torch import TorchEngine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    kw = dict(block_size=64, vocab_size=512, n_layer=2, n_head=4, n_embd=64, dropout=0.0, bias=True, parameter_sharing=False)
    cfg = make_config(model={k: kw[k] for k in ("block_size", "vocab_size", "n_layer", "n_head", "n_embd")},
                      train={"inner_optimizer": {"type": "AdamW", "lr": 1e-2},
                             "outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}},
                      swarm={"num_stages": 1}, amp={"enable": False})
    eng = TorchEngine(GPT2Config(**kw), single_world(), cfg, torch.device("cpu"))
    inner = ref.model.GPT2(ref.model.GPT2Config(**kw))
    inner.load_state_dict(eng.model.state_dict())
    eng.reset_outer()
    outer = ref.utils.get_outer_model(inner)
    opt_in = ref.utils.get_optimizer(inner, ref.config.OptimizerConfig(type="AdamW", lr=1e-2))
    opt_out = ref.utils.get_optimizer(outer, ref.config.OptimizerConfig(type="SGD", lr=0.7, nesterov=True))
    g = torch.Generator().manual_seed(3)
    loss_fn = torch.nn.CrossEntropyLoss()
    for round_ in range(2):                       # two outer steps, so that the momentum buffer matters
        for _ in range(2):
            ids = torch.randint(0, 512, (2, 17), generator=g)
            inp, tgt, mask = ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), torch.ones(2, 16, dtype=torch.long)
            opt_in.zero_grad()
            loss_fn(*ref.utils.filter_logits_targets(inner(inp), tgt, mask)).backward()
            torch.nn.utils.clip_grad_norm_(inner.parameters(), 1.0)
            opt_in.step()
            eng.train()
            eng.zero_grad()
            eng.forward_backward(0, inp, None, tgt, mask, 1.0)
            eng.optimizer_step(1e-2, 1.0)
        ref.utils.compute_pseudo_gradient(inner, outer)
        opt_out.step()
        opt_out.zero_grad()
        ref.utils.sync_inner_model(outer, inner)
        eng.outer_step()
        sa, sb = inner.state_dict(), eng.model.state_dict()
        assert all(torch.allclose(sa[k], sb[k], atol=2e-6) for k in sa), round_


@pytest.mark.parametrize("n_layer,stages", [(12, 2), (12, 5), (4, 3), (24, 4)])
def test_layer_split_and_stage_shards(ref, n_layer, stages):
    """Block ranges per stage as ShardedGPT2.distribute_layers gives them (src/model.py:195-198), and for
    the small cases the stage modules themselves: a stage of ours holds the tensors of the reference's shard
    under the same (stage-local) names."""
    from diloco_swarm_b200.models.gpt2 import GPT2Config, TorchStage, split_layers
    ours = split_layers(n_layer, stages, "even")
    for s in range(stages):
        w = types.SimpleNamespace(num_stages=stages, stage=s)
        assert ours[s] == ref.model.ShardedGPT2.distribute_layers(None, w, n_layer)
    if n_layer <= 4:
        kw = dict(block_size=32, vocab_size=256, n_layer=n_layer, n_head=2, n_embd=32, dropout=0.0, bias=True,
                  parameter_sharing=False)
        for s in range(stages):
            w = types.SimpleNamespace(num_stages=stages, stage=s, is_first_stage=s == 0, is_last_stage=s == stages - 1)
            shard = ref.model.ShardedGPT2(ref.model.GPT2(ref.model.GPT2Config(**kw)), w)
            mine = TorchStage(GPT2Config(**kw), s, stages)
            theirs = {k: tuple(v.shape) for k, v in shard.state_dict().items()}
            assert {k: tuple(v.shape) for k, v in mine.state_dict().items()} == theirs


def test_microbatch_partition_and_sampler(ref):
    """Rows of a batch per first-stage rank: the reference's BatchSampler (src/sampler.py:16-39) and ours."""
    from diloco_swarm_b200.utils import data as D
    batch = {"input_ids": torch.arange(22 * 3).reshape(22, 3)}
    for ranks, mbs in (([0, 2, 4], 4), ([0], 8), ([1, 3], 2)):
        for r in ranks:
            a = list(ref.sampler.BatchSampler(ref.sampler.BatchData(batch), r, ranks, mbs))
            b = list(D.BatchSampler(D.BatchData(batch), r, ranks, mbs))
            assert a == b, (ranks, mbs, r)


def test_learning_rate_schedule(ref):
    from diloco_swarm_b200.config import SchedulerConfig
    from diloco_swarm_b200.optim import lr_factor
    p = [torch.nn.Parameter(torch.zeros(1))]
    opt = torch.optim.SGD(p, lr=1.0)
    sched = ref.utils.get_scheduler(opt, ref.config.SchedulerConfig(enable=True, num_warmup_steps=5))
    ours = SchedulerConfig(enable=True, num_warmup_steps=5)
    for step in range(12):
        assert sched.get_last_lr()[0] == pytest.approx(lr_factor(step, ours, 100))
        opt.step()
        sched.step()


def test_metric_values(ref):
    """The same sequence of step outputs through the reference's Metrics and ours: same keys, same values
    (perplexity averaged arithmetically, throughput = tokens / time, totals and running means)."""
    from diloco_swarm_b200.utils import metrics as M
    rm = ref.metrics
    theirs = rm.Metrics([rm.Step(), rm.Time(), rm.MicroTime(), rm.Tokens(), rm.NumMicroBatches(), rm.Norm(), rm.Loss(),
                         rm.Perplexity(), rm.Throughput(), rm.LearningRate()], name="train/global")
    ours = M.train_metrics("train/global")
    e_t = rm.Metrics([rm.Throughput(), rm.Loss(), rm.Perplexity()], name="eval")
    e_o = M.eval_metrics("eval")
    for step in range(1, 5):
        kw = dict(step=step, time=0.5 + 0.1 * step, loss=3.0 / step, tokens=4096 * step, num_micro_batches=4,
                  lr=1e-3 * step, norm=1.0 + step, micro_step_time=0.05 * step)
        theirs.update(rm.Outputs(**kw))
        ours.update(M.Outputs(**kw))
        e_t.update(rm.Outputs(step=step, time=kw["time"], loss=kw["loss"], tokens=kw["tokens"]))
        e_o.update(M.Outputs(step=step, time=kw["time"], loss=kw["loss"], tokens=kw["tokens"]))
        for a, b in ((theirs.compute(), ours.compute()), (e_t.compute(), e_o.compute())):
            assert set(a) == set(b)
            for k in a:
                assert (a[k] is None and b[k] is None) or a[k] == pytest.approx(b[k]), k
    assert ours.compute()["train/global/perplexity/average"] == pytest.approx(
        sum(math.exp(3.0 / s) for s in range(1, 5)) / 4)


@pytest.mark.parametrize("world_size,local_rank", [(1, 0), (4, 3)])
def test_checkpoint_files_are_interchangeable(ref, tmp_path, world_size, local_rank):
    """A stage saved by the reference's Checkpoint is loaded by ours and the other way round: same
    directory and file names (src/ckpt.py:45-51), same state-dict keys."""
    from diloco_swarm_b200.utils.ckpt import Checkpoint
    theirs_model, ours_model = _pair(ref)
    world = types.SimpleNamespace(world_size=world_size, local_rank=local_rank)
    a, b = ref.ckpt.Checkpoint(str(tmp_path / "a")), Checkpoint(str(tmp_path / "a"))
    a.setup(world)
    b.setup(world)
    path = a.save(7, theirs_model)
    assert os.path.basename(path) == ("model.pt" if world_size == 1 else f"model.{local_rank}.pt")
    assert b.get_latest_step() == a.get_latest_step() == 7
    ours_model.load_state_dict(b.load(7))
    c, d = Checkpoint(str(tmp_path / "b")), ref.ckpt.Checkpoint(str(tmp_path / "b"))
    c.setup(world)
    d.setup(world)
    assert os.path.relpath(c.save(9, ours_model), tmp_path / "b") == os.path.relpath(path, tmp_path / "a").replace("step_7", "step_9")
    theirs_model.load_state_dict(d.load(9))


def test_every_reference_config_field_exists_with_its_default(ref):
    """The configuration schema (src/config.py:5-95): same classes, every field present, same defaults;
    fields that only this framework has are additions on top."""
    import diloco_swarm_b200.config as ours
    classes = [n for n in dir(ref.config) if n.endswith("Config") and n != "BaseConfig"]
    assert len(classes) >= 13
    for name in classes:
        theirs_cls, ours_cls = getattr(ref.config, name), getattr(ours, name)
        for field, info in theirs_cls.model_fields.items():
            assert field in ours_cls.model_fields, f"{name}.{field} is missing"
            a, b = info.default, ours_cls.model_fields[field].default
            if hasattr(a, "model_dump"):
                a, b = a.model_dump(), {k: v for k, v in b.model_dump().items() if k in a.model_dump()}
            assert repr(a) == repr(b), f"{name}.{field}: {a!r} vs {b!r}"
    # the comma-separated list of wandb tags (src/config.py:84-88)
    assert ours.WandbLoggingConfig(tags="a,b").tags == ref.config.WandbLoggingConfig(tags="a,b").tags == ["a", "b"]


def test_batching_helpers(ref):
    """collate_batch, get_micro_batches, get_num_steps, get_train_setup, the number formats and the
    progress texts (src/utils.py:107-182) against their counterparts."""
    from diloco_swarm_b200.utils import data as D
    from diloco_swarm_b200.utils import metrics as M
    from diloco_swarm_b200.utils import misc
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 1000, (12, 9), generator=g)
    mask = (torch.rand(12, 9, generator=g) > 0.2).long()
    theirs = ref.utils.collate_batch([{"input_ids": r.tolist(), "attention_mask": m.tolist()} for r, m in zip(ids, mask)])
    ours = D.collate(D.TokenDataset(ids, mask), 0, 12)
    assert set(theirs) == set(ours) and all(torch.equal(theirs[k], ours[k]) for k in theirs)
    # the (root rank, local micro step) naming of microbatches and their rows
    world = types.SimpleNamespace(first_stage_ranks=[0, 2, 4])
    a = {(r, s): mb for r, s, mb in ref.utils.get_micro_batches(theirs, 2, world)}
    b = {(r, s): mb for r, s, mb in D.get_micro_batches(ours, 2, [0, 2, 4])}
    assert set(a) == set(b) and all(torch.equal(a[k]["input_ids"], b[k]["input_ids"]) for k in a)
    for args in ((10, -1, 100, 8), (-1, 2, 100, 8), (10, 1, 100, 8), (1000, 3, 64, 16)):
        assert ref.utils.get_num_steps(*args) == D.get_num_steps(*args)
    assert ref.utils.get_train_setup(20, 64, 128, 8, 5000) == D.get_train_setup(20, 64, 128, 8, 5000)
    for n in (7, 999, 1000, 123456, 7_654_321, 12_345_678_901):
        assert ref.utils.format_int(n) == misc.format_int(n) and ref.utils.format_int(n, 1) == misc.format_int(n, 1)
    assert ref.utils.format_float(3.14159, 3) == misc.format_float(3.14159, 3)
    rm = ref.metrics
    tm = rm.Metrics([rm.Step(), rm.Time(), rm.MicroTime(), rm.Tokens(), rm.NumMicroBatches(), rm.Norm(), rm.Loss(),
                     rm.Perplexity(), rm.Throughput(), rm.LearningRate()], name="train/global")
    om = M.train_metrics("train/global")
    kw = dict(step=3, time=0.7, loss=2.5, tokens=8192, num_micro_batches=4, lr=1e-3, norm=1.5, micro_step_time=0.1)
    tm.update(rm.Outputs(**kw))
    om.update(M.Outputs(**kw))
    assert ref.utils.get_train_pbar_description(tm, "[TRAIN]") == misc.get_train_pbar_description(om, "[TRAIN]")
    assert ref.utils.get_eval_pbar_description(tm, "[EVAL]") == misc.get_eval_pbar_description(om, "[EVAL]")


@pytest.mark.parametrize("temperature,top_k", [(1.0, None), (0.7, 5), (1.3, 50)])
def test_single_process_sampler(ref, temperature, top_k):
    """GPT2.generate (src/model.py:160-175): with the same weights and the same random stream both
    samplers emit the same tokens."""
    theirs, ours = _pair(ref)
    prompt = torch.randint(0, 512, (3, 5), generator=torch.Generator().manual_seed(9))
    torch.manual_seed(11)
    a = theirs.generate(prompt.clone(), 12, temperature=temperature, top_k=top_k)
    torch.manual_seed(11)
    b = ours.generate(prompt.clone(), 12, temperature=temperature, top_k=top_k)
    assert torch.equal(a, b)


@pytest.mark.parametrize("is_master", [True, False])
def test_logger_files_and_lines(ref, tmp_path, is_master):
    """Same calls into the reference's Logger (src/logger.py:21-111) and ours: the same files with the same
    lines (timestamps aside; the reference's file format opens the rank tag with a doubled bracket).  Ours
    adds the metric history and the saved configuration next to them."""
    import re
    import src.logger as rl
    from helpers import make_config
    from diloco_swarm_b200.utils import logger as ol
    world = types.SimpleNamespace(rank=1, local_rank=1, world_size=2, num_stages=2, is_master=is_master)
    cfg = make_config()

    def drive(mod, log_dir):
        lc = (ref.config.LoggingConfig if mod is rl else type(cfg.logging))(
            log_dir=str(log_dir), run_id="run", console={"log_level": "ERROR"}, file={"log_level": "DEBUG"})
        lg = mod.Logger(world, lc)
        lg.log_message("hello", master=False, level=mod.Level.INFO)
        lg.log_message("to the master", master=True, level=mod.Level.WARNING)
        lg.log_config(cfg)
        lg.log_metrics({"train/local/loss/current": 1.5}, step=1, master=False)
        lg.log_metrics({"train/global/loss/current": 1.25}, step=1, master=True)
        lg.log_samples(["first sample", "second sample"], step=4)
        for h in [h for name in list(__import__("logging").root.manager.loggerDict) for h in
                  __import__("logging").getLogger(name).handlers if getattr(h, "baseFilename", "").startswith(str(log_dir))]:
            h.flush()
        return os.path.join(str(log_dir), "run")

    a, b = drive(rl, tmp_path / "theirs"), drive(ol, tmp_path / "ours")
    files = lambda root: sorted(os.path.relpath(os.path.join(d, f), root) for d, _, fs in os.walk(root) for f in fs)
    dirs = lambda root: sorted(os.path.relpath(os.path.join(d, x), root) for d, xs, _ in os.walk(root) for x in xs)
    # in the reference every rank writes samples/<step>.txt (all ranks, the same file at once); here the master does
    expected = set(files(a)) - (set() if is_master else {"samples/4.txt"})
    assert expected <= set(files(b)) and set(dirs(a)) <= set(dirs(b))
    assert set(files(b)) - set(files(a)) <= {"config.yaml", "metrics/1.jsonl", "metrics/master.jsonl"}
    norm = lambda path: [re.sub(r"^\[[^\]]*\]", "", line).replace("[[", "[") for line in open(path).read().splitlines()]
    for f in files(a):
        if f.endswith(".log"):
            assert norm(os.path.join(a, f)) == norm(os.path.join(b, f)), f
    if is_master:
        assert open(os.path.join(a, "samples/4.txt")).read() == open(os.path.join(b, "samples/4.txt")).read()


@pytest.mark.parametrize("world_size,stages", [(1, 1), (2, 1), (2, 2), (4, 2), (9, 3), (8, 2), (8, 4), (7, 3)])
def test_world_rank_arithmetic(ref, monkeypatch, world_size, stages):
    """Stage, leaders, master and neighbours of every rank (src/world.py:10-118), with the reference's
    process-group calls replaced by no-ops so that all ranks can be built in one process."""
    import src.world as rw
    from diloco_swarm_b200.world import World
    fake = types.SimpleNamespace(TCPStore=lambda **kw: None, init_process_group=lambda **kw: None,
                                 new_group=lambda *a, **kw: tuple(a[0]) if a else None, barrier=lambda: None)
    monkeypatch.setattr(rw, "dist", fake)
    for rank in range(world_size):
        for k, v in (("RANK", rank), ("LOCAL_RANK", rank), ("WORLD_SIZE", world_size), ("LOCAL_WORLD_SIZE", world_size),
                     ("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", 29400)):
            monkeypatch.setenv(k, str(v))
        theirs = rw.World(ref.config.SwarmConfig(num_stages=stages))
        ours = World(stages, init=False)
        for attr in ("rank", "local_rank", "world_size", "local_world_size", "master_addr", "master_port", "num_stages",
                     "stage", "is_first_stage", "is_last_stage", "is_leader", "is_master", "first_stage_leader",
                     "last_stage_leader", "first_stage_ranks", "has_next_stage", "has_prev_stage"):
            assert getattr(theirs, attr) == getattr(ours, attr), (rank, attr)
        # the reference keeps default dicts, which grow when a neighbour that does not exist is asked for
        assert {s: theirs.stage2ranks[s] for s in range(stages)} == ours.stage2ranks
        assert {s: theirs.stage2leader[s] for s in range(stages)} == ours.stage2leader
        if ours.has_next_stage:
            assert theirs.next_stage_leader == ours.next_stage_leader
        if ours.has_prev_stage:
            assert theirs.prev_stage_leader == ours.prev_stage_leader
        assert repr(theirs) == repr(ours) and dict(theirs) == dict(ours)


def _global_losses(master_log, key="train/global/loss/current"):
    import ast
    import re
    out = []
    for text in re.findall(r"Global metrics: (\{[^}]*\})", open(master_log).read()):
        m = ast.literal_eval(text)
        if key in m:
            out.append(m[key])
    return out


@pytest.mark.parametrize("name,nproc,stages,H,outer", [
    ("single", 1, 1, 1, "None"),            # one process
    ("pipeline", 2, 2, 1, "None"),          # two stages, one replica each
    ("diloco_dp", 2, 1, 2, "nesterov"),     # two replicas of one stage, DiLoCo with an outer step every 2 steps
    ("swarm", 4, 2, 1, "None"),             # 2 stages x 2 replicas, stochastic wiring, gradient sync every step
    ("sparse_sync", 2, 1, 2, "None"),       # no outer optimiser but H = 2: gradients are averaged on every second
                                            # step only and the replicas are never re-aligned (src/train.py:248-251)
])
def test_loss_curve_of_the_reference_itself(ref, tmp_path, name, nproc, stages, H, outer):
    """The reference's own training run (its main(), gloo, CPU) and this framework's, from the same starting
    weights on the same batches: the loss curves agree to float32 rounding.  The reference's start weights
    are saved by the probe and enter here as a step-0 checkpoint; the token file is laid out so that this
    framework's seeded shuffle-split yields the reference's row order."""
    import subprocess
    import numpy as np
    from diloco_swarm_b200.utils.data import zipf_tokens
    steps, batch, mbs, seq, eval_size, seed = 4, (16 if name == "swarm" else 8), 2, 32, 0.1, 42
    eval_every = 2 if name in ("single", "pipeline") else 0      # these two also evaluate: before, during, after
    ids = zipf_tokens(120, seq + 1, 50257, 1.0, seed=0).numpy().astype(np.int32)
    np.save(tmp_path / "ref_tokens.npy", ids)
    n = ids.shape[0]
    k = max(1, int(round(n * eval_size)))
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed)).numpy()
    mine = np.empty_like(ids)
    mine[perm[k:]], mine[perm[:k]] = ids[k:], ids[:k]
    np.save(tmp_path / "our_tokens.npy", mine)
    port = 29600 + 11 * (os.getpid() % 30) + {"single": 0, "pipeline": 2, "diloco_dp": 4, "swarm": 6, "sparse_sync": 8}[name]
    run = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1"]
    env = dict(os.environ, OMP_NUM_THREADS="1")
    p = subprocess.run(run + ["--master-port", str(port), os.path.join(ROOT, "tests", "reference_probe.py"),
                              "--tokens", str(tmp_path / "ref_tokens.npy"), "--out", str(tmp_path / "ref"),
                              "--stages", str(stages), "--steps", str(steps), "--batch", str(batch), "--mbs", str(mbs),
                              "--seq", str(seq), "--H", str(H), "--outer", outer, "--eval-size", str(eval_size),
                              "--eval-every", str(eval_every)],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    theirs = _global_losses(tmp_path / "ref" / "ref" / "master.log")
    ck = tmp_path / "ours" / "run" / "checkpoints" / "step_0"
    os.makedirs(ck)
    for r in range(nproc):
        torch.save(torch.load(tmp_path / "ref" / f"w0.{r}.pt"), ck / ("model.pt" if nproc == 1 else f"model.{r}.pt"))
    outer_toml = "@configs/optimizer/none.toml" if outer == "None" else "@configs/optimizer/nesterov.toml"
    p = subprocess.run(run + ["--master-port", str(port + 10), "-m", "diloco_swarm_b200.train",
                              "--swarm.num_stages", str(stages), "--swarm.sync_every_n_steps", str(H), "--device", "cpu",
                              "--amp.enable", "false", "--model", "@configs/model/gpt2-tiny.toml",
                              "--data.path", f"tokens:{tmp_path / 'our_tokens.npy'}", "--data.seq_length", str(seq),
                              "--train.inner_optimizer", "@configs/optimizer/adamw.toml", "--train.inner_optimizer.lr", "6e-4",
                              "--train.outer_optimizer", outer_toml, "--train.outer_optimizer.lr", "0.7",
                              "--train.max_steps", str(steps), "--train.max_epochs", "-1", "--train.batch_size", str(batch),
                              "--train.micro_batch_size", str(mbs), "--train.max_micro_batches", "2", "--train.seed", str(seed),
                              "--eval.enable", "true" if eval_every else "false", "--eval.every_n_steps",
                              str(eval_every if eval_every else -1), "--eval.eval_size", str(eval_size), "--sample.enable", "false",
                              # which replica serves a microbatch does not change the gradients; the logged loss is a
                              # mean over the replicas that saw data, so both sides must leave no replica empty:
                              # balanced routing here, a seeded draw that happens to do so in the probe
                              "--swarm.routing", "balanced",
                              "--ckpt.resume", "true", "--ckpt.step", "0", "--logging.log_dir", str(tmp_path / "ours"),
                              "--logging.run_id", "run", "--logging.console.log_level", "ERROR"],
                       cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-3000:]
    ours = _global_losses(tmp_path / "ours" / "run" / "master.log")
    assert len(theirs) == len(ours) == steps // H, (theirs, ours)
    assert max(abs(a - b) for a, b in zip(theirs, ours)) < 2e-4, (theirs, ours)
    assert theirs[-1] < theirs[0]
    # the rest of the step's global record: counters exactly, the gradient norm (of the master's stage,
    # before clipping) to rounding, which says the gradients themselves agree
    for key, tol in (("step", 0), ("tokens", 0), ("num_micro_batches", 0), ("learning_rate", 1e-12), ("norm", 1e-4)):
        a = _global_losses(tmp_path / "ref" / "ref" / "master.log", f"train/global/{key}/current")
        b = _global_losses(tmp_path / "ours" / "run" / "master.log", f"train/global/{key}/current")
        assert len(a) == len(b) == steps // H and all(abs(x - y) <= tol * max(1.0, abs(x)) for x, y in zip(a, b)), (key, a, b)
    if eval_every:
        ev_t = _global_losses(tmp_path / "ref" / "ref" / "master.log", "eval/loss/average")
        ev_o = _global_losses(tmp_path / "ours" / "run" / "master.log", "eval/loss/average")
        assert len(ev_t) == len(ev_o) >= 3 and max(abs(a - b) for a, b in zip(ev_t, ev_o)) < 2e-4, (ev_t, ev_o)
