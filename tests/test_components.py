"""Unit tests of the host-side components (metrics, checkpoint, data, model split, optimiser maths)."""
import math
import os

import pytest
import torch

from helpers import make_config, single_world


def test_metrics_keys_and_semantics():
    from diloco_swarm_b200.utils.metrics import Outputs, aggregate_outputs, train_metrics
    m = train_metrics("train/global")
    m.update(Outputs(step=1, time=2.0, loss=1.0, tokens=100, num_micro_batches=4, lr=1e-3, norm=0.5, micro_step_time=0.5))
    m.update(Outputs(step=2, time=1.0, loss=2.0, tokens=100, num_micro_batches=4, lr=1e-3, norm=0.7, micro_step_time=0.25))
    out = m.compute()
    assert out["train/global/step/current"] == 2
    assert out["train/global/throughput/current"] == 100.0 and out["train/global/throughput/average"] == 75.0
    assert out["train/global/tokens/total"] == 200 and out["train/global/num_micro_batches/current"] == 8
    # perplexity average = mean of per-update exp(loss), not exp(mean loss)
    assert abs(out["train/global/perplexity/average"] - (math.e + math.e ** 2) / 2) < 1e-9
    a = Outputs(step=3, time=1.0, loss=2.0, tokens=10, num_micro_batches=1, lr=0.1, norm=1.0, micro_step_time=0.1)
    b = Outputs(step=3, time=3.0, loss=0.0, tokens=0, num_micro_batches=0, lr=0.1, norm=None, micro_step_time=0.3)
    agg = aggregate_outputs(a, [a, b])
    assert agg.tokens == 10 and agg.time == 2.0 and agg.loss == 2.0 and agg.norm == 1.0   # zeros and None are ignored
    v = Outputs.from_vector(b.to_vector())
    assert v.norm is None and v.tokens == 0 and v.time == 3.0


def test_checkpoint_layout_and_roundtrip(tmp_path):
    from diloco_swarm_b200.utils.ckpt import Checkpoint
    ck = Checkpoint(str(tmp_path / "checkpoints"))
    model = torch.nn.Linear(4, 3)
    p = ck.save(7, model)
    assert p.endswith(os.path.join("step_7", "model.pt"))
    ck.save(12, model)
    assert ck.get_latest_step() == 12
    sd = ck.load(7)
    assert torch.equal(sd["weight"], model.weight.detach())
    with pytest.raises(ValueError):
        ck.load(99)

    class W:
        world_size, local_rank = 4, 3
    ck.setup(W())
    assert ck.save(1, model).endswith(os.path.join("step_1", "model.3.pt"))
    ck.save_extra(1, "optim", {"opt_steps": 5})
    assert ck.load_extra(1, "optim")["opt_steps"] == 5 and ck.load_extra(1, "outer") is None
    ck.save_meta(1, {"step": 1})
    assert ck.load_meta(1)["step"] == 1


def test_data_pipeline():
    from diloco_swarm_b200.utils import data as D
    tok = D.ByteTokenizer()
    t = D.tokenize("I am", tok, max_length=8)
    assert t["input_ids"].tolist() == [[73, 32, 97, 109] + [50256] * 4] and t["attention_mask"].sum() == 4
    cfg = make_config(data={"path": "memorize", "seq_length": 16, "num_examples": 10}).data
    ds = D.get_dataset(cfg, tok, seed=0)
    assert len(ds) == 10 and ds.input_ids.shape == (10, 17)
    tr, va = ds.train_test_split(0.2, seed=1)
    assert len(tr) == 8 and len(va) == 2
    b = D.collate(ds, 0, 4)
    assert torch.equal(b["input_ids"][:, 1:], b["target_ids"][:, :-1]) and b["attention_mask"].shape == (4, 16)
    z1, z2 = D.zipf_tokens(64, 33, 50257, 1.0, 0), D.zipf_tokens(64, 33, 50257, 1.0, 0)
    assert torch.equal(z1, z2) and int(z1.max()) < 50257 and (z1 == 0).float().mean() > 0.05
    loader = D.BatchLoader(ds, 4)
    assert len(loader) == 2 and len(list(loader)) == 2       # drop_last
    assert D.get_num_steps(40, 1, 1000, 10) == 40 and D.get_num_steps(-1, 2, 100, 10) == 20
    assert D.micro_batch_rows(3, 4) == slice(12, 16)


def test_layer_split_and_shard_equivalence():
    from diloco_swarm_b200.models.gpt2 import GPT2Config, TorchStage, num_parameters, split_layers
    assert split_layers(12, 2) == [list(range(6)), list(range(6, 12))]
    assert split_layers(7, 3) == [[0, 1, 2], [3, 4], [5, 6]]            # remainder to the first stages
    assert split_layers(12, 2, "8,4")[1] == [8, 9, 10, 11]
    assert sum(len(x) for x in split_layers(24, 4, "balanced", 1024)) == 24
    cfg = GPT2Config(n_layer=4, n_head=4, n_embd=64, vocab_size=256, block_size=32)
    full = TorchStage(cfg)
    assert full.num_parameters() == num_parameters(cfg)
    ids = torch.randint(0, 256, (2, 16))
    for S_ in (2, 4):
        x = None
        for s in range(S_):
            st = TorchStage(cfg, s, S_)
            x = st(input_ids=ids if s == 0 else None, hidden_states=x)
        assert torch.allclose(x, full(input_ids=ids), atol=1e-5)
    # stage-local block numbering in the state dict (reference checkpoint layout)
    keys = list(TorchStage(cfg, 1, 2).state_dict().keys())
    assert keys[0] == "transformer.h.0.ln_1.weight" and keys[-1] == "lm_head.weight"


def test_lr_schedule_and_nesterov_reference():
    from diloco_swarm_b200.optim import lr_factor, nesterov_reference
    c = make_config(train={"scheduler": {"enable": True, "num_warmup_steps": 10}}).train.scheduler
    assert lr_factor(0, c, 100) == 0.0 and lr_factor(5, c, 100) == 0.5 and lr_factor(50, c, 100) == 1.0
    c = make_config(train={"scheduler": {"enable": True, "num_warmup_steps": 10, "type": "cosine"}}).train.scheduler
    assert abs(lr_factor(10, c, 110) - 1.0) < 1e-9 and abs(lr_factor(110, c, 110) - 0.1) < 1e-9
    p = torch.nn.Parameter(torch.randn(100))
    opt = torch.optim.SGD([p], lr=0.7, momentum=0.9, nesterov=True)
    theta, buf = p.detach().clone(), None
    for _ in range(3):
        g = torch.randn(100)
        p.grad = g.clone()
        opt.step()
        theta, buf = nesterov_reference(theta, g, buf, 0.7, 0.9)
    assert torch.allclose(theta, p.detach(), atol=1e-6)


def test_torch_engine_diloco_single_replica():
    from diloco_swarm_b200.models.engine_torch import TorchEngine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    cfg = make_config(train={"outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}})
    mc = cfg.model
    eng = TorchEngine(GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer,
                                 n_head=mc.n_head, n_embd=mc.n_embd), single_world(), cfg, torch.device("cpu"))
    ids = torch.randint(0, 500, (2, 17))
    theta0 = [p.detach().clone() for p in eng.model.parameters()]
    for _ in range(2):
        eng.forward_backward(0, ids[:, :-1], None, ids[:, 1:], torch.ones(2, 16, dtype=torch.long), 1.0)
        eng.optimizer_step(1e-3, 1.0)
        eng.zero_grad()
    inner = [p.detach().clone() for p in eng.model.parameters()]
    eng.outer_step()
    for p, t0, ti in zip(eng.model.parameters(), theta0, inner):
        d = t0 - ti
        assert torch.allclose(p.detach(), t0 - 0.7 * (d + 0.9 * d), atol=1e-6)


def test_comm_model_reproduces_the_notebook_figures():
    from diloco_swarm_b200.utils.comm_model import cumulative, run_cost, summary
    s = summary("small")
    assert abs(s["pp_gb_per_step"] - 12.88) < 0.01 and abs(s["dp_gb_per_sync"] - 1.08) < 1e-6
    c = run_cost(100, 2, 4, 2048, 1024, 768, 180e6, sync_every_n_steps=50)
    assert c.syncs == 2 and abs(cumulative(c, 50)[-1] - c.total) < 1e-3
    ours = run_cost(100, 2, 4, 2048, 1024, 768, 180e6, 50, pp_bytes_per_value=2)
    ref = run_cost(100, 2, 4, 2048, 1024, 768, 180e6, 50, pp_bytes_per_value=4, metadata_plane=True)
    assert abs(ref.pp_per_step / ours.pp_per_step - 4.0) < 1e-9     # bf16 payload, no metadata plane


def test_phase_timer_on_cpu():
    import time
    from diloco_swarm_b200.utils.timers import PhaseTimer
    t = PhaseTimer(torch.device("cpu"))
    with t.phase("a"):
        time.sleep(0.01)
    with t.phase("a"):
        time.sleep(0.01)
    out = t.collect()
    assert out["a"] >= 15 and t.collect() == {}


def test_serializer_and_micro_batch_naming():
    from diloco_swarm_b200.parallel.serializer import HEADER_BYTES, Serializer
    from diloco_swarm_b200.utils.data import get_micro_batches
    s = Serializer((2, 3, 4))
    x = torch.randn(2, 3, 4)
    msg = s.serialize(x, (5, 7))
    assert msg.numel() == HEADER_BYTES + x.numel() * 4          # a header, not a second plane
    y, meta = s.deserialize(msg)
    assert torch.equal(x, y) and meta == (5, 7)
    batch = {"input_ids": torch.arange(32).view(8, 4)}
    got = [(r, l, mb["input_ids"][0, 0].item()) for r, l, mb in get_micro_batches(batch, 2, [0, 2])]
    # rank 0 owns chunks 0 and 2 (rows 0-1, 4-5), rank 2 owns chunks 1 and 3: [k*R*mbs + i*mbs, +mbs)
    assert got == [(0, 1, 0), (2, 1, 8), (0, 2, 16), (2, 2, 24)]


def test_reference_named_helpers():
    """Helpers that exist under the reference's names: the row sampler states the same partition as the
    microbatch slices, the module-level DiLoCo helpers reproduce torch's SGD-Nesterov on pseudo-gradients,
    the factories build what the trainer builds."""
    import torch
    from helpers import make_config
    from diloco_swarm_b200 import optim as O
    from diloco_swarm_b200.train import get_model, get_sharded_model
    from diloco_swarm_b200.utils import data as D
    from diloco_swarm_b200.utils.misc import get_eval_pbar_description, get_train_pbar_description
    from diloco_swarm_b200.utils.metrics import Outputs, train_metrics
    from diloco_swarm_b200.world import World

    batch = {"input_ids": torch.arange(22).view(11, 2), "attention_mask": None}
    ds = D.BatchData(batch)
    assert len(ds) == 11 and ds[3]["input_ids"].tolist() == [6, 7] and ds[3]["attention_mask"] is None
    ranks = [0, 2, 4]
    rows = {r: list(D.BatchSampler(ds, r, ranks, 2)) for r in ranks}
    assert rows == {0: [0, 1, 6, 7], 2: [2, 3, 8, 9], 4: [4, 5, 10]}
    assert [len(D.BatchSampler(ds, r, ranks, 2)) for r in ranks] == [4, 4, 3]
    for root, k, mb in D.get_micro_batches({"input_ids": torch.arange(24).view(12, 2)}, 2, ranks):
        want = rows[root][2 * (k - 1): 2 * k] if root != 4 or k == 1 else [10, 11]
        assert (mb["input_ids"][:, 0] // 2).tolist() == want

    cfg = make_config(model={"n_layer": 2, "n_head": 2, "n_embd": 32, "vocab_size": 64, "block_size": 16})
    whole = get_model(cfg.model, seed=3)
    import os
    os.environ.update(RANK="1", WORLD_SIZE="2")
    try:
        w = World(2, init=False)          # rank 1 of 2: the second pipeline stage
    finally:
        os.environ.pop("RANK"); os.environ.pop("WORLD_SIZE")
    part = get_sharded_model(cfg.model, w, seed=3)
    assert part.is_last and not part.is_first
    sd = whole.state_dict()
    first_block = part.layers[0]                      # state-dict block numbers are local to the stage
    for k, v in part.state_dict().items():
        bits = k.split(".")
        if bits[1] == "h":
            bits[2] = str(int(bits[2]) + first_block)
        assert torch.equal(v, sd[".".join(bits)]), k

    inner = torch.nn.Linear(4, 3)
    outer = O.get_outer_model(inner)
    opt = torch.optim.SGD(outer.parameters(), lr=0.7, momentum=0.9, nesterov=True)
    theta, buf = outer.weight.detach().clone(), None
    for _ in range(3):
        with torch.no_grad():
            inner.weight.add_(torch.randn_like(inner.weight) * 0.1)
        O.compute_pseudo_gradient(inner, outer)
        theta, buf = O.nesterov_reference(theta, outer.weight.grad.clone(), buf, 0.7, 0.9)
        opt.step()
        O.sync_inner_model(outer, inner)
        assert torch.allclose(inner.weight, theta, atol=1e-6)
    sched = O.get_scheduler(O.get_optimizer(inner, cfg.train.inner_optimizer), cfg.train.scheduler)
    assert sched.get_last_lr()[0] <= cfg.train.inner_optimizer.lr

    m = train_metrics("train/global")
    m.update(Outputs(step=1, lr=1e-3, loss=2.0, tokens=10, norm=0.5, time=1.0, micro_step_time=0.5, num_micro_batches=2))
    assert "Loss: 2.0000" in get_train_pbar_description(m, "[TRAIN]")
    assert "Avg. Loss: 2.0000" in get_eval_pbar_description(m, "[EVAL]")


def test_pipeline_timing_model():
    """The timing model replays the trainer's own routing and plans: closed forms for the trivial worlds,
    more microbatches in flight never slow a pipeline down, balanced routing beats uniform on average."""
    from diloco_swarm_b200.benchmarks.pipeline_model import simulate
    one = simulate(1, 1, 8, 1, [2.0], [4.0], steps=3)
    assert abs(one["step_ms_mean"] - 8 * 6.0) < 1e-9 and abs(one["busiest_rank_utilisation"] - 1.0) < 1e-9
    # two equal stages, one replica each: with enough microbatches in flight only the fill and the drain are lost
    deep = simulate(2, 1, 16, 16, [1.0, 1.0], [2.0, 2.0], steps=2)["step_ms_mean"]
    assert 16 * 3.0 < deep <= 16 * 3.0 + 2 * 3.0 + 1e-9
    shallow = simulate(2, 1, 16, 1, [1.0, 1.0], [2.0, 2.0], steps=2)["step_ms_mean"]
    assert abs(shallow - 16 * 6.0) < 1e-9            # one in flight: the stages take turns
    prev = None
    for cap in (1, 2, 4, 8):
        t = simulate(2, 2, 16, cap, [1.0, 1.1], [2.0, 2.1], xfer=0.05, steps=20)["step_ms_mean"]
        assert prev is None or t <= prev + 1e-9
        prev = t
    uni = simulate(2, 4, 32, 8, [1.0, 1.0], [2.0, 2.0], routing="uniform", steps=60)
    bal = simulate(2, 4, 32, 8, [1.0, 1.0], [2.0, 2.0], routing="balanced", steps=60)
    assert bal["step_ms_mean"] < uni["step_ms_mean"]
    assert abs(bal["busiest_last_stage_replica_vs_even_share"] - 1.0) < 1e-9 < uni["busiest_last_stage_replica_vs_even_share"] - 1.0
    # one last-stage replica at half speed: routing by throughput beats both
    speed = [1, 1, 1, 1, 1, 1, 1, 0.5]
    het = {m: simulate(2, 4, 32, 8, [1.0, 1.0], [2.0, 2.0], routing=m, steps=60, speed=speed)["step_ms_mean"]
           for m in ("uniform", "balanced", "weighted")}
    assert het["weighted"] < 0.9 * min(het["uniform"], het["balanced"])


def test_local_token_and_text_datasets(tmp_path):
    """tokens:<file.npy> (memory-mapped, lazy split) and text:<file.txt>, and the tool that makes the former."""
    import numpy as np
    from diloco_swarm_b200.config import DataConfig
    from diloco_swarm_b200.utils import data as D
    tok = D.ByteTokenizer()
    lines = ["hello world", "", "a second line that is longer than the row", "x"]
    text = tmp_path / "t.txt"
    text.write_text("\n".join(lines) + "\n")
    n, width = D.prepare_tokens(str(text), str(tmp_path / "a.npy"), 16, tok)
    assert (n, width) == (3, 17)
    ds = D.get_dataset(DataConfig(path=f"tokens:{tmp_path / 'a.npy'}", seq_length=16), tok, seed=0)
    assert isinstance(ds, D.MappedTokenDataset) and len(ds) == 3
    ids, mask = ds.rows(0, 3)
    assert ids.dtype == torch.long and mask.sum(1).tolist() == [11, 17, 1]
    assert tok.decode(ids[0][:11]) == "hello world" and int(ids[2, 1]) == tok.pad_token_id
    # the same rows from the text file directly
    ds_t = D.get_dataset(DataConfig(path=f"text:{text}", seq_length=16), tok, seed=0)
    assert torch.equal(ds_t.input_ids, ids) and torch.equal(ds_t.attention_mask, mask)
    # split and select permute an index, the matrix stays on disk; rows come back in index order
    tr, te = ds.train_test_split(0.34, seed=1)
    assert len(tr) == 2 and len(te) == 1 and sorted(tr.index.tolist() + te.index.tolist()) == [0, 1, 2]
    assert tr.ids is ds.ids
    assert torch.equal(tr.rows(0, 2)[0], ids[torch.from_numpy(tr.index)])
    b = D.collate(tr, 0, 2)
    assert b["input_ids"].shape == (2, 16) and torch.equal(b["target_ids"][:, :-1], b["input_ids"][:, 1:])
    # a row narrower than seq_length + 1 is refused
    with pytest.raises(ValueError):
        D.load_token_file(str(tmp_path / "a.npy"), 18)
    # packed: one stream cut into full rows, no padding and no mask file
    n2, w2 = D.prepare_tokens(str(text), str(tmp_path / "b.npy"), 7, tok, pack=True)
    stream = sum((list(l.encode()) + [tok.eos_token_id] for l in lines if l), [])
    assert (n2, w2) == (len(stream) // 8, 8) and not (tmp_path / "b.mask.npy").exists()
    packed = D.load_token_file(str(tmp_path / "b.npy"), 8)
    assert packed.rows(0, n2)[0].reshape(-1).tolist() == stream[:n2 * 8] and int(packed.rows(0, 1)[1].min()) == 1
    assert np.load(tmp_path / "b.npy").dtype == np.int32


def test_hub_dataset_from_the_local_cache(tmp_path, monkeypatch):
    """Datasets named like the reference's hub ids (src/utils.py:88-100) load from the on-disk cache under
    $PERSISTENT_DIR/huggingface without a network: pre-tokenised rows as they are, text rows through the
    tokenizer when data.tokenize is set."""
    datasets = pytest.importorskip("datasets")
    from diloco_swarm_b200.config import DataConfig
    from diloco_swarm_b200.utils import data as D
    monkeypatch.setenv("PERSISTENT_DIR", str(tmp_path))
    tok = D.ByteTokenizer()
    rows = torch.randint(0, 1000, (6, 17), generator=torch.Generator().manual_seed(0))
    mask = torch.ones_like(rows)
    mask[2, 10:] = 0
    pre = datasets.DatasetDict({"train": datasets.Dataset.from_dict(
        {"input_ids": rows.tolist(), "attention_mask": mask.tolist()})})
    pre.save_to_disk(str(tmp_path / "huggingface" / "someone" / "pretokenized"))
    ds = D.get_dataset(DataConfig(path="someone/pretokenized", seq_length=16), tok, seed=0)
    assert len(ds) == 6 and torch.equal(ds.input_ids, rows) and torch.equal(ds.attention_mask, mask)
    text = datasets.DatasetDict({"train": datasets.Dataset.from_dict({"text": ["hello", "a longer line of text"]})})
    text.save_to_disk(str(tmp_path / "huggingface" / "someone" / "raw"))
    ds = D.get_dataset(DataConfig(path="someone/raw", seq_length=8, tokenize=True), tok, seed=0)
    assert ds.input_ids.shape == (2, 9) and ds.attention_mask.sum(1).tolist() == [5, 9]
    assert tok.decode(ds.input_ids[0][:5]) == "hello"
    half = D.get_dataset(DataConfig(path="someone/pretokenized", seq_length=16, subset_size=0.5), tok, seed=0)
    assert len(half) == 3


def test_wandb_run_per_rank_in_offline_mode(tmp_path, monkeypatch):
    """logging.wandb.enable (src/logger.py:50-58): one run per rank, grouped by the run id, fed by
    log_config / log_world / log_metrics; wandb's offline mode stands in for the service."""
    pytest.importorskip("wandb")
    from diloco_swarm_b200.config import LoggingConfig
    from diloco_swarm_b200.utils.logger import Logger
    monkeypatch.setenv("WANDB_MODE", "offline")
    monkeypatch.setenv("WANDB_SILENT", "true")
    lc = LoggingConfig(log_dir=str(tmp_path), run_id="w", console={"log_level": "ERROR"},
                       wandb={"enable": True, "project": "diloco-swarm", "tags": "bench,b200"})
    assert lc.wandb.tags == ["bench", "b200"]
    world = single_world()
    lg = Logger(world, lc)
    assert lg.wandb_run is not None and lg.wandb_run.group == "w" and lg.wandb_run.name == "rank0"
    lg.log_config(make_config())
    lg.log_world(world)
    lg.log_metrics({"train/global/loss/current": 1.0}, step=1, master=True)
    lg.log_metrics({"train/local/loss/current": 1.5}, step=1, master=False)
    assert lg.wandb_run.config["model"]["n_layer"] == make_config().model.n_layer
    assert lg.wandb_run.config["world"]["world_size"] == 1
    lg.close()
    assert lg.wandb_run is None
    assert any(d.startswith("offline-run") for d in os.listdir(tmp_path / "w" / "wandb"))


def test_dropout_is_applied_by_the_autograd_stage_in_training_only():
    """model.dropout (reference: src/model.py:48-49,67,86,114): active in training mode, off in evaluation,
    and a model built with dropout = 0 is unaffected."""
    import torch
    from diloco_swarm_b200.models.gpt2 import GPT2Config, TorchStage
    cfg = dict(block_size=32, vocab_size=64, n_layer=2, n_head=2, n_embd=32)
    ids = torch.randint(0, 64, (2, 16))
    plain, drop = TorchStage(GPT2Config(**cfg)), TorchStage(GPT2Config(**cfg, dropout=0.5))
    drop.eval(); plain.eval()
    assert torch.equal(drop(input_ids=ids), plain(input_ids=ids))          # same seeded weights, dropout off
    drop.train(); plain.train()
    a, b = drop(input_ids=ids), drop(input_ids=ids)
    assert not torch.equal(a, b)                                             # fresh masks per call
    assert torch.equal(plain(input_ids=ids), plain(input_ids=ids))


def test_stage_rendezvous_is_a_no_op_without_replicas():
    import torch
    from diloco_swarm_b200.parallel.collectives import StageRendezvous, wait_cycles_for
    r = StageRendezvous(None, torch.device("cpu"))
    r.meet()
    assert r.count == 0
    assert wait_cycles_for(2.0) == 4_000_000_000 and wait_cycles_for(0.0) == 1
