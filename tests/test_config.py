import os

import pytest

from diloco_swarm_b200.config import Config, config_from_argv, parse_argv

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BASE = ["--model", "@configs/model/gpt2-tiny.toml", "--data", "@configs/data/memorize.toml",
        "--train.inner_optimizer", "@configs/optimizer/adamw.toml",
        "--train.outer_optimizer", "@configs/optimizer/none.toml"]


def test_reference_launch_line_parses(monkeypatch):
    monkeypatch.chdir(ROOT)
    c = config_from_argv(["--swarm.num_stages", "2", "--device", "cpu"] + BASE + [
        "--data.tokenize", "true", "--data.seq_length", "128", "--train.inner_optimizer.lr", "0.006",
        "--train.max_steps", "40", "--amp.enable", "false", "--logging.wandb.tags", "a,b"])
    assert c.swarm.num_stages == 2 and c.device == "cpu"
    assert (c.model.n_layer, c.model.n_head, c.model.n_embd) == (4, 4, 128)
    assert c.train.inner_optimizer.type == "AdamW" and c.train.inner_optimizer.lr == 0.006
    assert c.train.outer_optimizer.type == "None"
    assert c.data.tokenize is True and c.amp.enable is False
    assert c.logging.wandb.tags == ["a", "b"]


def test_defaults_match_reference(monkeypatch):
    monkeypatch.chdir(ROOT)
    c = config_from_argv(BASE)
    assert c.swarm.num_stages == 2 and c.swarm.sync_every_n_steps == 1
    assert c.train.micro_batch_size == 16 and c.train.batch_size == 512 and c.train.max_micro_batches == 1
    assert c.train.seed == 42 and c.train.max_norm == 1.0 and c.train.step_timeout == 60
    assert c.train.inner_optimizer.weight_decay == 0.1 and c.train.inner_optimizer.betas == [0.9, 0.95]
    assert c.data.seq_length == 1024 and c.amp.dtype == "bfloat16" and c.amp.precision == "high"
    assert c.sample.num_samples == 5 and c.sample.prompt == "I am" and c.sample.top_k == 20
    assert c.eval.eval_size == 0.1 and c.logging.log_dir == "logs"
    assert c.model.vocab_size == 50304 and c.model.parameter_sharing is False


def test_dotted_override_after_toml_and_unknown_key(monkeypatch):
    monkeypatch.chdir(ROOT)
    t = parse_argv(["--model", "@configs/model/gpt2-small.toml", "--model.n_layer", "3", "--flag", "--no-other"])
    assert t["model"] == {"n_layer": 3, "n_head": 12, "n_embd": 768} and t["flag"] is True and t["other"] is False
    with pytest.raises(Exception):
        config_from_argv(BASE + ["--train.nonexistent", "1"])


def test_presets_exist():
    for m, dims in {"tiny": (4, 4, 128), "small": (12, 12, 768), "medium": (24, 16, 1024), "large": (36, 20, 1280),
                    "xl": (48, 25, 1600)}.items():
        t = parse_argv(["--model", f"@{ROOT}/configs/model/gpt2-{m}.toml"])["model"]
        assert (t["n_layer"], t["n_head"], t["n_embd"]) == dims


def test_added_list_and_flag_fields_parse_from_the_command_line(monkeypatch):
    monkeypatch.chdir(ROOT)
    cfg = config_from_argv(BASE + ["--swarm.routing", "weighted", "--swarm.routing_weights", "1,1,2.5,0",
                                   "--train.deterministic", "true", "--elastic.enable", "true", "--elastic.die_rank", "3"])
    assert cfg.swarm.routing == "weighted" and cfg.swarm.routing_weights == [1.0, 1.0, 2.5, 0.0]
    assert cfg.train.deterministic is True and cfg.elastic.die_rank == 3 and cfg.elastic.die_at_step == -1
