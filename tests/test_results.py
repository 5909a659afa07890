"""Offline metric history written by the Logger and the result tables built from it
(the counterpart of the reference's wandb-based notebooks/3.0-results.ipynb)."""
import math
import os
from types import SimpleNamespace

import pytest

from diloco_swarm_b200.config import Config
from diloco_swarm_b200.utils import comm_model, results
from diloco_swarm_b200.utils.logger import Logger


def _world(world_size, num_stages, rank=0):
    # the master is the leader of the last stage: rank num_stages - 1
    is_master = rank == num_stages - 1
    return SimpleNamespace(rank=rank, local_rank=rank, world_size=world_size, num_stages=num_stages, is_master=is_master)


def _fake_run(tmp_path, run_id, world_size, num_stages, H, ppl, tput):
    cfg = Config(model={"n_layer": 12, "n_head": 12, "n_embd": 768},
                 data={"path": "synthetic:zipf", "seq_length": 1024},
                 train={"batch_size": 2048, "micro_batch_size": 32, "max_micro_batches": 12,
                        "inner_optimizer": {"type": "AdamW", "lr": 4e-4}, "outer_optimizer": {"type": "None", "lr": 0.0}},
                 swarm={"num_stages": num_stages, "sync_every_n_steps": H},
                 logging={"log_dir": str(tmp_path), "run_id": run_id, "console": {"log_level": "ERROR"}})
    log = Logger(_world(world_size, num_stages, rank=num_stages - 1), cfg.logging)
    log.log_config(cfg)
    for step, (p, t) in enumerate(zip(ppl, tput), start=1):
        log.log_metrics({"train/local/loss/current": 1.0}, step=step, master=False)
        log.log_metrics({"train/global/throughput/current": t, "train/global/loss/current": math.log(p)}, step=step)
        if step % 2 == 0:
            log.log_metrics({"eval/perplexity/average": p, "eval/loss/average": math.log(p)}, step=step)
    log.close()
    return os.path.join(str(tmp_path), run_id)


def test_history_files_and_tables(tmp_path):
    a = _fake_run(tmp_path, "single", 1, 1, 1, [90, 60, 40, 30.0], [10e3, 11e3, 12e3, 11e3])
    b = _fake_run(tmp_path, "swarm", 8, 2, 1, [80, 50, 35, 25.0], [60e3, 70e3, 65e3, 66e3])
    c = _fake_run(tmp_path, "diloco", 8, 2, 2, [85, 55, 38, 26.5], [70e3, 80e3, 82e3, 81e3])
    assert sorted(os.listdir(os.path.join(b, "metrics"))) == ["1.jsonl", "master.jsonl"]     # master = rank 1 of 2 stages
    h = results.load_history(b)
    assert list(h["_step"]) == [1, 2, 2, 3, 4, 4] and h["eval/perplexity/average"].dropna().tolist() == [50, 25.0]
    assert len(results.load_history(b, "1")) == 4
    cfg = results.load_config(c)
    assert cfg["world"] == {"world_size": 8, "num_stages": 2} and cfg["swarm"]["sync_every_n_steps"] == 2

    runs = {"Single-GPU": a, "SWARM": b, "DiLoCo-SWARM": c}
    tab = results.perplexity_table(runs)
    assert tab["run"].tolist() == ["SWARM", "DiLoCo-SWARM", "Single-GPU"]
    assert tab["perplexity"].tolist() == [25.0, 26.5, 30.0]
    assert tab["change (abs / rel)"].tolist() == ["-", "1.5 / 6.0%", "5.0 / 20.0%"]

    tp = results.throughput_table(runs)
    assert tp["run"].tolist() == ["DiLoCo-SWARM", "SWARM", "Single-GPU"]
    assert tp["parallelism"].tolist() == ["SWARM", "SWARM", "Single GPU"]
    assert tp["peak tokens/s"].tolist() == [82e3, 70e3, 12e3] and tp["num_nodes"].tolist() == [8, 8, 1]
    assert results.parallelism(2, 1) == "Data Parallel" and results.parallelism(3, 3) == "Pipeline Parallel"

    m = results.method_table({"GPT-2 Small Single-GPU": a, "GPT-2 Small DiLoCo-SWARM": c})
    assert m["model"].tolist() == ["GPT-2 Small"] and m["DiLoCo-SWARM"].tolist() == [26.5] and m["Single-GPU"].tolist() == [30.0]


def test_comm_cost_column_matches_the_closed_forms(tmp_path):
    c = _fake_run(tmp_path, "diloco", 8, 2, 2, [85, 55, 38, 26.5], [1, 1, 1, 1.0])
    cfg = results.load_config(c)
    h = results.with_comm_cost(results.load_history(c), cfg, num_params=180e6, bytes_per_value=4)
    pp = comm_model.pp_bytes_per_step(2, 2048, 1024, 768, 4)
    dp = comm_model.dp_bytes_per_sync(2, 4, 180e6)
    by_step = dict(zip(h["_step"], h["comm_bytes"]))
    assert by_step[1] == pytest.approx(pp) and by_step[2] == pytest.approx(2 * pp + dp)
    assert by_step[4] == pytest.approx(4 * pp + 2 * dp)
    # a single process moves nothing
    a = _fake_run(tmp_path, "single", 1, 1, 1, [9, 8.0], [1, 1.0])
    assert results.with_comm_cost(results.load_history(a), results.load_config(a))["comm_bytes"].max() == 0.0


def test_cli_prints_a_table(tmp_path, capsys, monkeypatch):
    a = _fake_run(tmp_path, "one", 1, 1, 1, [9, 8.0], [5e3, 6e3])
    monkeypatch.setattr("sys.argv", ["results", f"baseline={a}", "--table", "throughput"])
    results.main()
    out = capsys.readouterr().out
    assert "baseline" in out and "Single GPU" in out and "6000" in out


def test_figures_without_matplotlib(tmp_path):
    """The notebook's two figures as SVG: perplexity against steps and against communication volume."""
    import xml.dom.minidom
    b = _fake_run(tmp_path, "swarm", 8, 2, 1, [80, 50, 35, 25.0], [1, 1, 1, 1.0])
    c = _fake_run(tmp_path, "diloco", 8, 2, 2, [85, 55, 38, 26.5], [1, 1, 1, 1.0])
    runs = {"SWARM": b, "DiLoCo-SWARM": c}
    for x in ("step", "comm_bytes"):
        out = tmp_path / f"fig_{x}.svg"
        results.plot_curves(runs, str(out), x=x)
        text = open(out if out.exists() else str(out) + ".svg").read()
        xml.dom.minidom.parseString(text)                       # well-formed
        assert text.count("<path ") == 2 and "SWARM (25)" in text and "DiLoCo-SWARM (26.5)" in text
        assert ("Training steps" if x == "step" else "Communication cost (TB)") in text
    assert results._nice_ticks(0, 10) == [0, 2, 4, 6, 8, 10] and results._nice_ticks(21, 100)[0] >= 21
