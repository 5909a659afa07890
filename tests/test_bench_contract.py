"""bench.py without a GPU: defaults, the configuration it trains, and the clock summary."""
import datetime
import os
import sys
from types import SimpleNamespace

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def _args(*argv):
    old = sys.argv
    sys.argv = ["bench.py", *argv]
    try:
        return bench.parse_args()
    finally:
        sys.argv = old


def test_defaults_and_headline_configuration():
    a = _args()
    assert (a.gpus, a.impl, a.engine) == (1, "ours", "b200") and a.warmup >= 3 and a.steps >= 1
    cfg, H = bench.build_config(a, 1)
    m, t = cfg.model, cfg.train
    assert (m.n_layer, m.n_head, m.n_embd, m.vocab_size) == (12, 12, 768, 50304)
    assert (t.batch_size, t.micro_batch_size, cfg.data.seq_length) == (512, 16, 1024)
    assert t.inner_optimizer.type == "AdamW" and t.inner_optimizer.lr == 6e-4
    assert (t.outer_optimizer.type, t.outer_optimizer.lr, t.outer_optimizer.momentum, t.outer_optimizer.nesterov) == \
        ("SGD", 0.7, 0.9, True)
    assert H == min(50, a.steps) and cfg.swarm.sync_every_n_steps == H and cfg.engine == "b200"
    assert cfg.data.path == "synthetic:zipf" and cfg.amp.enable and cfg.amp.dtype == "bfloat16"
    assert bench.TOPOLOGY == {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (2, 4)}
    plain, _ = bench.build_config(_args("--no-outer"), 2)
    assert plain.train.outer_optimizer.type == "None" and plain.swarm.sync_every_n_steps == 1 and plain.swarm.num_stages == 2


def test_clock_summary_counts_only_the_timed_windows(tmp_path):
    rows = [  # timestamp, index, sm, max sm, power, active mask, hw_slowdown, hw_thermal, sw_thermal, sw_power_cap
        "2026/11/25 10:00:00.000, 0, 345, 1965, 140.0, 0x0000000000000001, Not Active, Not Active, Not Active, Not Active",
        "2026/11/25 10:00:01.000, 0, 1850, 1965, 960.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "2026/11/25 10:00:01.200, 0, 1870, 1965, 970.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "2026/11/25 10:00:01.400, 0, 1860, 1965, 250.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
        "2026/11/25 10:00:05.000, 0, 1200, 1965, 900.0, 0x0000000000000040, Active, Active, Not Active, Not Active",
        "garbage line",
    ]
    path = tmp_path / "smi.csv"
    path.write_text("\n".join(rows) + "\n")
    s = bench.ClockSampler(False)
    s.proc = SimpleNamespace(terminate=lambda: None, wait=lambda timeout=None: 0, kill=lambda: None)
    s.path = str(path)
    t = lambda sec: datetime.datetime(2026, 11, 25, 10, 0, 0) + datetime.timedelta(seconds=sec)
    out = s.stop([(t(0.5), t(2.0))])
    assert out == {"sm_mhz": 1860.0, "sm_max_mhz": 1965.0, "power_w_max": 970.0, "samples_under_load": 2,
                   "reasons": ["sw_power_cap"]}
    assert not os.path.exists(path)
    # without a sampler the summary says so instead of inventing numbers
    assert bench.ClockSampler(False).stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}


def test_reference_arm_says_unavailable_without_the_install(monkeypatch, tmp_path):
    from baseline import run_reference as R
    monkeypatch.setattr(R, "REF", str(tmp_path / "missing"))
    monkeypatch.delenv("RANK", raising=False)
    out = R.run_reference(_args("--impl", "reference"))
    assert out["impl"] == "reference" and "unavailable" in out and "\n" not in out["unavailable"]
    # wrong number of ranks for --gpus is also reported, not raised
    monkeypatch.setattr(R, "REF", os.path.join(ROOT, "baseline", "_ref"))
    if os.path.isdir(os.path.join(R.REF, "src")):
        monkeypatch.setenv("WORLD_SIZE", "1")
        out = R.run_reference(_args("--impl", "reference", "--gpus", "2"))
        assert "unavailable" in out


def test_reference_arm_dataset_stand_in():
    import torch
    from baseline.run_reference import _Tokenizer, _ZipfDataset
    ds = _ZipfDataset(torch.arange(40).reshape(10, 4))
    parts = ds.train_test_split(0.2)
    assert len(parts["train"]) == 8 and len(parts["test"]) == 2 and len(ds.select([0, 3])) == 2
    assert ds[1] == {"input_ids": [4, 5, 6, 7], "attention_mask": [1, 1, 1, 1]}
    assert len(_Tokenizer()) == 50257 and _Tokenizer().decode([1, 2]) == "1 2"
