"""Result tables from run directories, without wandb.

The reference analyses its experiments in a notebook that pulls every run's
history from the wandb service (notebooks/3.0-results.ipynb, cells 7-31 and
36-47).  Here the Logger keeps the same history on disk (``metrics/*.jsonl``
with wandb's ``_step`` column, ``config.yaml``), and this module turns run
directories into the notebook's tables:

``load_history``       a run's metric history as a DataFrame (cell 7);
``perplexity_table``   final validation perplexity per run with absolute and
                       relative change against the best (cells 26 and 31);
``with_comm_cost``     a history with the cumulative communication volume of
                       its configuration (cells 16-20, formulas in comm_model);
``throughput_table``   peak tokens/s per run, labelled Single GPU / Data
                       Parallel / Pipeline Parallel / SWARM (cells 36-47).

    python -m diloco_swarm_b200.utils.results logs/run_a logs/run_b [--table throughput] [--latex]

Figures need matplotlib, which is optional: ``plot_curves`` raises a clear
error when it is missing; the tables never need it.
"""
from __future__ import annotations

import argparse
import json
import os
from typing import Dict, Mapping, Optional

import pandas as pd
import yaml

from . import comm_model

PERPLEXITY = "eval/perplexity/average"
THROUGHPUT = "train/global/throughput/current"


def load_history(run_dir: str, which: str = "master") -> pd.DataFrame:
    """Metric history of one run: one row per ``log_metrics`` call, ``_step`` plus the metric keys.
    ``which``: "master" (global and evaluation metrics) or a local rank number."""
    path = os.path.join(run_dir, "metrics", f"{which}.jsonl")
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path}: the run has no metric history (was it written by this framework's Logger?)")
    with open(path) as f:
        rows = [json.loads(line) for line in f if line.strip()]
    return pd.DataFrame(rows)


def load_config(run_dir: str) -> dict:
    with open(os.path.join(run_dir, "config.yaml")) as f:
        return yaml.safe_load(f)


def _series(history: pd.DataFrame, key: str) -> pd.DataFrame:
    if key not in history.columns:
        return pd.DataFrame(columns=["step", key])
    out = history[["_step", key]].dropna().rename(columns={"_step": "step"})
    return out.reset_index(drop=True)


def _change_column(values: pd.Series, base: float) -> pd.Series:
    """The notebook's "abs / rel%" text; "-" for the row that is the base."""
    out = []
    for v in values:
        a = round(abs(v - base), 2)
        out.append("-" if a == 0 else f"{a} / {round(a / base * 100, 2)}%")
    return pd.Series(out, index=values.index)


def perplexity_table(runs: Mapping[str, str], key: str = PERPLEXITY) -> pd.DataFrame:
    """``runs``: label -> run directory.  Final value of ``key`` per run, best first, with the
    change against the best run."""
    final = {}
    for label, run_dir in runs.items():
        s = _series(load_history(run_dir), key)
        if len(s):
            final[label] = float(s[key].iloc[-1])
    ppl = pd.Series(final, dtype=float).sort_values().round(2)
    if ppl.empty:
        return pd.DataFrame(columns=["run", "perplexity", "change (abs / rel)"])
    return pd.DataFrame({"run": ppl.index, "perplexity": ppl.values,
                         "change (abs / rel)": _change_column(ppl, ppl.iloc[0]).values})


def method_table(runs: Mapping[str, str], key: str = PERPLEXITY) -> pd.DataFrame:
    """Labels of the form "<model> <method>" (e.g. "GPT-2 Small DiLoCo-SWARM"): one row per model, one
    column per method, and the change between the first two methods (the notebook's model-size table)."""
    rows = []
    for label, run_dir in runs.items():
        s = _series(load_history(run_dir), key)
        if len(s):
            model, method = label.rsplit(" ", 1)
            rows.append({"model": model, "method": method, key: round(float(s[key].iloc[-1]), 2)})
    if not rows:
        return pd.DataFrame()
    tab = pd.DataFrame(rows).pivot(index="model", columns="method", values=key).reset_index().rename_axis(None, axis=1)
    methods = [c for c in tab.columns if c != "model"]
    if len(methods) >= 2:
        a, b = tab[methods[0]], tab[methods[1]]
        change = (b - a).abs().round(2)
        tab["change (abs / rel)"] = [("-" if c == 0 or pd.isna(c) else f"{c} / {round(c / base * 100, 2)}%")
                                     for c, base in zip(change, a)]
    return tab


def with_comm_cost(history: pd.DataFrame, config: dict, num_params: Optional[float] = None,
                   bytes_per_value: int = 2, metadata_plane: bool = False) -> pd.DataFrame:
    """Adds ``comm_bytes``: the cumulative communication volume of the run's configuration at each row's
    step.  Defaults describe this framework's wire format (bf16 payload, no metadata plane); pass
    ``bytes_per_value=4, metadata_plane=True`` for the reference's."""
    world = config.get("world", {})
    S = int(world.get("num_stages", config["swarm"]["num_stages"]))
    R = max(1, int(world.get("world_size", S)) // S)
    m, t, d = config["model"], config["train"], config["data"]
    if num_params is None:
        num_params = 12 * m["n_layer"] * m["n_embd"] ** 2 + 2 * m.get("vocab_size", 50304) * m["n_embd"]
    H = max(1, int(config["swarm"]["sync_every_n_steps"]))
    steps = int(history["_step"].max()) if len(history) else 0
    cost = comm_model.run_cost(steps, S, R, t["batch_size"], d["seq_length"], m["n_embd"], num_params, H,
                               pp_bytes_per_value=bytes_per_value, metadata_plane=metadata_plane)
    curve = comm_model.cumulative(cost, H)
    out = history.copy()
    out["comm_bytes"] = [curve[int(s) - 1] if s and 0 < int(s) <= len(curve) else 0.0 for s in out["_step"]]
    return out


def parallelism(world_size: int, num_stages: int) -> str:
    if world_size == 1:
        return "Single GPU"
    if num_stages == 1:
        return "Data Parallel"
    if num_stages == world_size:
        return "Pipeline Parallel"
    return "SWARM"


def throughput_table(runs: Mapping[str, str], key: str = THROUGHPUT) -> pd.DataFrame:
    """Peak and mean of the throughput metric per run with the run's topology, fastest first."""
    rows = []
    for label, run_dir in runs.items():
        s = _series(load_history(run_dir), key)
        cfg = load_config(run_dir)
        world = cfg.get("world", {})
        S = int(world.get("num_stages", cfg["swarm"]["num_stages"]))
        W = int(world.get("world_size", S))
        rows.append({"run": label, "parallelism": parallelism(W, S), "num_nodes": W, "num_stages": S,
                     "micro_batch_size": cfg["train"]["micro_batch_size"],
                     "max_micro_batches": cfg["train"]["max_micro_batches"],
                     "peak tokens/s": float(s[key].max()) if len(s) else float("nan"),
                     "mean tokens/s": float(s[key].mean()) if len(s) else float("nan")})
    return pd.DataFrame(rows).sort_values("peak tokens/s", ascending=False).reset_index(drop=True)


def plot_curves(runs: Mapping[str, str], path: str, key: str = PERPLEXITY, x: str = "step") -> None:
    """Metric against steps (or against ``comm_bytes``) for several runs, written to ``path``."""
    try:
        import matplotlib
        matplotlib.use("Agg")
        from matplotlib import pyplot as plt
    except ImportError as e:
        raise RuntimeError("plot_curves needs matplotlib, which is not installed; the tables do not") from e
    fig, ax = plt.subplots(figsize=(6, 4), dpi=200)
    for label, run_dir in runs.items():
        h = load_history(run_dir)
        if x == "comm_bytes":
            h = with_comm_cost(h, load_config(run_dir))
        h = h.dropna(subset=[key])
        ax.plot(h["_step"] if x == "step" else h[x] / 1e12, h[key], label=label)
    ax.set_xlabel("Training steps" if x == "step" else "Communication cost (TB)")
    ax.set_ylabel(key)
    ax.grid(True, alpha=0.3)
    ax.legend()
    fig.savefig(path, bbox_inches="tight")


def _labelled(paths) -> Dict[str, str]:
    """``label=dir`` or just ``dir`` (label = directory name)."""
    out = {}
    for p in paths:
        label, _, d = p.rpartition("=")
        out[label or os.path.basename(os.path.normpath(d))] = d
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description="Result tables from run directories (logs/<run_id>)")
    ap.add_argument("runs", nargs="+", help="run directories, optionally as label=dir")
    ap.add_argument("--table", default="perplexity", choices=["perplexity", "method", "throughput", "history"])
    ap.add_argument("--key", default=None, help="metric key (default depends on the table)")
    ap.add_argument("--latex", action="store_true")
    ap.add_argument("--plot", default=None, help="also write the curves of --key to this file (needs matplotlib)")
    a = ap.parse_args()
    runs = _labelled(a.runs)
    if a.table == "perplexity":
        tab = perplexity_table(runs, a.key or PERPLEXITY)
    elif a.table == "method":
        tab = method_table(runs, a.key or PERPLEXITY)
    elif a.table == "throughput":
        tab = throughput_table(runs, a.key or THROUGHPUT)
    else:
        label, run_dir = next(iter(runs.items()))
        tab = with_comm_cost(load_history(run_dir), load_config(run_dir))
    print(tab.to_latex(index=False) if a.latex else tab.to_markdown(index=False))
    if a.plot:
        plot_curves(runs, a.plot, a.key or PERPLEXITY)


if __name__ == "__main__":
    main()
