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

``plot_curves`` draws the notebook's two figures (perplexity against steps and
against communication volume): with matplotlib when it is installed, as a plain
SVG file otherwise.
"""
from __future__ import annotations

import argparse
import json
import math
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


def _series_for_plot(runs: Mapping[str, str], key: str, x: str) -> Dict[str, tuple]:
    out = {}
    for label, run_dir in runs.items():
        h = load_history(run_dir)
        if x == "comm_bytes":
            h = with_comm_cost(h, load_config(run_dir))
        if key not in h.columns:
            continue
        h = h.dropna(subset=[key])
        xs = h["_step"].tolist() if x == "step" else (h[x] / 1e12).tolist()
        out[label] = (xs, h[key].tolist())
    return out


_COLOURS = ["#1b9e77", "#d95f02", "#7570b3", "#e7298a", "#66a61e", "#e6ab02", "#a6761d", "#666666"]


def _nice_ticks(lo: float, hi: float, n: int = 5) -> list:
    if hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 5, 10)), key=lambda s_: abs(s_ - raw))
    first = math.ceil(lo / step) * step
    return [round(first + i * step, 10) for i in range(int((hi - first) / step) + 1)]


def write_svg(series: Dict[str, tuple], path: str, xlabel: str, ylabel: str, width: int = 640, height: int = 420) -> None:
    """A line chart as a plain SVG file: what ``plot_curves`` falls back to without matplotlib.
    ``series``: label -> (xs, ys)."""
    pts = [(x, y) for xs, ys in series.values() for x, y in zip(xs, ys)]
    if not pts:
        raise ValueError("nothing to plot")
    x0, x1 = min(p[0] for p in pts), max(p[0] for p in pts)
    y0, y1 = min(p[1] for p in pts), max(p[1] for p in pts)
    x1, y1 = (x1 if x1 > x0 else x0 + 1), (y1 if y1 > y0 else y0 + 1)
    L, R, T, B = 70, 20, 20, 50
    sx = lambda v: L + (v - x0) / (x1 - x0) * (width - L - R)
    sy = lambda v: height - B - (v - y0) / (y1 - y0) * (height - T - B)
    fmt = lambda v: f"{v:g}"
    o = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="12">',
         f'<rect width="{width}" height="{height}" fill="white"/>']
    for t in _nice_ticks(x0, x1):
        o.append(f'<line x1="{sx(t):.1f}" y1="{T}" x2="{sx(t):.1f}" y2="{height - B}" stroke="#dddddd"/>')
        o.append(f'<text x="{sx(t):.1f}" y="{height - B + 16}" text-anchor="middle">{fmt(t)}</text>')
    for t in _nice_ticks(y0, y1):
        o.append(f'<line x1="{L}" y1="{sy(t):.1f}" x2="{width - R}" y2="{sy(t):.1f}" stroke="#dddddd"/>')
        o.append(f'<text x="{L - 6}" y="{sy(t) + 4:.1f}" text-anchor="end">{fmt(t)}</text>')
    o.append(f'<rect x="{L}" y="{T}" width="{width - L - R}" height="{height - T - B}" fill="none" stroke="black"/>')
    o.append(f'<text x="{(L + width - R) / 2:.1f}" y="{height - 10}" text-anchor="middle">{xlabel}</text>')
    o.append(f'<text x="16" y="{(T + height - B) / 2:.1f}" text-anchor="middle" transform="rotate(-90 16 {(T + height - B) / 2:.1f})">{ylabel}</text>')
    for i, (label, (xs, ys)) in enumerate(series.items()):
        colour = _COLOURS[i % len(_COLOURS)]
        path_d = " ".join(f"{'M' if j == 0 else 'L'}{sx(x):.1f},{sy(y):.1f}" for j, (x, y) in enumerate(zip(xs, ys)))
        o.append(f'<path d="{path_d}" fill="none" stroke="{colour}" stroke-width="2"/>')
        o.append(f'<rect x="{width - R - 170}" y="{T + 8 + 18 * i}" width="12" height="3" fill="{colour}"/>')
        o.append(f'<text x="{width - R - 152}" y="{T + 14 + 18 * i}">{label} ({fmt(round(ys[-1], 2))})</text>')
    o.append("</svg>")
    with open(path, "w") as f:
        f.write("\n".join(o) + "\n")


def plot_curves(runs: Mapping[str, str], path: str, key: str = PERPLEXITY, x: str = "step") -> None:
    """Metric against steps (or against ``comm_bytes``, the cumulative communication volume in TB) for
    several runs, the reference notebook's two figures (cells 14 and 20).  With matplotlib the file type
    follows ``path``; without it the chart is written as SVG by ``write_svg``."""
    series = _series_for_plot(runs, key, x)
    xlabel = "Training steps" if x == "step" else "Communication cost (TB)"
    try:
        import matplotlib
        matplotlib.use("Agg")
        from matplotlib import pyplot as plt
    except ImportError:
        write_svg(series, path if path.endswith(".svg") else path + ".svg", xlabel, key)
        return
    fig, ax = plt.subplots(figsize=(6, 4), dpi=200)
    for label, (xs, ys) in series.items():
        ax.plot(xs, ys, label=f"{label} ({ys[-1]:.2f})")
    ax.set_xlabel(xlabel)
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
    ap.add_argument("--plot", default=None, help="also write the curves of --key to this file (SVG without matplotlib)")
    ap.add_argument("--plot-x", default="step", choices=["step", "comm_bytes"])
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
        plot_curves(runs, a.plot, a.key or PERPLEXITY, a.plot_x)


if __name__ == "__main__":
    main()
