"""Per-rank logging to files, console and (optionally) wandb.

What a user of the reference finds unchanged (src/logger.py:31-47,60-93): the run directory
``<log_dir>/<run_id>/`` with one ``<local_rank>.log`` per rank, ``master.log`` written by the master
rank, ``checkpoints/`` and ``samples/<step>.txt``; the ``Level`` enum; the five ``log_*`` calls and the
text they produce.  What differs: messages go through a small table of channels instead of four
hand-wired loggers, logger names carry the run id and the global rank (two runs in one process, as in
the tests, do not share handlers), only the master writes the samples file (in the reference every
rank writes the same file at once), wandb failures on an offline box do not stop the run, and
``close()`` releases the files.  Added for boxes without wandb: every ``log_metrics`` call also appends
one JSON line to ``metrics/<local_rank>.jsonl`` (local metrics) or ``metrics/master.jsonl`` (global and
evaluation metrics, master only), and the master saves the configuration and the world size as
``config.yaml``; ``utils/results.py`` builds the reference's result tables from these files.
"""
from __future__ import annotations

import json
import logging
import os
from datetime import datetime
from enum import Enum
from typing import Any, Dict, List, Optional

import yaml

FILE_FORMAT = "[%(asctime)s][%(levelname)s][{tag}] %(message)s"
CONSOLE_FORMAT = "[%(levelname)s][{tag}] %(message)s"


class Level(Enum):
    DEBUG = logging.DEBUG
    INFO = logging.INFO
    WARNING = logging.WARNING
    ERROR = logging.ERROR


class _Channel:
    """One destination: a python logger that owns exactly one handler."""

    def __init__(self, key: str, handler: logging.Handler, fmt: str, tag: str, threshold: str):
        handler.setFormatter(logging.Formatter(fmt.format(tag=tag)))
        self.log = logging.getLogger(key)
        self.log.propagate = False
        self.log.setLevel(threshold)
        self.log.addHandler(handler)
        self.handler = handler

    def emit(self, level: Level, text: str) -> None:
        self.log.log(level.value, text)

    def close(self) -> None:
        self.handler.flush()
        self.handler.close()
        self.log.removeHandler(self.handler)


class Logger:
    def __init__(self, world, config):
        self.world, self.config = world, config
        self.is_master = world.is_master
        self.name = f"rank{world.local_rank}"
        self.run_id = config.run_id if config.run_id is not None else datetime.now().strftime("%Y%m%d_%H%M%S")
        root = os.path.join(config.log_dir, self.run_id)
        self.log_dir, self.checkpoint_dir, self.samples_dir = root, os.path.join(root, "checkpoints"), os.path.join(root, "samples")
        self.metrics_dir = os.path.join(root, "metrics")
        for path in (self.log_dir, self.checkpoint_dir, self.samples_dir, self.metrics_dir):
            os.makedirs(path, exist_ok=True)
        self._history: Dict[str, Any] = {}          # open metric files by name

        # channel table: "own" = this rank's file (sees every message), "local" = what a non-master
        # message also reaches, "master" = what a master message also reaches (empty on other ranks)
        uid, tag = f"{self.run_id}.{world.rank}", str(world.local_rank)
        own = self._file(f"dsw.file.{uid}", tag)
        self._channels: Dict[str, List[_Channel]] = {
            "own": [own],
            "local": [self._console(f"dsw.console.{uid}", tag)],
            "master": ([self._console(f"dsw.console.master.{uid}", "*"), self._file(f"dsw.file.master.{uid}", "master")]
                       if self.is_master else []),
        }
        self.wandb_run = self._start_wandb() if config.wandb.enable else None

    # ------------------------------------------------------------------ messages
    def log_message(self, message: Any, master: bool, level: Level = Level.INFO) -> None:
        text = str(message)
        for ch in self._channels["own"] + self._channels["master" if master else "local"]:
            ch.emit(level, text)

    def log_config(self, config) -> None:
        as_dict = config.model_dump()
        body = yaml.dump(as_dict, sort_keys=False).strip().replace("\n", "\n\t")
        self.log_message("Setting configuration:\n\t" + body, master=True, level=Level.INFO)
        if self.is_master:
            with open(os.path.join(self.log_dir, "config.yaml"), "w") as f:
                yaml.dump({**as_dict, "world": {"world_size": self.world.world_size,
                                                "num_stages": self.world.num_stages}}, f, sort_keys=False)
        if self.wandb_run:
            self.wandb_run.config.update(as_dict)

    def log_world(self, world) -> None:
        self.log_message(world, master=False, level=Level.INFO)
        if self.wandb_run:
            self.wandb_run.config.update({"world": dict(world)})

    def log_metrics(self, metrics: Dict[str, float], step: Optional[int] = None, master: bool = True) -> None:
        scope = "Global" if master else "Local"
        self.log_message(f"{scope} metrics: {metrics}", master=master, level=Level.DEBUG)
        if metrics and (self.is_master or not master):
            self._append_history("master" if master else str(self.world.local_rank), step, metrics)
        # local metrics go to every rank's wandb run, global ones to the master's only
        if self.wandb_run and (self.is_master or not master):
            self.wandb_run.log(metrics, step=step)

    def log_samples(self, samples: List[str], step: int) -> None:
        for number, text in enumerate(samples, start=1):
            self.log_message(f"Sample {number}: {text}", master=True, level=Level.INFO)
        if self.is_master:
            with open(os.path.join(self.samples_dir, f"{step}.txt"), "w") as f:
                f.writelines(text + "\n" for text in samples)

    def _append_history(self, name: str, step: Optional[int], metrics: Dict[str, float]) -> None:
        f = self._history.get(name)
        if f is None:
            f = self._history[name] = open(os.path.join(self.metrics_dir, f"{name}.jsonl"), "a")
        f.write(json.dumps({"_step": step, **metrics}) + "\n")
        f.flush()

    def close(self) -> None:
        for f in self._history.values():
            f.close()
        self._history = {}
        for group in self._channels.values():
            for ch in group:
                ch.close()
        self._channels = {"own": [], "local": [], "master": []}
        if self.wandb_run:
            self.wandb_run.finish()
            self.wandb_run = None

    # ------------------------------------------------------------------ construction
    def _file(self, key: str, tag: str) -> _Channel:
        handler = logging.FileHandler(os.path.join(self.log_dir, f"{tag}.log"))
        return _Channel(key, handler, FILE_FORMAT, tag, self.config.file.log_level)

    def _console(self, key: str, tag: str) -> _Channel:
        return _Channel(key, logging.StreamHandler(), CONSOLE_FORMAT, tag, self.config.console.log_level)

    def _start_wandb(self):
        cfg = self.config.wandb
        try:
            import wandb
            return wandb.init(name=self.name, project=cfg.project, entity=cfg.entity, tags=cfg.tags,
                              group=cfg.group or self.run_id, dir=self.log_dir)
        except Exception as e:          # no network, not logged in: training goes on without it
            self.log_message(f"wandb disabled: {e}", master=False, level=Level.WARNING)
            return None
