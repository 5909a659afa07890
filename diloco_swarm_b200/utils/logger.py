"""Console / file / optional wandb logging per rank.

Directory layout as in the reference (src/logger.py:31-47,90-93):
``<log_dir>/<run_id>/{<local_rank>.log, master.log, checkpoints/, samples/<step>.txt}``.
Only the master writes the samples file (in the reference every rank writes
the same file concurrently).
"""
from __future__ import annotations

import logging
import os
from datetime import datetime
from enum import Enum
from typing import Any, Dict, List, Optional

import yaml


class Level(Enum):
    DEBUG = logging.DEBUG
    INFO = logging.INFO
    WARNING = logging.WARNING
    ERROR = logging.ERROR


class Logger:
    def __init__(self, world, config):
        self.world, self.config = world, config
        self.name = f"rank{world.local_rank}"
        self.run_id = config.run_id or datetime.now().strftime("%Y%m%d_%H%M%S")
        self.is_master = world.is_master
        self.wandb_run = None
        self.log_dir = os.path.join(config.log_dir, self.run_id)
        self.checkpoint_dir = os.path.join(self.log_dir, "checkpoints")
        self.samples_dir = os.path.join(self.log_dir, "samples")
        for d in (self.log_dir, self.checkpoint_dir, self.samples_dir):
            os.makedirs(d, exist_ok=True)
        uid = f"{self.run_id}-{world.rank}"
        self.file_logger = self._file_logger(f"file-{uid}", str(world.local_rank), config.file.log_level)
        self.console_logger = self._console_logger(f"console-{uid}", str(world.local_rank), config.console.log_level)
        self.master_file_logger = self.master_console_logger = None
        if self.is_master:
            self.master_file_logger = self._file_logger(f"master-file-{uid}", "master", config.file.log_level)
            self.master_console_logger = self._console_logger(f"master-console-{uid}", "*", config.console.log_level)
        if config.wandb.enable:
            try:
                import wandb
                self.wandb_run = wandb.init(name=self.name, project=config.wandb.project,
                                            entity=config.wandb.entity, tags=config.wandb.tags,
                                            group=config.wandb.group or self.run_id, dir=self.log_dir)
            except Exception as e:  # offline boxes: keep training
                self.log_message(f"wandb disabled: {e}", master=False, level=Level.WARNING)

    def log_message(self, message: Any, master: bool, level: Level = Level.INFO) -> None:
        message = str(message)
        self.file_logger.log(level.value, message)
        if master:
            if self.master_console_logger:
                self.master_console_logger.log(level.value, message)
            if self.master_file_logger:
                self.master_file_logger.log(level.value, message)
        else:
            self.console_logger.log(level.value, message)

    def log_config(self, config) -> None:
        d = config.model_dump()
        text = "Setting configuration:\n\t" + yaml.dump(d, sort_keys=False).replace("\n", "\n\t").strip()
        self.log_message(text, master=True, level=Level.INFO)
        if self.wandb_run:
            self.wandb_run.config.update(d)

    def log_world(self, world) -> None:
        self.log_message(world, master=False, level=Level.INFO)
        if self.wandb_run:
            self.wandb_run.config.update({"world": dict(world)})

    def log_metrics(self, metrics: Dict[str, float], step: Optional[int] = None, master: bool = True) -> None:
        self.log_message(f"{'Global' if master else 'Local'} metrics: {metrics}", master=master, level=Level.DEBUG)
        if self.wandb_run and (not master or self.is_master):
            self.wandb_run.log(metrics, step=step)

    def log_samples(self, samples: List[str], step: int) -> None:
        for i, s in enumerate(samples):
            self.log_message(f"Sample {i + 1}: {s}", master=True, level=Level.INFO)
        if self.is_master:
            with open(os.path.join(self.samples_dir, f"{step}.txt"), "w") as f:
                for s in samples:
                    f.write(s + "\n")

    def close(self) -> None:
        for lg in (self.file_logger, self.console_logger, self.master_file_logger, self.master_console_logger):
            if lg is None:
                continue
            for h in list(lg.handlers):
                h.flush()
                h.close()
                lg.removeHandler(h)
        if self.wandb_run:
            self.wandb_run.finish()

    def _file_logger(self, name: str, short: str, level: str) -> logging.Logger:
        lg = logging.getLogger(name)
        lg.setLevel(level)
        lg.propagate = False
        h = logging.FileHandler(os.path.join(self.log_dir, f"{short}.log"))
        h.setFormatter(logging.Formatter(f"[%(asctime)s][%(levelname)s][{short}] %(message)s"))
        lg.addHandler(h)
        return lg

    def _console_logger(self, name: str, short: str, level: str) -> logging.Logger:
        lg = logging.getLogger(name)
        lg.setLevel(level)
        lg.propagate = False
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(f"[%(levelname)s][{short}] %(message)s"))
        lg.addHandler(h)
        return lg
