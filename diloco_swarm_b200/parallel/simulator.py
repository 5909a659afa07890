"""Single-process virtual swarm.

Runs an S x R world inside one process: one autograd stage engine per virtual
rank, the same seeded routing table as the real run (parallel/schedule.py),
tensors handed from engine to engine instead of sent.  Because routing is a
pure function of (seed, step), the simulator reproduces the loss curve of the
multi-process run on the same data (up to floating-point summation order),
which is what the topology tests compare against.  The reference has nothing
like it: its routing is unseeded (src/comm.py:91), so two runs of the same
world never agree.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from ..config import Config
from ..models.engine_torch import TorchEngine
from ..models.gpt2 import GPT2Config
from ..optim import lr_factor
from ..utils import data as D
from ..utils.metrics import Outputs, aggregate_outputs
from ..world import World
from . import schedule


def _virtual_world(rank: int, world_size: int, num_stages: int) -> World:
    saved = {k: os.environ.get(k) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "LOCAL_WORLD_SIZE")}
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world_size), LOCAL_RANK=str(rank),
                      LOCAL_WORLD_SIZE=str(world_size))
    try:
        return World(num_stages, init=False)
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


class VirtualSwarm:
    def __init__(self, config: Config, world_size: int, device: Optional[torch.device] = None):
        self.config, self.world_size = config, world_size
        self.device = device or torch.device("cpu")
        S = config.swarm.num_stages
        mc = config.model
        g = GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                       n_embd=mc.n_embd, dropout=mc.dropout, bias=mc.bias, parameter_sharing=mc.parameter_sharing)
        self.worlds = [_virtual_world(r, world_size, S) for r in range(world_size)]
        self.engines = [TorchEngine(g, w, config, self.device) for w in self.worlds]
        tc = config.train
        self.mbs, self.seq = tc.micro_batch_size, config.data.seq_length
        self.num_micro = max(1, tc.batch_size // tc.micro_batch_size)
        last = self.worlds[0].last_stage_ranks
        self.micro_per_device = max(1, self.num_micro // len(last))
        self.loss_scale = 1.0 / self.micro_per_device
        self.seed = config.swarm.routing_seed if config.swarm.routing_seed is not None else tc.seed
        self.opt_steps = 0
        self.num_train_steps = 0
        self.master = self.worlds[0].last_stage_leader
        self.alive: List[bool] = [True] * world_size

    # ------------------------------------------------------------------
    def _stage_groups(self) -> List[List[int]]:
        w = self.worlds[0]
        return [[r for r in w.stage2ranks[s] if self.alive[r]] for s in range(w.num_stages)]

    def set_alive(self, alive: Sequence[bool]) -> None:
        """Ranks that take part from now on (the trainer's membership mask): routing draws from them,
        the stage groups shrink to them, the microbatch share per last-stage replica follows."""
        self.alive = list(alive)
        last = self._stage_groups()[-1]
        self.micro_per_device = max(1, self.num_micro // len(last))
        self.loss_scale = 1.0 / self.micro_per_device
        self.master = last[0]

    def _sync_gradients(self) -> None:
        for ranks in self._stage_groups():
            if len(ranks) == 1:
                continue
            plists = [list(self.engines[r].model.parameters()) for r in ranks]
            for ps in zip(*plists):
                mean = torch.stack([p.grad for p in ps]).sum(0) / len(ranks)
                for p in ps:
                    p.grad.copy_(mean)

    def _outer_step(self) -> None:
        for ranks in self._stage_groups():
            engs = [self.engines[r] for r in ranks]
            with torch.no_grad():
                deltas = []
                for e in engs:
                    deltas.append([po.data - pi.data for po, pi in zip(e.outer_params, e.model.parameters())])
                for i in range(len(deltas[0])):
                    mean = torch.stack([d[i] for d in deltas]).sum(0) / len(ranks)
                    for e in engs:
                        e.outer_params[i].grad = mean.clone()
            for e in engs:
                e.outer_opt.step()
                with torch.no_grad():
                    for po, pi in zip(e.outer_params, e.model.parameters()):
                        pi.data.copy_(po.data)

    # ------------------------------------------------------------------
    def train_step(self, step: int, batch: Dict[str, torch.Tensor], dropped: bool = False) -> Dict[str, object]:
        """One step of every live rank.  ``dropped``: the step is abandoned as the trainer abandons a step
        that not every rank got through (no gradient is applied, the optimiser does not advance)."""
        cfg, S, W = self.config, self.config.swarm.num_stages, self.world_size
        if dropped:
            return {"local": None, "global": None, "do_sync": False}
        path = schedule.route(self.seed, step, S, W, self.num_micro, self.alive, mode=cfg.swarm.routing,
                              weights=cfg.swarm.routing_weights)
        for e in self.engines:
            e.train()
            e.zero_grad()
        loss = [0.0] * W
        count = [0] * W
        for mb in range(self.num_micro):
            rows = D.micro_batch_rows(mb, self.mbs)
            ids, tg, mask = (batch[k][rows].to(self.device) for k in ("input_ids", "target_ids", "attention_mask"))
            hidden = None
            for s in range(S):
                r = int(path[mb, s])
                count[r] += 1
                e = self.engines[r]
                if s < S - 1:
                    hidden = e.forward(mb, ids if s == 0 else None, hidden)
                else:
                    l, dx = e.forward_backward(mb, ids if s == 0 else None, hidden, tg, mask, self.loss_scale)
                    loss[r] += float(l)
            for s in range(S - 2, -1, -1):
                dx = self.engines[int(path[mb, s])].backward(mb, dx)
        H = cfg.swarm.sync_every_n_steps
        do_sync = (H > 0 and step % H == 0) or step == self.num_train_steps
        has_outer = self.engines[0].has_outer
        if do_sync and not has_outer:
            self._sync_gradients()
        lr = cfg.train.inner_optimizer.lr * lr_factor(self.opt_steps, cfg.train.scheduler, self.num_train_steps)
        norms = [e.optimizer_step(lr, cfg.train.max_norm) if self.alive[r] else 0.0 for r, e in enumerate(self.engines)]
        self.opt_steps += 1
        if do_sync and has_outer:
            self._outer_step()
        outs = [Outputs(step=step, time=1.0, loss=loss[r], tokens=count[r] * self.mbs * self.seq,
                        num_micro_batches=count[r], lr=lr, norm=norms[r], micro_step_time=1.0) for r in range(W)]
        last = self._stage_groups()[-1]
        glob = aggregate_outputs(outs[self.master], [outs[r] for r in last])
        return {"local": outs, "global": glob, "do_sync": do_sync}

    def run(self, loader: D.BatchLoader, num_steps: int) -> List[float]:
        """Global loss (the master's view) of every step."""
        self.num_train_steps = num_steps
        it = iter(loader)
        return [self.train_step(step, next(it))["global"].loss for step in range(1, num_steps + 1)]
