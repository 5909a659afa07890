"""DiLoCo-SWARM training entry point.

    torchrun --nproc_per_node 8 -m diloco_swarm_b200.train --swarm.num_stages 2 \
        --model @configs/model/gpt2-small.toml --data @configs/data/synthetic-zipf.toml \
        --train.inner_optimizer @configs/optimizer/adamw.toml \
        --train.outer_optimizer @configs/optimizer/none.toml

Same flags and run phases as the reference's ``src/train.py`` (sample and
evaluate before training, train, evaluate/sample every n steps, final test and
sample; src/train.py:283-349).  What differs is how a step runs: a precomputed
plan instead of a polling event loop, device-side transfers instead of host
staging, fused kernels for the optimiser and the two stage-wide
synchronisations.
"""
from __future__ import annotations

import contextlib
import os
import sys
import time
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from tqdm import tqdm

from .config import Config, config_from_argv
from .models.gpt2 import GPT2Config, sample_next
from .optim import lr_factor
from .parallel import schedule
from .parallel.comm import InferenceComm, PipelineComm, StepTimeout, sync_outputs
from .parallel.schedule import BWD, FWD, FWD_BWD
from .utils import data as D
from .utils.ckpt import Checkpoint
from .utils.logger import Level, Logger
from .utils.metrics import Outputs, eval_metrics, train_metrics
from .utils.timers import PhaseTimer
from .utils.misc import (format_float, format_int, get_device, get_eval_pbar_description,
                         get_train_pbar_description, seed_everything)
from .world import World


def _gpt2_config(mc) -> GPT2Config:
    return GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                      n_embd=mc.n_embd, dropout=mc.dropout, bias=mc.bias, parameter_sharing=mc.parameter_sharing)


def get_model(model_config, seed: int = 42):
    """The whole GPT-2 as one autograd module (reference: get_model, src/utils.py:48-49)."""
    from .models.gpt2 import TorchStage
    return TorchStage(_gpt2_config(model_config), 0, 1, seed=seed)


def get_sharded_model(model_config, world: World, seed: int = 42, layer_split: str = "even"):
    """This rank's pipeline stage as an autograd module (reference: get_sharded_model,
    src/utils.py:51-52).  Only the stage's own tensors are built; the per-tensor seeded init makes them
    equal to the corresponding tensors of ``get_model`` with the same seed."""
    from .models.gpt2 import TorchStage
    return TorchStage(_gpt2_config(model_config), world.stage, world.num_stages, seed=seed, layer_split=layer_split)


def get_logger(world: World, logging_config) -> Logger:
    return Logger(world, logging_config)


def make_engine(config: Config, world: World, device: torch.device):
    gcfg = _gpt2_config(config.model)
    kind = config.engine
    if kind == "auto":
        kind = "b200" if device.type == "cuda" else "torch"
    if kind == "b200":
        from .models.engine_b200 import B200Engine
        return B200Engine(gcfg, world, config, device)
    from .models.engine_torch import TorchEngine
    return TorchEngine(gcfg, world, config, device)


class Trainer:
    """Owns the world, the stage engine, the pipeline transport and the step logic."""

    def __init__(self, config: Config, world: Optional[World] = None, logger: Optional[Logger] = None):
        self.config = config
        dev_type = (config.device or ("cuda" if torch.cuda.is_available() else "cpu")).split(":")[0]
        if dev_type == "cuda":
            os.environ.setdefault("CUDA_DEVICE_MAX_CONNECTIONS", "32")
        self.world = world or World(config.swarm.num_stages, device_type=dev_type,
                                    timeout_s=max(60.0, 10 * config.train.step_timeout))
        w = self.world
        self.device = get_device(config.device, w.local_rank)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.logger = logger or Logger(w, config.logging)
        seed_everything(config.train.seed)
        torch.set_float32_matmul_precision(config.amp.precision)
        tc = config.train
        self.seq = config.data.seq_length
        self.mbs = tc.micro_batch_size
        self.num_micro = max(1, tc.batch_size // tc.micro_batch_size)
        # reference: num_micro_steps // |last stage|, at least 1 (src/train.py:168)
        self.micro_per_device = max(1, self.num_micro // len(w.last_stage_ranks))
        self.loss_scale = 1.0 / self.micro_per_device
        self.routing_seed = config.swarm.routing_seed if config.swarm.routing_seed is not None else tc.seed
        self._resolve_layer_split()
        self.engine = make_engine(config, w, self.device)
        self.comm = self._make_comm()
        if self.device.type == "cuda" and tc.reserve_memory_gb > 0:
            # one large block, freed at once: it stays with the caching allocator, which cuts later tensors from it
            pool = torch.empty(int(tc.reserve_memory_gb * 2 ** 30), dtype=torch.uint8, device=self.device)
            del pool
        if hasattr(self.engine, "warmup"):
            self.engine.warmup(self.mbs, self.seq)
        self.comm.warmup()
        self.alive: Optional[List[bool]] = None
        self._step_failed = False    # the last step was dropped by the common verdict
        self.membership = None
        if config.elastic.enable and w.world_size > 1:
            if self.engine.name != "torch":
                raise NotImplementedError("elastic membership is implemented for the autograd engine (CPU/gloo): "
                                          "the fused collectives would have to re-map their peer buffers")
            from .parallel.liveness import Membership
            self.membership = Membership(w.rank, w.world_size, w.master_addr, w.master_port + 1, config.elastic.timeout)
            self.comm.tolerant = True
        # routing weights: fixed ones from the configuration, or (routing = "adaptive") measured ones
        self.adaptive = config.swarm.routing == "adaptive"
        self.route_weights: Optional[List[float]] = list(config.swarm.routing_weights) or None
        self.rank_ms: List[float] = [0.0] * w.world_size      # running compute time per microbatch, per rank
        if self.adaptive and config.elastic.enable:
            raise NotImplementedError("adaptive routing shares its measurements over the whole world and does "
                                      "not follow membership changes; use routing = weighted with elastic runs")
        self._verify_plans = os.environ.get("DSWARM_VERIFY_PLANS", "0") == "1"
        self.timeline = None
        if config.logging.timeline_steps > 0:
            from .utils.timeline import StepTimeline
            self.timeline = StepTimeline(self.device, os.path.join(self.logger.log_dir, "timeline"), w.rank)
        self.opt_steps = 0           # optimiser steps taken so far (drives the LR schedule)
        self.num_train_steps = 0
        self.ckpt = Checkpoint(self.logger.checkpoint_dir)
        self.ckpt.setup(w)
        self.last_enqueue_s: float = 0.0
        self.timer = PhaseTimer(self.device, nvtx=os.environ.get("DSWARM_NVTX", "0") == "1")
        self.last_phase_ms: Dict[str, float] = {}
        self.last_sync_phase_ms: Dict[str, float] = {}
        self.step_timed_out = False  # the last step ran past train.step_timeout (NCCL: warned, then drained)
        self.timeouts_seen = 0

    # ------------------------------------------------------------------
    def _make_comm(self):
        """Pipeline transport: copy engines with stream-ordered flags where every rank can map every other
        rank's inbox (CUDA, one node, at most 8 ranks, no membership changes), NCCL / gloo point-to-point else."""
        cfg, w = self.config, self.world
        shape = (self.mbs, self.seq, cfg.model.n_embd)
        kind = cfg.swarm.p2p
        one_node = w.local_world_size == w.world_size
        fits = self.device.type == "cuda" and one_node and 1 < w.world_size <= 8 and not cfg.elastic.enable
        if kind == "auto":
            kind = "copy" if fits and w.num_stages > 1 else "nccl"
        if kind == "copy":
            if not fits:
                raise ValueError("swarm.p2p = copy needs CUDA ranks of one node (at most 8) and a static membership")
            from .parallel.ce_comm import CopyEngineComm
            return CopyEngineComm(w, shape, self.engine.act_dtype, self.device, slots=cfg.swarm.p2p_slots)
        return PipelineComm(w, shape, self.engine.act_dtype, self.device, prefetch=max(0, cfg.swarm.recv_prefetch))

    def _resolve_layer_split(self) -> None:
        """``layer_split = balanced`` becomes explicit block counts before the stage is built: the cut that
        minimises the busiest stage's time per step under this run's routing (the busiest replica of a later
        stage serves more than its even share of the microbatches when the wiring is uniformly random).
        Also fixes the per-stage forward / backward costs that order each rank's operations in the plan:
        with the nominal 1 : 2 of every stage the simulated arrival order differs from the real one wherever
        stages are uneven, and a rank then waits for a tensor while another one is already there."""
        from .models.gpt2 import FWD_SHARE, balanced_split, split_layers, stage_cost_blocks
        sw, mc, w = self.config.swarm, self.config.model, self.world
        S = w.num_stages
        if sw.layer_split == "balanced" and S > 1:
            mode = "weighted" if sw.routing == "adaptive" else sw.routing
            weights = list(sw.routing_weights) or None
            loads = schedule.busiest_replica_loads(self.routing_seed, S, w.world_size, self.num_micro, mode, weights)
            counts = balanced_split(mc.n_layer, S, mc.n_embd, mc.vocab_size, loads)
            sw.layer_split = ",".join(str(c) for c in counts)
        layers = split_layers(mc.n_layer, S, sw.layer_split, mc.n_embd, mc.vocab_size)
        cost = [stage_cost_blocks(len(layers[s]), s == 0, s == S - 1, mc.n_embd, mc.vocab_size) for s in range(S)]
        self.cost_f = [FWD_SHARE * c for c in cost]
        self.cost_b = [(1.0 - FWD_SHARE) * c for c in cost]

    def _plan(self, step: int, phase: int, forward_only: bool):
        w = self.world
        # phase separates the routing streams of train / eval / test steps
        mode = "weighted" if self.adaptive else self.config.swarm.routing
        path = schedule.route(self.routing_seed + 7919 * phase, step, w.num_stages, w.world_size,
                              self.num_micro, self.alive, mode=mode, weights=self.route_weights)
        cap = self.config.train.max_micro_batches
        if self._verify_plans:
            # debugging aid: every rank derives all ranks' plans and replays them before it runs its own
            every = {r: schedule.plan(path, w.world_size, r, cap, forward_only=forward_only,
                                      cost_f=self.cost_f, cost_b=self.cost_b)
                     for r in range(w.world_size) if self.alive is None or self.alive[r]}
            schedule.check_plans(path, every, cap, forward_only=forward_only)
        return path, schedule.plan(path, w.world_size, w.rank, cap, forward_only=forward_only,
                                   cost_f=self.cost_f, cost_b=self.cost_b)

    def _traced(self, name: str):
        """A named span on this rank's lane of the timeline, when one is being recorded."""
        if self.timeline is not None and self.timeline.step is not None:
            return self.timeline.op(name)
        return contextlib.nullcontext()

    def _compute(self, name: str):
        """Brackets one forward / backward of the step: a span on the timeline, and the compute time per
        microbatch when routing adapts to measured speeds (device time on GPUs, events on the compute
        stream after the wait for the op's input; wall time on CPU)."""
        sw = self.config.swarm
        if self.adaptive or (sw.straggler_rank == self.world.rank and sw.straggler_ms > 0):
            return self._both(self._traced(name), self._measured())
        return self._traced(name)

    def _measured(self):
        sw = self.config.swarm
        if sw.straggler_rank == self.world.rank and sw.straggler_ms > 0:
            return self._slowed(sw.straggler_ms)
        return self.timer.phase("compute")

    @staticmethod
    @contextlib.contextmanager
    def _both(a, b):
        with a, b:
            yield

    @contextlib.contextmanager
    def _slowed(self, ms: float):
        with self.timer.phase("compute"):
            time.sleep(ms / 1e3)          # injected heterogeneity: this rank is that much slower per op
            yield

    def _share_speeds(self, compute_ms: float, n_ops: int) -> None:
        """Every rank contributes its compute time per microbatch of this step; the running means become
        the routing weights (1 / time) of the following steps, the same on every rank.  The first stage
        keeps its round-robin chunks, so only later stages are rebalanced."""
        w, a = self.world, self.config.swarm.adaptive_ema
        mine = torch.tensor([compute_ms / n_ops if n_ops else 0.0], dtype=torch.float64, device=self.device)
        got = [torch.zeros_like(mine) for _ in range(w.world_size)]
        dist.all_gather(got, mine)
        for r, t in enumerate(got):
            v = float(t.item())
            if v > 0:
                self.rank_ms[r] = v if self.rank_ms[r] == 0 else (1 - a) * self.rank_ms[r] + a * v
        known = [t for t in self.rank_ms if t > 0]
        if known:
            default = sum(known) / len(known)         # a rank that has not worked yet counts as average
            self.route_weights = [1.0 / (t if t > 0 else default) for t in self.rank_ms]

    def _stage_batch(self, batch: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        """Move what this stage needs of the global batch to the device."""
        eng, out = self.engine, {}
        if eng.is_first:
            out["input_ids"] = batch["input_ids"].to(self.device, non_blocking=True)
        if eng.is_last:
            out["target_ids"] = batch["target_ids"].to(self.device, non_blocking=True)
            out["attention_mask"] = batch["attention_mask"].to(self.device, non_blocking=True)
        return out

    # ------------------------------------------------------------------
    def _update_membership(self, step: int) -> None:
        mask = self.membership.begin_step(step)
        if self.alive is None or mask != self.alive:
            if self.alive is not None or not all(mask):
                gone = [r for r, a in enumerate(mask) if not a]
                self.logger.log_message(f"Step {step}: ranks {gone} are gone, re-routing around them",
                                        master=False, level=Level.WARNING)
                self.world.regroup(mask, rebuild_p2p=self._step_failed)
                self._step_failed = False
                self.micro_per_device = max(1, self.num_micro // len(self.world.last_stage_ranks))
                self.loss_scale = 1.0 / self.micro_per_device
            self.alive = mask
        if self._step_failed:
            # the last step was abandoned with transfers in flight and nobody left: fresh pipeline groups
            # all the same, so that its leftovers cannot meet this step's messages
            self.world.regroup(mask, rebuild_p2p=True)
            self._step_failed = False

    def _run_plan(self, ops, dev: Dict[str, torch.Tensor], loss_acc: torch.Tensor, sync_here: bool, last_bwd: int) -> None:
        """This rank's forwards and backwards of one training step in plan order, with their transfers.
        ``loss_acc`` collects the last stage's scaled losses; ``self._served`` counts the microbatches
        started, so that a step that is cut short still reports what it did."""
        eng, comm = self.engine, self.comm
        comm.begin_step(ops, timeout_s=self.config.train.step_timeout)
        for i, op in enumerate(ops):
            rows = D.micro_batch_rows(op.mb, self.mbs)
            comm.tick(i)
            if op.kind == BWD:
                dy = comm.recv(i)
                with self._compute(f"B{op.mb}"):
                    dx = eng.backward(op.mb, dy, sync=sync_here and i == last_bwd)
                if op.prev >= 0:
                    comm.send_backward(dx, op.prev)
                continue
            self._served += 1
            ids = dev["input_ids"][rows] if eng.is_first else None
            hidden = comm.recv(i) if op.prev >= 0 else None
            if op.kind == FWD:
                with self._compute(f"F{op.mb}"):
                    y = eng.forward(op.mb, ids, hidden)
                comm.send_forward(y, op.next)
            else:
                with self._compute(f"FB{op.mb}"):
                    loss, dx = eng.forward_backward(op.mb, ids, hidden, dev["target_ids"][rows],
                                                    dev["attention_mask"][rows], self.loss_scale,
                                                    sync=sync_here and i == last_bwd)
                loss_acc += loss
                if op.prev >= 0:
                    comm.send_backward(dx, op.prev)
        comm.end_step()

    def _watch_step_deadline(self, step: int, deadline: float, what: str = "Train") -> None:
        """Step timeout on NCCL.  The reference warns and leaves its event loop when a step takes longer than
        ``train.step_timeout`` and still reaches the barrier (src/train.py:186,245).  Here the whole step is
        already queued on the device when the host gets here, and a posted NCCL transfer cannot be withdrawn, so
        the host watches an event at the end of the step's work: past the deadline it logs the reference's
        warning once and then keeps waiting until everything posted has drained (the slow peer does arrive, or
        the process group's own timeout ends the job), so that no leftover of this step can meet the next one.
        The step's update is applied: unlike the reference's abandoned loop, every microbatch did finish."""
        done = torch.cuda.Event()
        done.record()
        self.step_timed_out = False
        while not done.query():
            if time.time() > deadline:
                self.step_timed_out = True
                self.timeouts_seen += 1
                self.logger.log_message(f"{what} step {step} timed out", master=False, level=Level.WARNING)
                self.logger.log_message(f"Step {step}: waiting for the transfers already posted to drain",
                                        master=False, level=Level.WARNING)
                break
            time.sleep(0.0005)

    def train_step(self, step: int, batch: Dict[str, torch.Tensor]) -> Tuple[Outputs, Optional[Outputs]]:
        cfg, w, eng, comm = self.config, self.world, self.engine, self.comm
        start = time.time()
        if self.membership is not None:
            self._update_membership(step)
            el = cfg.elastic
            if el.die_rank == w.rank and el.die_at_step == step:
                # host-side fault injection: the step's routing counts on this rank and it is gone
                self.logger.log_message(f"Rank {w.rank} dies silently at step {step}", master=False, level=Level.WARNING)
                self.logger.close()
                os._exit(0)
        lg = cfg.logging
        if self.timeline is not None and lg.timeline_start <= step < lg.timeline_start + lg.timeline_steps:
            self.timeline.begin_step(step)
        eng.train()
        eng.zero_grad()
        _, ops = self._plan(step, 0, forward_only=False)
        dev = self._stage_batch(batch)
        tokens_per_mb = self.mbs * self.seq
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        H = cfg.swarm.sync_every_n_steps
        do_sync = (H > 0 and step % H == 0) or step == self.num_train_steps
        # the static plan tells which backward is this rank's last one: when the step ends with a
        # gradient all-reduce, that backward sends each bucket as soon as it is complete
        last_bwd = max((i for i, op in enumerate(ops) if op.kind in (BWD, FWD_BWD)), default=-1)
        sync_here = do_sync and not eng.has_outer
        failed = False
        tolerated = (StepTimeout, RuntimeError) if self.membership is not None else (StepTimeout,)
        self._served = 0             # microbatches this rank has started in this step
        with self.timer.phase("pipeline"):
            try:
                self._run_plan(ops, dev, loss_acc, sync_here, last_bwd)
            except tolerated as e:
                failed = True
                self.logger.log_message(f"Train step {step} timed out" if isinstance(e, StepTimeout) and "imeout" in str(e)
                                        else f"Train step {step} failed: {type(e).__name__}: {str(e)[:200]}",
                                        master=False, level=Level.WARNING)
                comm.abandon_step()
        n_local = self._served

        lr = cfg.train.inner_optimizer.lr * lr_factor(self.opt_steps, cfg.train.scheduler, self.num_train_steps)
        applied = True
        if self.membership is not None:
            # one verdict for everybody: either every live rank applies this step or none does
            applied = self.membership.vote(step, not failed, cfg.train.step_timeout + cfg.elastic.timeout)
            if not applied:
                self._step_failed = True
                self.logger.log_message(f"Step {step} is dropped: not every rank got through it", master=False,
                                        level=Level.WARNING)
        norm = 0.0
        if applied:
            if do_sync and not eng.has_outer:
                with self.timer.phase("grad_sync"), self._traced("grad_sync"):
                    eng.sync_gradients()
            with self.timer.phase("optimizer"), self._traced("optimizer"):
                norm = eng.optimizer_step(lr, cfg.train.max_norm)
            self.opt_steps += 1
            if do_sync and eng.has_outer:
                with self._traced("outer_sync"):
                    eng.outer_step(timer=self.timer)     # phases "outer_wait" (replica skew) and "outer_sync"
        self.last_enqueue_s = time.time() - start   # host time to queue the whole step
        if comm.device_async and w.world_size > 1 and not failed:
            self._watch_step_deadline(step, start + cfg.train.step_timeout)
        loss_val = float(loss_acc.item())      # the step's one device-to-host read
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        eng.check_status()
        self.last_phase_ms = self.timer.collect()
        if do_sync and applied:
            self.last_sync_phase_ms = dict(self.last_phase_ms)     # phases of the latest step that synchronised
        if self.timeline is not None:
            self.timeline.end_step()
        if self.adaptive and w.world_size > 1:
            self._share_speeds(self.last_phase_ms.get("compute", 0.0), len(ops))
        self.logger.log_message(f"Step {step} device phases (ms): {self.last_phase_ms}", master=False, level=Level.DEBUG)
        step_time = time.time() - start
        local = Outputs(step=step, lr=lr, loss=loss_val, tokens=n_local * tokens_per_mb, norm=float(norm),
                        time=step_time, micro_step_time=step_time / self.micro_per_device,
                        num_micro_batches=n_local)
        stage = sync_outputs(w, local, self.device) if (do_sync and applied) else None
        if self.membership is not None:
            self.membership.end_step(step)
        return local, stage

    # ------------------------------------------------------------------
    @torch.no_grad()
    def eval_step(self, step: int, eval_type: str, batch: Dict[str, torch.Tensor]) -> Tuple[Outputs, Outputs]:
        w, eng, comm = self.world, self.engine, self.comm
        start = time.time()
        eng.eval()
        _, ops = self._plan(step, 1 if eval_type == "eval" else 2, forward_only=True)
        dev = self._stage_batch(batch)
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        n_local = 0
        comm.begin_step(ops)
        for i, op in enumerate(ops):
            rows = D.micro_batch_rows(op.mb, self.mbs)
            comm.tick(i)
            n_local += 1
            ids = dev["input_ids"][rows] if eng.is_first else None
            hidden = comm.recv(i) if op.prev >= 0 else None
            if eng.is_last:
                loss_acc += eng.forward_loss(ids, hidden, dev["target_ids"][rows],
                                             dev["attention_mask"][rows], self.loss_scale)
            else:
                comm.send_forward(eng.forward(op.mb, ids, hidden, keep=False), op.next)
        comm.end_step()
        if comm.device_async and w.world_size > 1:
            # the reference's evaluation loop has no deadline at all (src/train.py:99); here a peer that is late
            # gets the same warning as in training before the host blocks on the loss
            self._watch_step_deadline(step, start + self.config.train.step_timeout, what=eval_type.capitalize())
        loss_val = float(loss_acc.item())
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        local = Outputs(step=step, time=time.time() - start, loss=loss_val,
                        tokens=n_local * self.mbs * self.seq, num_micro_batches=n_local)
        return local, sync_outputs(w, local, self.device)

    def eval_loop(self, eval_type: str, loader: D.BatchLoader, metrics) -> Dict[str, float]:
        metrics.reset()
        limit = self.config.eval.max_steps
        total = min(limit, len(loader)) if limit > 0 else len(loader)
        # second progress bar on the master's terminal, as in the reference (src/train.py:147)
        bar = tqdm(total=total, position=1, leave=False, disable=not (self.world.is_master and sys.stderr.isatty()))
        for step, batch in enumerate(loader, start=1):
            if 0 < limit < step:
                break
            _, stage = self.eval_step(step, eval_type, batch)
            if self.world.is_master:
                metrics.update(stage)
                bar.set_description(get_eval_pbar_description(metrics, f"[{eval_type.upper()}]"))
            bar.update(1)
        bar.close()
        return metrics.compute()

    # ------------------------------------------------------------------
    @torch.no_grad()
    def sample_loop(self, tokenizer) -> List[str]:
        """Autoregressive sampling through the stage leaders with whole-sequence
        recompute per token, as in the reference (src/train.py:46-74).  Hidden
        states travel leader to leader; the new ids and the stop flag come back
        in one broadcast from the last leader, so every rank ends with the final
        ids.  Temperature and top-k are applied (the reference ignores them)."""
        sc, w, eng = self.config.sample, self.world, self.engine
        eng.eval()
        prompt_len = len(tokenizer.encode(sc.prompt))
        total = min(prompt_len + sc.max_new_tokens, self.config.model.block_size)
        ids = D.tokenize(sc.prompt, tokenizer, max_length=total)["input_ids"].repeat(sc.num_samples, 1)
        # last column carries the stop flag
        state = torch.cat([ids, torch.zeros(sc.num_samples, 1, dtype=torch.long)], dim=1).to(self.device)
        ring = InferenceComm(w, self.device)
        d = self.config.model.n_embd
        gen = torch.Generator(device=self.device).manual_seed(self.config.train.seed + 17)
        multi = w.world_size > 1
        for pos in range(prompt_len, total):
            if w.is_leader:
                hidden = None
                if not w.is_first_stage:
                    hidden = ring.recv_hidden((sc.num_samples, total, d), torch.float32)
                out = eng.forward_infer(state[:, :total] if w.is_first_stage else None, hidden)
                if w.is_last_stage:
                    nxt = sample_next(out[:, pos - 1, :].float(), sc.temperature, sc.top_k, gen)
                    state[:, pos] = nxt.squeeze(1)
                    if bool((nxt == tokenizer.eos_token_id).all()):
                        state[:, total] = 1
                else:
                    ring.send_hidden(out)
            if multi:
                self._share_sample_state(state)
            if bool(state[0, total].item()):
                break
        return [tokenizer.decode(row, skip_special_tokens=True) for row in state[:, :total].cpu()]

    def _share_sample_state(self, state: torch.Tensor) -> None:
        """New ids and stop flag from the last leader to everybody.  One broadcast while the world is
        whole; once ranks are gone the broadcast's group would wait for them, so the last leader sends to
        each live rank instead."""
        w = self.world
        if self.alive is None or all(self.alive):
            dist.broadcast(state, src=w.last_stage_leader)
        elif w.rank == w.last_stage_leader:
            for r, a in enumerate(self.alive):
                if a and r != w.rank:
                    dist.send(state, dst=r)
        else:
            dist.recv(state, src=w.last_stage_leader)

    # ------------------------------------------------------------------
    def save_checkpoint(self, step: int) -> None:
        eng = self.engine
        self.ckpt.save(step, eng)
        self.ckpt.save_extra(step, "optim", {"engine": eng.optim_state(), "opt_steps": self.opt_steps})
        outer = eng.outer_state()
        if outer is not None:
            self.ckpt.save_extra(step, "outer", outer)
        if self.world.is_master:
            self.ckpt.save_meta(step, {
                "step": step, "opt_steps": self.opt_steps, "world_size": self.world.world_size,
                "num_stages": self.world.num_stages, "routing_seed": self.routing_seed,
                "engine": eng.name, "config": self.config.model_dump()})
        self.world.barrier()

    def load_checkpoint(self, step: Optional[int] = None) -> int:
        step = step if step is not None else self.ckpt.get_latest_step()
        if step is None:
            return 0
        self.engine.load_state_dict(self.ckpt.load(step))
        opt = self.ckpt.load_extra(step, "optim")
        if opt is not None:
            self.engine.load_optim_state(opt["engine"])
            self.opt_steps = int(opt["opt_steps"])
        outer = self.ckpt.load_extra(step, "outer")
        if outer is not None:
            self.engine.load_outer_state(outer)
        elif self.engine.has_outer:
            self.engine.reset_outer()       # weights without their DiLoCo state (a resharded checkpoint)
        self.world.barrier()
        return step

    # ------------------------------------------------------------------
    def train_loop(self, train_loader: D.BatchLoader, eval_loader: Optional[D.BatchLoader], tokenizer,
                   num_train_steps: int) -> Dict[str, float]:
        cfg, w, log = self.config, self.world, self.logger
        self.num_train_steps = num_train_steps
        local_m, global_m, eval_m = train_metrics("train/local"), train_metrics("train/global"), eval_metrics("eval")
        start_step = 0
        if cfg.ckpt.resume:
            start_step = self.load_checkpoint(cfg.ckpt.step)
            log.log_message(f"Resumed from step {start_step}", master=True, level=Level.INFO)
        if cfg.sample.enable and start_step == 0:
            log.log_samples(self.sample_loop(tokenizer), step=0)
        if cfg.eval.enable and start_step == 0:
            log.log_metrics(self.eval_loop("eval", eval_loader, eval_m), step=0, master=True)
        last: Dict[str, float] = {}
        it = iter(train_loader)
        for _ in range(start_step):      # sequential loader: skip what was consumed
            next(it)
        step = start_step
        # progress bar on the master's terminal, as in the reference (src/train.py:311); off when the
        # output is not a terminal so that logs and test captures stay clean
        bar = tqdm(total=num_train_steps, initial=start_step, position=0, leave=False,
                   disable=not (w.is_master and sys.stderr.isatty()))
        for step in range(start_step + 1, num_train_steps + 1):
            batch = next(it)
            el = cfg.elastic
            if self.membership is not None and el.leave_rank == w.rank and el.leave_after_step == step:
                self.membership.announce_leave(step)
            local, stage = self.train_step(step, batch)
            local_m.update(local)
            log.log_metrics(local_m.compute(), step=step, master=False)
            bar.update(1)
            if w.is_master and stage is not None:
                global_m.update(stage)
                bar.set_description(get_train_pbar_description(global_m, "[TRAIN]"))
                last = global_m.compute()
                log.log_metrics(last, step=step, master=True)
                g = last
                log.log_message(
                    f"[TRAIN] Step: {step} - Time: {g['train/global/time/current']:.2f}s - "
                    f"Loss: {g['train/global/loss/current']:.4f} - Norm: {g['train/global/norm/current'] or 0:.4f} - "
                    f"Perplexity: {g['train/global/perplexity/current']:.1f} - "
                    f"Throughput: {g['train/global/throughput/current']:.1f}", master=True, level=Level.INFO)
            if cfg.sample.enable and cfg.sample.every_n_steps > 0 and step % cfg.sample.every_n_steps == 0:
                log.log_samples(self.sample_loop(tokenizer), step=step)
            if cfg.eval.enable and cfg.eval.every_n_steps > 0 and step % cfg.eval.every_n_steps == 0:
                log.log_metrics(self.eval_loop("eval", eval_loader, eval_m), step=step, master=True)
            if cfg.ckpt.enable and cfg.ckpt.every_n_steps > 0 and step % cfg.ckpt.every_n_steps == 0:
                self.save_checkpoint(step)
            if self.membership is not None and el.leave_rank == w.rank and el.leave_after_step == step:
                log.log_message(f"Rank {w.rank} leaves after step {step}", master=False, level=Level.WARNING)
                self.left = True
                bar.close()
                return last
        bar.close()
        if cfg.eval.enable:
            out = self.eval_loop("test", eval_loader, eval_m)
            log.log_metrics(out, step=step, master=True)
            if w.is_master:
                log.log_message(f"[TEST] Avg. Loss: {out['eval/loss/average']:.4f}, "
                                f"Avg. Perplexity: {out['eval/perplexity/average']:.1f}", master=True, level=Level.INFO)
        if cfg.sample.enable:
            log.log_samples(self.sample_loop(tokenizer), step=step)
        if cfg.ckpt.enable:
            self.save_checkpoint(step)
        return last


def main(config: Config) -> Dict[str, float]:
    dump_s = float(os.environ.get("DSWARM_STACK_DUMP_S", "0"))
    if dump_s > 0:
        # hang diagnosis: print every thread's Python stack if the run is still going after dump_s seconds
        import faulthandler
        faulthandler.dump_traceback_later(dump_s, repeat=False, file=sys.stderr)
    trainer = Trainer(config)
    w, log = trainer.world, trainer.logger
    log.log_message(f"Starting process {w.local_rank}", master=False, level=Level.INFO)
    log.log_config(config)
    log.log_world(w)
    log.log_message(f"Using device {trainer.device}, engine {trainer.engine.name}", master=False, level=Level.INFO)
    log.log_message(f"Initialized stage model ({format_int(trainer.engine.num_parameters(), 2)} parameters)",
                    master=False, level=Level.INFO)
    tokenizer = D.get_tokenizer()
    log.log_message(f"Loaded tokenizer ({format_int(len(tokenizer), 0)} vocab size)", master=True, level=Level.INFO)
    data = D.get_dataset(config.data, tokenizer, seed=config.train.seed)
    train_data, val_data = data.train_test_split(config.eval.eval_size, seed=config.train.seed)
    log.log_message(f"Split dataset {config.data.path} into {format_int(len(train_data))} train, "
                    f"{format_int(len(val_data))} validation examples", master=True, level=Level.INFO)
    bs = config.train.batch_size
    train_loader = D.BatchLoader(train_data, bs, config.data.pin_memory)
    eval_loader = D.BatchLoader(val_data, bs, config.data.pin_memory)
    num_steps = D.get_num_steps(config.train.max_steps, config.train.max_epochs, len(train_data), bs)
    setup = D.get_train_setup(num_steps, bs, config.data.seq_length, config.train.micro_batch_size, len(train_data))
    log.log_message("Train setup:\t" + "\t".join(
        f"{k.replace('_', ' ').title()}: {format_int(v, 1) if isinstance(v, int) else format_float(v)}"
        for k, v in setup.items()), master=True, level=Level.INFO)
    out = trainer.train_loop(train_loader, eval_loader, tokenizer, num_steps)
    if trainer.membership is not None:
        # ranks that left are not waited for, and the process group is not torn down collectively
        if not getattr(trainer, "left", False):
            trainer.membership.barrier("end")
            if w.rank == 0:
                time.sleep(1.0)          # the store lives here: let the others read the barrier first
        log.close()
        os._exit(0)
    w.barrier()
    log.close()
    w.destroy()
    return out


if __name__ == "__main__":
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    main(config_from_argv())
