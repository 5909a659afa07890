"""Stage engine on library ops with autograd.

This is the CPU/gloo path, the debugging path on GPUs and the oracle the
sm_100a engine is tested against.  It follows the reference's numerics: fp32
parameters, optional autocast (src/train.py:199), mean cross-entropy over the
unmasked tokens divided by the per-replica microbatch count
(src/utils.py:184-193, src/train.py:217-218), per-rank gradient clipping
(src/train.py:255), AdamW, and the DiLoCo outer step of src/train.py:261-269
(kept on the device instead of the host).
"""
from __future__ import annotations

import contextlib
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .gpt2 import GPT2Config, TorchStage
from ..optim import make_inner_optimizer


class TorchEngine:
    name = "torch"

    def __init__(self, cfg: GPT2Config, world, config, device: torch.device):
        self.cfg, self.world, self.config, self.device = cfg, world, config, device
        self.model = TorchStage(cfg, world.stage, world.num_stages, seed=config.train.seed,
                                layer_split=config.swarm.layer_split).to(device)
        self.is_first, self.is_last = self.model.is_first, self.model.is_last
        amp = config.amp
        self.autocast = amp.enable and amp.dtype != "float32"
        self.amp_dtype = getattr(torch, amp.dtype)
        self.act_dtype = torch.float32      # residual stream stays fp32 under autocast
        self.inner = make_inner_optimizer(self.model.parameters(), config.train.inner_optimizer)
        self.base_lr = config.train.inner_optimizer.lr
        oc = config.train.outer_optimizer
        self.has_outer = oc.type != "None"
        self.outer_params = None
        self.outer_opt = None
        if self.has_outer:
            self.outer_params = [p.detach().clone().requires_grad_(True) for p in self.model.parameters()]
            self.outer_opt = make_inner_optimizer(self.outer_params, oc)
        for p in self.model.parameters():   # reference: initialize_gradients (src/utils.py:195-198)
            p.grad = torch.zeros_like(p)
        self.stash: Dict[int, Tuple[Optional[torch.Tensor], torch.Tensor]] = {}
        self.status = 0

    # ------------------------------------------------------------------
    def _ctx(self):
        if self.autocast:
            return torch.autocast(device_type=self.device.type, dtype=self.amp_dtype)
        return contextlib.nullcontext()

    def train(self):
        self.model.train()

    def eval(self):
        self.model.eval()

    def zero_grad(self) -> None:
        for p in self.model.parameters():
            if p.grad is not None:
                p.grad.zero_()

    def num_parameters(self) -> int:
        return self.model.num_parameters()

    # -- pipeline pieces -----------------------------------------------------
    def forward(self, key: int, input_ids: Optional[torch.Tensor], hidden: Optional[torch.Tensor],
                keep: bool = True) -> torch.Tensor:
        """Forward of a non-last stage.  ``keep`` stashes what backward needs."""
        if hidden is not None:
            hidden = hidden.to(self.device, self.act_dtype)
            if keep:
                hidden.requires_grad_(True)
        with self._ctx():
            y = self.model(input_ids=input_ids, hidden_states=hidden)
        if keep:
            self.stash[key] = (hidden, y)
        return y.detach()

    def backward(self, key: int, grad_out: torch.Tensor, sync: bool = False) -> Optional[torch.Tensor]:
        x, y = self.stash.pop(key)
        torch.autograd.backward(y, grad_tensors=grad_out.to(y.dtype))
        return x.grad if x is not None else None

    def _loss(self, logits: torch.Tensor, targets: torch.Tensor, mask: torch.Tensor, scale: float):
        keep = mask.reshape(-1).bool()
        lg = logits.reshape(-1, logits.size(-1))[keep]
        tg = targets.reshape(-1)[keep]
        return F.cross_entropy(lg.float() if not self.autocast else lg, tg) * scale

    def forward_backward(self, key: int, input_ids, hidden, targets, mask, scale: float, sync: bool = False
                         ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Last stage: forward, masked mean CE times ``scale``, backward."""
        if hidden is not None:
            hidden = hidden.to(self.device, self.act_dtype).requires_grad_(True)
        with self._ctx():
            logits = self.model(input_ids=input_ids, hidden_states=hidden)
            loss = self._loss(logits, targets, mask, scale)
        loss.backward()
        return loss.detach(), (hidden.grad if hidden is not None else None)

    @torch.no_grad()
    def forward_loss(self, input_ids, hidden, targets, mask, scale: float) -> torch.Tensor:
        with self._ctx():
            logits = self.model(input_ids=input_ids, hidden_states=hidden)
            return self._loss(logits, targets, mask, scale)

    @torch.no_grad()
    def forward_infer(self, input_ids, hidden) -> torch.Tensor:
        """Hidden states (non-last stage) or logits (last stage), no stash."""
        with self._ctx():
            return self.model(input_ids=input_ids, hidden_states=hidden).float()

    # -- synchronisation and optimisers ------------------------------------------
    def sync_gradients(self) -> None:
        """Average gradients over the stage's replicas (reference: per-parameter
        all_reduce then divide, src/comm.py:117-123; here one flat buffer)."""
        R = self.world.num_replicas
        if R == 1:
            return
        grads = [p.grad for p in self.model.parameters()]
        flat = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.world.curr_stage_group)
        flat.div_(R)
        off = 0
        for g in grads:
            n = g.numel()
            g.copy_(flat[off:off + n].view_as(g))
            off += n

    def optimizer_step(self, lr: float, max_norm: float) -> float:
        norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), max_norm)
        for grp in self.inner.param_groups:
            grp["lr"] = lr
        self.inner.step()
        return float(norm)

    def outer_step(self, timer=None) -> None:
        """pseudo-gradient = outer - inner, averaged over the stage, outer
        optimiser step, inner <- outer (src/utils.py:218-226, src/train.py:261-269)."""
        if timer is not None:
            with timer.phase("outer_sync"):
                return self.outer_step()
        R = self.world.num_replicas
        with torch.no_grad():
            for po, pi in zip(self.outer_params, self.model.parameters()):
                po.grad = po.data - pi.data
            if R > 1:
                flat = torch.cat([p.grad.reshape(-1) for p in self.outer_params])
                dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=self.world.curr_stage_group)
                flat.div_(R)
                off = 0
                for p in self.outer_params:
                    n = p.numel()
                    p.grad.copy_(flat[off:off + n].view_as(p))
                    off += n
        self.outer_opt.step()
        with torch.no_grad():
            for po, pi in zip(self.outer_params, self.model.parameters()):
                pi.data.copy_(po.data)

    def check_status(self) -> None:
        pass

    # -- checkpoint ------------------------------------------------------------
    def state_dict(self) -> Dict[str, torch.Tensor]:
        return self.model.state_dict()

    def load_state_dict(self, sd) -> None:
        self.model.load_state_dict(sd)

    def optim_state(self) -> dict:
        return {"inner": self.inner.state_dict()}

    def load_optim_state(self, st: dict) -> None:
        self.inner.load_state_dict(st["inner"])

    def outer_state(self) -> Optional[dict]:
        if not self.has_outer:
            return None
        return {"params": [p.detach().cpu() for p in self.outer_params], "opt": self.outer_opt.state_dict()}

    def reset_outer(self) -> None:
        """Global weights := current weights, outer momentum := 0 (after loading weights that come
        without their DiLoCo state, e.g. a checkpoint moved to another topology)."""
        if not self.has_outer:
            return
        with torch.no_grad():
            for po, pi in zip(self.outer_params, self.model.parameters()):
                po.copy_(pi)
        self.outer_opt.state.clear()

    def load_outer_state(self, st: Optional[dict]) -> None:
        if st is None or not self.has_outer:
            return
        with torch.no_grad():
            for p, q in zip(self.outer_params, st["params"]):
                p.copy_(q)
        self.outer_opt.load_state_dict(st["opt"])
