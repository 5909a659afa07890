"""Learning-rate schedule and the library-op optimiser scheme (inner AdamW,
DiLoCo outer SGD-Nesterov) used by the autograd stage.

Reference: get_optimizer / get_scheduler (src/utils.py:59-85) and the DiLoCo
helpers (src/utils.py:195-226).  The sm_100a stage implements the same maths
in fused kernels (ops/optim.py); this file is also their oracle.
"""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch


def lr_factor(step_index: int, sched, num_steps: int) -> float:
    """Multiplier of the base learning rate for the ``step_index``-th optimiser
    step (0-based), i.e. what ``LambdaLR.get_last_lr()`` returns before that
    step in the reference (src/train.py:256).  Linear warm-up from 0, then
    constant (src/utils.py:78-85) or the cosine variant (src/utils.py:67-76)."""
    if not sched.enable:
        return 1.0
    w = sched.num_warmup_steps
    if step_index < w:
        return step_index / max(1, w)
    if sched.type == "constant":
        return 1.0
    progress = (step_index - w) / max(1, num_steps - w)
    progress = min(1.0, progress)
    cos = 0.5 * (1.0 + math.cos(math.pi * sched.num_cycles * 2.0 * progress))
    return sched.min_lr_factor + (1.0 - sched.min_lr_factor) * cos


def make_inner_optimizer(params: Iterable[torch.nn.Parameter], cfg) -> torch.optim.Optimizer:
    """One parameter group: weight decay applies to every tensor, biases,
    LayerNorm and embeddings included, as in the reference (src/utils.py:61)."""
    if cfg.type == "AdamW":
        return torch.optim.AdamW(params, lr=cfg.lr, weight_decay=cfg.weight_decay,
                                 betas=tuple(cfg.betas), eps=cfg.eps)
    if cfg.type == "SGD":
        return torch.optim.SGD(params, lr=cfg.lr, momentum=cfg.momentum, nesterov=cfg.nesterov)
    raise ValueError(f"Invalid optimizer type: {cfg.type}")


def nesterov_reference(theta_g: torch.Tensor, delta: torch.Tensor, buf: Optional[torch.Tensor],
                       lr: float, momentum: float, nesterov: bool = True):
    """torch.optim.SGD's update written out: buf <- mu*buf + g (buf = g on the
    first step), theta <- theta - lr*(g + mu*buf) with Nesterov, else
    theta <- theta - lr*buf.  Returns (theta, buf)."""
    if momentum == 0:
        return theta_g - lr * delta, buf
    buf = delta.clone() if buf is None else momentum * buf + delta
    upd = delta + momentum * buf if nesterov else buf
    return theta_g - lr * upd, buf


# ---------------------------------------------------------------------- DiLoCo helpers on modules
# The engines carry their own outer state (flat fp32 buffers on the GPU, sharded across replicas in the
# fused path).  These three functions are the module-level form of the same steps, for code written against
# the reference's helpers (src/utils.py:213-226): the outer copy stays where the caller puts it, by default
# on the device of the inner model (the reference moves it to the host and pays two copies per outer step).
def get_outer_model(inner_model: torch.nn.Module, device: Optional[torch.device] = None) -> torch.nn.Module:
    import copy
    outer = copy.deepcopy(inner_model)
    return outer.to(device) if device is not None else outer


@torch.no_grad()
def compute_pseudo_gradient(inner_model: torch.nn.Module, outer_model: torch.nn.Module) -> None:
    """outer.grad <- outer - inner, parameter by parameter."""
    for po, pi in zip(outer_model.parameters(), inner_model.parameters()):
        po.grad = po.detach() - pi.detach().to(po.device, po.dtype)


@torch.no_grad()
def sync_inner_model(outer_model: torch.nn.Module, inner_model: torch.nn.Module) -> None:
    """inner <- outer, parameter by parameter."""
    for po, pi in zip(outer_model.parameters(), inner_model.parameters()):
        pi.copy_(po.detach().to(pi.device, pi.dtype))


# ---------------------------------------------------------------------- factories under the reference's names
def get_optimizer(model, optimizer_config) -> Optional[torch.optim.Optimizer]:
    """torch optimiser over ``model.parameters()`` (one group), or None for ``type = "None"``
    (reference: src/utils.py:59-65)."""
    if optimizer_config.type == "None":
        return None
    return make_inner_optimizer(model.parameters(), optimizer_config)


def get_scheduler(optimizer: torch.optim.Optimizer, scheduler_config, num_steps: int = 0):
    """LambdaLR that follows ``lr_factor``: linear warm-up then constant as in the reference
    (src/utils.py:78-85), or warm-up plus cosine when ``scheduler_config.type == "cosine"``
    (``num_steps`` is then the length of the run)."""
    return torch.optim.lr_scheduler.LambdaLR(optimizer, lambda step: lr_factor(step, scheduler_config, num_steps))
