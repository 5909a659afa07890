"""Step outputs and running metrics.

Key format and semantics follow the reference (src/metrics.py:6-192):
``{name}/{metric}/{current|average|total}`` with names ``train/local``,
``train/global`` and ``eval``; throughput is tokens / time per update;
perplexity "average" is the arithmetic mean of per-update exp(loss)
(src/metrics.py:136-140), which is what the published perplexities use.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence


@dataclass
class Outputs:
    step: int
    time: float
    loss: float
    tokens: int
    num_micro_batches: int = 1
    lr: Optional[float] = None
    norm: Optional[float] = None
    micro_step_time: Optional[float] = None

    FIELDS = ("step", "time", "loss", "tokens", "num_micro_batches", "lr", "norm", "micro_step_time")

    def to_vector(self) -> List[float]:
        """Fixed-width float vector for the packed metrics all-gather (the
        reference pickles the object, src/comm.py:129).  None becomes NaN."""
        return [float("nan") if getattr(self, f) is None else float(getattr(self, f)) for f in self.FIELDS]

    @classmethod
    def from_vector(cls, v: Sequence[float]) -> "Outputs":
        def opt(x):
            return None if math.isnan(x) else float(x)
        return cls(step=int(v[0]), time=float(v[1]), loss=float(v[2]), tokens=int(v[3]),
                   num_micro_batches=int(v[4]), lr=opt(v[5]), norm=opt(v[6]), micro_step_time=opt(v[7]))


def aggregate_outputs(local: Outputs, all_outputs: Sequence[Outputs]) -> Outputs:
    """Combine the outputs of a stage's replicas (reference: sync_outputs,
    src/comm.py:125-149): tokens and microbatch counts are summed; time, loss,
    lr, norm and micro-step time are averaged over the replicas whose value is
    neither 0 nor missing, so a replica that received no microbatch does not
    dilute the loss."""
    def total(vals):
        return sum(v for v in vals if v is not None and v != 0)

    def mean(vals):
        kept = [v for v in vals if v is not None and v != 0]
        return sum(kept) / len(kept) if kept else 0

    return Outputs(
        step=local.step,
        tokens=int(total([o.tokens for o in all_outputs])),
        num_micro_batches=int(total([o.num_micro_batches for o in all_outputs])),
        time=mean([o.time for o in all_outputs]),
        loss=mean([o.loss for o in all_outputs]),
        lr=mean([o.lr for o in all_outputs]),
        norm=mean([o.norm for o in all_outputs]),
        micro_step_time=mean([o.micro_step_time for o in all_outputs]),
    )


class Metric:
    name = "metric"

    def __init__(self):
        self.values: List[float] = []

    def pick(self, o: Outputs) -> float:
        raise NotImplementedError

    def update(self, o: Outputs) -> None:
        self.values.append(self.pick(o))

    def reset(self) -> None:
        self.values = []

    def _cur(self) -> float:
        return self.values[-1] if self.values else 0

    def _avg(self) -> float:
        return sum(self.values) / len(self.values) if self.values else 0

    def compute(self) -> Dict[str, float]:
        return {"current": self._cur()}


class Step(Metric):
    name = "step"
    def pick(self, o): return o.step
    def reset(self): self.values = []


class Time(Metric):
    name = "time"
    def pick(self, o): return o.time


class MicroTime(Metric):
    name = "micro_time"
    def pick(self, o): return o.micro_step_time


class Tokens(Metric):
    name = "tokens"
    def pick(self, o): return o.tokens
    def compute(self): return {"current": self._cur(), "total": sum(self.values)}


class NumMicroBatches(Metric):
    """Running total, reported as ``current`` (src/metrics.py:87-99)."""
    name = "num_micro_batches"
    def pick(self, o): return o.num_micro_batches
    def compute(self): return {"current": sum(self.values)}


class Norm(Metric):
    name = "norm"
    def pick(self, o): return o.norm


class Loss(Metric):
    name = "loss"
    def pick(self, o): return o.loss
    def compute(self): return {"current": self._cur(), "average": self._avg()}


class Perplexity(Metric):
    name = "perplexity"
    def pick(self, o): return math.exp(min(o.loss, 700.0)) if o.loss > 0 else 0
    def compute(self): return {"current": self._cur(), "average": self._avg()}


class Throughput(Metric):
    name = "throughput"
    def pick(self, o): return o.tokens / o.time if o.time else 0.0
    def compute(self): return {"current": self._cur(), "average": self._avg()}


class LearningRate(Metric):
    name = "learning_rate"
    def pick(self, o): return o.lr


class Metrics:
    def __init__(self, metrics: List[Metric], name: str):
        self.metrics, self.name = metrics, name

    def update(self, o: Outputs) -> None:
        for m in self.metrics:
            m.update(o)

    def compute(self) -> Dict[str, float]:
        out: Dict[str, float] = {}
        for m in self.metrics:
            for k, v in m.compute().items():
                out[f"{self.name}/{m.name}/{k}"] = v
        return out

    def reset(self) -> None:
        for m in self.metrics:
            m.reset()


def train_metrics(name: str) -> Metrics:
    return Metrics([Step(), Time(), MicroTime(), Tokens(), NumMicroBatches(), Norm(), Loss(),
                    Perplexity(), Throughput(), LearningRate()], name=name)


def eval_metrics(name: str = "eval") -> Metrics:
    return Metrics([Throughput(), Loss(), Perplexity()], name=name)
