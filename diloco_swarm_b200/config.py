"""Configuration schema and command-line grammar.

Field names and defaults follow the reference's pydantic schema
(src/config.py:5-95 and the top-level model at src/train.py:35-44) so that the
reference's launch lines keep working.  The parser is self-contained: the
reference depends on an external ``parse_argv`` that is not installable
offline.

Grammar (observed in experiments/experiment1.sh:10-79 and
tests/test_memorize.py:10-33):

* ``--a.b.c value``  sets a nested key;
* ``--section @file.toml`` loads a TOML file as that sub-tree; dotted flags
  given later override keys inside it;
* booleans are the strings ``true`` / ``false``;
* ``--flag`` with no value means ``true``; ``--no-flag`` means ``false``.

Fields that do not exist in the reference are marked "(added)".
"""
from __future__ import annotations

import os
import sys
import tomllib
from typing import Any, Dict, List, Literal, Optional, Sequence

from pydantic import BaseModel, ConfigDict, field_validator


class BaseConfig(BaseModel):
    model_config = ConfigDict(extra="forbid", validate_assignment=True)


class SwarmConfig(BaseConfig):
    num_stages: int = 2
    sync_every_n_steps: int = 1
    # (added) seed of the counter-based routing generator; None = train.seed
    routing_seed: Optional[int] = None
    # (added) "uniform" = independent uniform draw per hop (reference, src/comm.py:91);
    # "balanced" = seeded random permutation with equal shares per replica.
    # "weighted" = draw proportional to routing_weights; "adaptive" = the same with weights measured while
    # training: the inverse of every rank's compute time per microbatch, shared after each step.
    routing: Literal["uniform", "balanced", "weighted", "adaptive"] = "uniform"
    # (added) one relative throughput per rank for routing = "weighted" (empty: all equal)
    routing_weights: List[float] = []
    # (added) weight of the newest measurement in the running mean that "adaptive" keeps per rank
    adaptive_ema: float = 0.5
    # (added) host-side heterogeneity injector for tests: this rank sleeps so long per microbatch op
    straggler_rank: int = -1
    straggler_ms: float = 0.0

    @field_validator("routing_weights", mode="before")
    @classmethod
    def _split_weights(cls, v):
        if isinstance(v, str):
            return [float(x) for x in v.split(",") if x.strip()]
        return [v] if isinstance(v, (int, float)) else v
    # (added) "even" = reference split (n_layer // S, remainder to the first
    # stages); "balanced" = weigh embedding / LM head when splitting blocks;
    # or an explicit comma list such as "7,5".
    layer_split: str = "even"
    # (added) stage-wide synchronisations: "fused" = hand-written kernels over peer loads / stores,
    # "nvls" = the same kernels with the reduction and the broadcast done inside the NVSwitch (multimem
    # instructions on multicast-bound buffers; falls back to "fused" where the box has no NVLS),
    # "nccl" = library all-reduce followed by separate update kernels.
    collective: Literal["fused", "nvls", "nccl"] = "fused"
    # (added) wire dtype of the per-step gradient all-reduce
    grad_wire_dtype: Literal["float32", "bfloat16"] = "float32"
    # (added) a pipeline receive is posted this many operations of the rank's plan before the operation that
    # consumes it (a posted NCCL receive is a resident kernel that waits for its sender, so more look-ahead
    # hides latency but holds SMs that the persistent GEMMs want)
    recv_prefetch: int = 1
    # (added) pipeline transport between stages: "nccl" = isend / irecv (a waiting transfer is a resident kernel),
    # "copy" = copy engines + stream-ordered flags into peer-mapped inboxes (no kernel at all; one node, up to 8
    # ranks); "auto" = "copy" where that applies (CUDA, one node), else "nccl"
    p2p: Literal["auto", "nccl", "copy"] = "auto"
    # (added) message slots per (sender, receiver) ring of the copy transport
    p2p_slots: int = 4
    # (added) bound of the fused collectives' waits for a peer GPU, in seconds (the kernels count clock cycles at
    # a nominal 2 GHz); a wait that runs out ends the kernel with a status that the host raises as an error
    peer_wait_s: float = 2.0


class ModelConfig(BaseConfig):
    n_layer: int
    n_head: int
    n_embd: int
    parameter_sharing: bool = False
    vocab_size: int = 50304  # (added) reference hard-codes it, src/model.py:16
    block_size: int = 1024   # (added) src/model.py:15
    bias: bool = True        # (added) src/model.py:21
    dropout: float = 0.0     # (added) src/model.py:20


class DataConfig(BaseConfig):
    path: str
    seq_length: int = 1024
    subset_size: float = 1.0
    tokenize: bool = False
    pin_memory: bool = True
    num_workers: int = 4
    # (added) number of synthetic sequences for the built-in generators
    num_examples: int = 0
    zipf_s: float = 1.0
    vocab_limit: int = 50257


class OptimizerConfig(BaseConfig):
    type: Literal["SGD", "AdamW", "None"]
    lr: float
    nesterov: bool = False
    momentum: float = 0.9
    weight_decay: float = 0.1
    betas: List[float] = [0.9, 0.95]
    eps: float = 1e-8  # (added) torch default used by the reference


class SchedulerConfig(BaseConfig):
    enable: bool = False
    num_warmup_steps: int = 100
    last_epoch: int = -1
    # (added) "constant" is the reference's live schedule (src/utils.py:78-85);
    # "cosine" is its commented-out variant (src/utils.py:67-76).
    type: Literal["constant", "cosine"] = "constant"
    min_lr_factor: float = 0.1
    num_cycles: float = 0.5


class AmpConfig(BaseConfig):
    enable: bool = True
    precision: Literal["highest", "high", "medium"] = "high"
    dtype: Literal["float32", "float16", "bfloat16"] = "bfloat16"


class TrainConfig(BaseConfig):
    max_epochs: int = 1
    max_steps: int = -1
    micro_batch_size: int = 16
    batch_size: int = 512
    max_micro_batches: int = 1
    seed: int = 42
    max_norm: float = 1.0
    step_timeout: float = 60
    deterministic: bool = False  # (added) fixed order of additions in the gradient kernels (sorted embedding scatter, no split-K)
    # (added) the LM head, the cross-entropy and the head's two gradient GEMMs run over this many slices of a
    # microbatch's token rows, one after the other, so that only a slice of the [tokens, vocabulary] logits
    # exists at a time (GPT-2 small, 16 x 1024 tokens: 1.65 GB for one slice, 0.41 GB for four); b200 engine
    lm_head_chunks: int = 1
    # (added) GB of device memory taken from the driver in one piece when the trainer starts and handed to the
    # caching allocator: later tensors are cut from it, so steps whose set of live tensors differs from every
    # step before (other routing, another batch layout) do not stop for cudaMalloc; 0 = off
    reserve_memory_gb: float = 0.0
    inner_optimizer: OptimizerConfig
    outer_optimizer: OptimizerConfig
    scheduler: SchedulerConfig = SchedulerConfig()


class EvalConfig(BaseConfig):
    enable: bool = True
    every_n_steps: int = -1
    eval_size: float = 0.1
    max_steps: int = -1  # (added) tests/test_train.py:19 passes it


class SampleConfig(BaseConfig):
    enable: bool = True
    every_n_steps: int = -1
    num_samples: int = 5
    prompt: str = "I am"
    max_new_tokens: int = 20
    temperature: float = 1.0
    top_k: Optional[int] = 20


class ConsoleLoggingConfig(BaseConfig):
    log_level: str = "INFO"


class FileLoggingConfig(BaseConfig):
    log_level: str = "DEBUG"


class WandbLoggingConfig(BaseConfig):
    enable: bool = False
    entity: Optional[str] = "mikasenghaas"
    project: Optional[str] = "diloco-swarm"
    tags: List[str] = []
    group: Optional[str] = None
    cache_dir: Optional[str] = None

    @field_validator("tags", mode="before")
    @classmethod
    def _split_tags(cls, v):
        return v.split(",") if isinstance(v, str) else v


class LoggingConfig(BaseConfig):
    log_dir: str = "logs"
    run_id: Optional[str] = None
    console: ConsoleLoggingConfig = ConsoleLoggingConfig()
    file: FileLoggingConfig = FileLoggingConfig()
    wandb: WandbLoggingConfig = WandbLoggingConfig()
    # (added) record start and end of every forward / backward of this many training steps, beginning
    # with step timeline_start, into <run>/timeline/<rank>.jsonl (utils/timeline.py); 0 = off
    timeline_steps: int = 0
    timeline_start: int = 2


class ElasticConfig(BaseConfig):
    """(added) host-side membership tracking and re-routing around ranks that leave.
    The reference's world is static (src/world.py) and has no counterpart."""
    enable: bool = False
    timeout: float = 30.0            # seconds the coordinator waits for a rank's end-of-step report
    # host-side fault injection for tests: this rank announces a leave and exits after that step
    leave_rank: int = -1
    leave_after_step: int = -1
    # ... and this rank exits without a word at the start of that step, after the step's routing
    # has been fixed with it in (the others find out by their transfers failing or timing out)
    die_rank: int = -1
    die_at_step: int = -1


class CkptConfig(BaseConfig):
    """(added) the reference defines a checkpoint layout (src/ckpt.py) but
    never writes one from the training loop."""
    enable: bool = False
    every_n_steps: int = -1
    resume: bool = False
    step: Optional[int] = None


class Config(BaseConfig):
    """Top-level configuration (reference: src/train.py:35-44)."""
    model: ModelConfig
    data: DataConfig
    train: TrainConfig
    device: Optional[str] = None
    amp: AmpConfig = AmpConfig()
    swarm: SwarmConfig = SwarmConfig()
    eval: EvalConfig = EvalConfig()
    sample: SampleConfig = SampleConfig()
    logging: LoggingConfig = LoggingConfig()
    ckpt: CkptConfig = CkptConfig()
    elastic: ElasticConfig = ElasticConfig()
    # (added) "torch" = autograd stage on library ops (CPU oracle and
    # debugging); "b200" = flat-buffer stage on the sm_100a kernels;
    # "auto" = b200 on CUDA devices, torch elsewhere.
    engine: Literal["auto", "torch", "b200"] = "auto"


# --------------------------------------------------------------------------
# command line
# --------------------------------------------------------------------------

def _coerce(text: str) -> Any:
    low = text.lower()
    if low == "true":
        return True
    if low == "false":
        return False
    if low in ("none", "null"):
        return None
    for cast in (int, float):
        try:
            return cast(text)
        except ValueError:
            pass
    return text


def _set_path(tree: Dict[str, Any], dotted: str, value: Any, merge: bool) -> None:
    keys = dotted.split(".")
    node = tree
    for k in keys[:-1]:
        nxt = node.get(k)
        if not isinstance(nxt, dict):
            nxt = {}
            node[k] = nxt
        node = nxt
    last = keys[-1]
    if merge and isinstance(value, dict) and isinstance(node.get(last), dict):
        _deep_update(node[last], value)
    else:
        node[last] = value


def _deep_update(dst: Dict[str, Any], src: Dict[str, Any]) -> None:
    for k, v in src.items():
        if isinstance(v, dict) and isinstance(dst.get(k), dict):
            _deep_update(dst[k], v)
        else:
            dst[k] = v


def load_toml(path: str, search: Sequence[str] = ()) -> Dict[str, Any]:
    """Load a preset.  Relative paths are tried against the working directory
    and then against each directory in ``search`` (the package ships the
    reference's preset names under ``configs/``)."""
    candidates = [path] + [os.path.join(s, path) for s in search]
    for c in candidates:
        if os.path.isfile(c):
            with open(c, "rb") as f:
                return tomllib.load(f)
    raise FileNotFoundError(f"preset not found: {path} (tried {candidates})")


def repo_root() -> str:
    return os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def parse_argv(argv: Optional[Sequence[str]] = None) -> Dict[str, Any]:
    """Turn ``--a.b value --c @file.toml`` into a nested dict."""
    args = list(sys.argv[1:] if argv is None else argv)
    tree: Dict[str, Any] = {}
    i = 0
    while i < len(args):
        tok = args[i]
        if not tok.startswith("--"):
            raise ValueError(f"expected a --flag, got {tok!r}")
        key = tok[2:]
        if "=" in key:
            key, val = key.split("=", 1)
            i += 1
        elif i + 1 < len(args) and not _looks_like_flag(args[i + 1]):
            val = args[i + 1]
            i += 2
        else:
            val = None
            i += 1
        if val is None:
            if key.startswith("no-") or key.startswith("no_"):
                _set_path(tree, key[3:], False, merge=False)
            else:
                _set_path(tree, key, True, merge=False)
        elif val.startswith("@"):
            _set_path(tree, key, load_toml(val[1:], search=(repo_root(),)), merge=True)
        else:
            _set_path(tree, key, _coerce(val), merge=False)
    return tree


def _looks_like_flag(tok: str) -> bool:
    if not tok.startswith("--"):
        return False
    return len(tok) > 2 and not tok[2].isdigit()


def config_from_argv(argv: Optional[Sequence[str]] = None) -> Config:
    return Config(**parse_argv(argv))
