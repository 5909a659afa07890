"""GPT-2 in plain PyTorch: the numerical oracle and the CPU/gloo stage.

Architecture as in the reference (src/model.py:13-152): learned positions,
pre-LayerNorm blocks (eps 1e-5), fused QKV projection, causal attention with
scale 1/sqrt(head_size), exact-erf GELU MLP of width 4d, final LayerNorm and
a bias-free LM head; weights N(0, 0.02), residual output projections
N(0, 0.02/sqrt(2*n_layer)), biases zero.

Unlike the reference (src/train.py:376-377, every rank builds the whole model
and throws most of it away) a stage builds only its own tensors.  Every tensor
is drawn from its own generator seeded by (seed, global tensor name), so any
S x R split starts from exactly the single-process model.
"""
from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPT2Config:
    block_size: int = 1024
    vocab_size: int = 50304
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    dropout: float = 0.0
    bias: bool = True
    parameter_sharing: bool = False


# Cost of the non-block parts of a stage in units of one transformer block, as measured on B200 for a
# 16k-token GPT-2 small microbatch (block 1.21 ms; final LayerNorm + LM head + loss 3.9 ms, which by FLOPs
# alone would be V / (12 d) = 5.5 blocks: a block also carries attention, LayerNorms and bias work;
# embedding forward + backward 0.2 ms).
HEAD_COST_PER_FLOP_BLOCK = 0.59
EMBED_COST_BLOCKS = 0.15
FWD_SHARE = 0.32          # forward part of a block's (and the head's) forward + backward time


def stage_cost_blocks(n_blocks: int, first: bool, last: bool, n_embd: int, vocab_size: int) -> float:
    """Forward + backward time of a stage per microbatch, in units of one transformer block."""
    c = float(n_blocks)
    if first:
        c += EMBED_COST_BLOCKS
    if last:
        c += HEAD_COST_PER_FLOP_BLOCK * vocab_size / (12.0 * n_embd)
    return c


def balanced_split(n_layer: int, num_stages: int, n_embd: int, vocab_size: int,
                   loads: Optional[Sequence[float]] = None) -> List[int]:
    """Blocks per stage (each at least one) that minimise the busiest stage's time per step,
    max over stages of load_s * cost_s.  ``loads`` = microbatches the busiest replica of each stage serves
    per step (all equal when omitted): under uniform stochastic wiring the later stages' busiest replicas
    get more than their even share, so they should carry less work per microbatch."""
    S = num_stages
    if S > n_layer:
        raise ValueError(f"{S} stages need at least {S} layers")
    w = [1.0] * S if loads is None else [float(x) for x in loads]
    INF = float("inf")
    # dp[s][i]: best bottleneck with stages 0..s covering blocks 0..i-1; second key = sum of squares (evenness)
    dp = [[(INF, INF)] * (n_layer + 1) for _ in range(S)]
    cut = [[0] * (n_layer + 1) for _ in range(S)]
    for i in range(1, n_layer + 1):
        c = w[0] * stage_cost_blocks(i, True, S == 1, n_embd, vocab_size)
        dp[0][i] = (c, c * c)
    for s in range(1, S):
        for i in range(s + 1, n_layer + 1):
            for j in range(s, i):
                if dp[s - 1][j][0] == INF:
                    continue
                c = w[s] * stage_cost_blocks(i - j, False, s == S - 1, n_embd, vocab_size)
                cand = (max(dp[s - 1][j][0], c), dp[s - 1][j][1] + c * c)
                if cand < dp[s][i]:
                    dp[s][i], cut[s][i] = cand, j
    counts, i = [0] * S, n_layer
    for s in range(S - 1, 0, -1):
        j = cut[s][i]
        counts[s], i = i - j, j
    counts[0] = i
    return counts


def split_layers(n_layer: int, num_stages: int, mode: str = "even",
                 n_embd: int = 768, vocab_size: int = 50304) -> List[List[int]]:
    """Block indices per stage.

    "even": n_layer // S each, remainder to the first stages (src/model.py:195-198).
    "balanced": fewer blocks on the last stage to make room for the LM head and the loss
    (``balanced_split`` with equal loads; the trainer replaces "balanced" by the explicit counts it gets
    with the loads of the run's routing before it builds the stage).
    "a,b,c": explicit counts.
    """
    S = num_stages
    if mode == "even":
        counts = [n_layer // S + (1 if i < n_layer % S else 0) for i in range(S)]
    elif mode == "balanced":
        counts = balanced_split(n_layer, S, n_embd, vocab_size)
    else:
        counts = [int(x) for x in mode.split(",")]
        if len(counts) != S or sum(counts) != n_layer:
            raise ValueError(f"layer_split {mode!r} does not cover {n_layer} layers over {S} stages")
    out, start = [], 0
    for c in counts:
        out.append(list(range(start, start + c)))
        start += c
    return out


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def init_tensor(name: str, shape: Sequence[int], seed: int, n_layer: int) -> torch.Tensor:
    """Deterministic fp32 initial value of the tensor with the given GLOBAL name."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "bias":
        return torch.zeros(*shape)
    if ".ln_" in name or name.startswith("transformer.ln_f"):
        return torch.ones(*shape)
    std = 0.02 / math.sqrt(2 * n_layer) if name.endswith("c_proj.weight") else 0.02
    g = torch.Generator(device="cpu")
    g.manual_seed(tensor_seed(seed, name))
    return torch.empty(*shape).normal_(0.0, std, generator=g)


def block_param_shapes(d: int, bias: bool = True) -> List[Tuple[str, Tuple[int, ...]]]:
    names = [("ln_1.weight", (d,)), ("ln_1.bias", (d,)),
             ("attn.c_attn.weight", (3 * d, d)), ("attn.c_attn.bias", (3 * d,)),
             ("attn.c_proj.weight", (d, d)), ("attn.c_proj.bias", (d,)),
             ("ln_2.weight", (d,)), ("ln_2.bias", (d,)),
             ("mlp.c_fc.weight", (4 * d, d)), ("mlp.c_fc.bias", (4 * d,)),
             ("mlp.c_proj.weight", (d, 4 * d)), ("mlp.c_proj.bias", (d,))]
    return [(n, s) for n, s in names if bias or not n.endswith(".bias")]


def stage_param_specs(cfg: GPT2Config, layers: Sequence[int], first: bool, last: bool
                      ) -> List[Tuple[str, str, Tuple[int, ...]]]:
    """(local state-dict key, global name, shape) of a stage, in the reference's
    parameter order.  Local keys number the blocks from 0 within the stage, as
    the reference's ``ShardedGPT2.state_dict()`` does (src/model.py:187)."""
    d = cfg.n_embd
    specs: List[Tuple[str, str, Tuple[int, ...]]] = []
    if first:
        specs.append(("transformer.wte.weight", "transformer.wte.weight", (cfg.vocab_size, d)))
        specs.append(("transformer.wpe.weight", "transformer.wpe.weight", (cfg.block_size, d)))
    for li, gi in enumerate(layers):
        for n, shp in block_param_shapes(d, cfg.bias):
            specs.append((f"transformer.h.{li}.{n}", f"transformer.h.{gi}.{n}", shp))
    if last:
        specs.append(("transformer.ln_f.weight", "transformer.ln_f.weight", (d,)))
        if cfg.bias:
            specs.append(("transformer.ln_f.bias", "transformer.ln_f.bias", (d,)))
        tied = cfg.parameter_sharing and first
        if not tied:
            # untied, or tied but on another rank: the head has its own tensor.
            # With tying requested and S > 1 both copies start equal (same
            # global name) and then drift, as in the reference.
            gname = "transformer.wte.weight" if cfg.parameter_sharing else "lm_head.weight"
            specs.append(("lm_head.weight", gname, (cfg.vocab_size, d)))
    return specs


class _LayerNorm(nn.Module):
    def __init__(self, d: int, bias: bool):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.bias = nn.Parameter(torch.zeros(d)) if bias else None

    def forward(self, x):
        return F.layer_norm(x, self.weight.shape, self.weight, self.bias, 1e-5)


class _Attention(nn.Module):
    """Dropout sits where the reference has it: on the attention probabilities and on the projected
    output (src/model.py:48-49,67,77)."""

    def __init__(self, d: int, n_head: int, bias: bool, dropout: float = 0.0):
        super().__init__()
        self.n_head = n_head
        self.dropout = dropout
        self.c_attn = nn.Linear(d, 3 * d, bias=bias)
        self.c_proj = nn.Linear(d, d, bias=bias)

    def forward(self, x):
        B, T, C = x.shape
        hs = C // self.n_head
        q, k, v = (t.view(B, T, self.n_head, hs).transpose(1, 2) for t in self.c_attn(x).split(C, dim=2))
        p = self.dropout if self.training else 0.0
        y = F.scaled_dot_product_attention(q, k, v, dropout_p=p, is_causal=True)
        return F.dropout(self.c_proj(y.transpose(1, 2).reshape(B, T, C)), p, self.training)


class _MLP(nn.Module):
    def __init__(self, d: int, bias: bool, dropout: float = 0.0):
        super().__init__()
        self.dropout = dropout
        self.c_fc = nn.Linear(d, 4 * d, bias=bias)
        self.c_proj = nn.Linear(4 * d, d, bias=bias)

    def forward(self, x):
        return F.dropout(self.c_proj(F.gelu(self.c_fc(x))), self.dropout, self.training)    # src/model.py:86,89


class _Block(nn.Module):
    def __init__(self, d: int, n_head: int, bias: bool, dropout: float = 0.0):
        super().__init__()
        self.ln_1 = _LayerNorm(d, bias)
        self.attn = _Attention(d, n_head, bias, dropout)
        self.ln_2 = _LayerNorm(d, bias)
        self.mlp = _MLP(d, bias, dropout)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.mlp(self.ln_2(x))


class _Transformer(nn.Module):
    pass


class TorchStage(nn.Module):
    """One pipeline stage on library ops with autograd (reference: ShardedGPT2,
    src/model.py:177-209).  With ``num_stages == 1`` it is the whole model."""

    def __init__(self, cfg: GPT2Config, stage: int = 0, num_stages: int = 1, seed: int = 42,
                 layer_split: str = "even"):
        super().__init__()
        self.config = cfg
        self.stage, self.num_stages = stage, num_stages
        self.is_first, self.is_last = stage == 0, stage == num_stages - 1
        self.layers = split_layers(cfg.n_layer, num_stages, layer_split, cfg.n_embd, cfg.vocab_size)[stage]
        d = cfg.n_embd
        t = _Transformer()
        if self.is_first:
            t.wte = nn.Embedding(cfg.vocab_size, d)
            t.wpe = nn.Embedding(cfg.block_size, d)
        t.h = nn.ModuleList([_Block(d, cfg.n_head, cfg.bias, cfg.dropout) for _ in self.layers])
        if self.is_last:
            t.ln_f = _LayerNorm(d, cfg.bias)
        self.transformer = t
        if self.is_last:
            self.lm_head = nn.Linear(d, cfg.vocab_size, bias=False)
            if cfg.parameter_sharing and self.is_first:
                self.lm_head.weight = t.wte.weight
        self.specs = stage_param_specs(cfg, self.layers, self.is_first, self.is_last)
        sd = dict(self.named_parameters())
        with torch.no_grad():
            for key, gname, shape in self.specs:
                sd[key].copy_(init_tensor(gname, shape, seed, cfg.n_layer))

    # -- pieces (reference: encode_tokens / forward_layers / forward_logits) --
    def encode_tokens(self, input_ids: torch.Tensor) -> torch.Tensor:
        pos = torch.arange(input_ids.size(1), device=input_ids.device)
        x = self.transformer.wte(input_ids) + self.transformer.wpe(pos)
        return F.dropout(x, self.config.dropout, self.training)                               # src/model.py:114,139

    def forward(self, input_ids: Optional[torch.Tensor] = None,
                hidden_states: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.encode_tokens(input_ids) if self.is_first else hidden_states
        for blk in self.transformer.h:
            x = blk(x)
        if self.is_last:
            x = self.lm_head(self.transformer.ln_f(x))
        return x

    def num_parameters(self, exclude_positional: bool = True) -> int:
        n = sum(p.numel() for p in self.parameters())
        if exclude_positional and self.is_first:
            n -= self.transformer.wpe.weight.numel()
        return n

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = None, eos_token_id: Optional[int] = None,
                 generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Single-process sampler (reference: GPT2.generate, src/model.py:160-175)."""
        assert self.num_stages == 1
        for _ in range(max_new_tokens):
            ctx = input_ids[:, -self.config.block_size:]
            logits = self(input_ids=ctx)[:, -1, :].float()
            nxt = sample_next(logits, temperature, top_k, generator)
            input_ids = torch.cat([input_ids, nxt], dim=1)
            if eos_token_id is not None and bool((nxt == eos_token_id).all()):
                break
        return input_ids


def sample_next(logits: torch.Tensor, temperature: float = 1.0, top_k: Optional[int] = None,
                generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Temperature / top-k sampling of one token per row.  The reference's
    distributed sampler ignores both knobs (src/train.py:64-65); here they apply."""
    if temperature <= 0:
        return logits.argmax(dim=-1, keepdim=True)
    logits = logits / temperature
    if top_k is not None and top_k > 0:
        kth = torch.topk(logits, min(top_k, logits.size(-1))).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probs = F.softmax(logits, dim=-1)
    return torch.multinomial(probs, num_samples=1, generator=generator)


def num_parameters(cfg: GPT2Config, exclude_positional: bool = True) -> int:
    d = cfg.n_embd
    n = cfg.n_layer * sum(math.prod(s) for _, s in block_param_shapes(d, cfg.bias))
    n += cfg.vocab_size * d * (1 if cfg.parameter_sharing else 2)
    n += d * (2 if cfg.bias else 1)
    if not exclude_positional:
        n += cfg.block_size * d
    return n
