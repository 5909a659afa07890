"""Small helpers (reference: src/utils.py:24-46,128-182)."""
from __future__ import annotations

import random
from typing import Optional

import numpy as np
import torch


def seed_everything(seed: int) -> None:
    """Seeds torch, CUDA, numpy and also Python's ``random`` (the reference
    leaves the latter unseeded although it drives its routing)."""
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def get_device(device: Optional[str] = None, local_rank: int = 0) -> torch.device:
    if device:
        d = torch.device(device)
        if d.type == "cuda" and d.index is None:
            d = torch.device("cuda", local_rank)
        return d
    if torch.cuda.is_available():
        return torch.device("cuda", local_rank)
    return torch.device("cpu")


def get_dtype(name: str) -> torch.dtype:
    return getattr(torch, name)


def format_int(num: float, prec: int = 2) -> str:
    for lim, suf in ((1e3, ""), (1e6, "K"), (1e9, "M")):
        if num < lim:
            return str(num) if suf == "" else f"{num / (lim / 1e3):.{prec}f}{suf}"
    return f"{num / 1e9:.{prec}f}B"


def format_float(num: float, prec: int = 2) -> str:
    return f"{num:.{prec}f}"


def get_hf_cache_dir() -> str:
    """Where Hugging Face downloads go (reference: src/utils.py:31-34 reads PERSISTENT_DIR from .env)."""
    import os
    base = os.environ.get("PERSISTENT_DIR") or os.environ.get("HF_HOME") or os.path.expanduser("~/.cache/huggingface")
    return os.path.join(base, "huggingface") if os.environ.get("PERSISTENT_DIR") else base


def nullcontext():
    import contextlib
    return contextlib.nullcontext()


def get_train_pbar_description(metrics, prefix: str) -> str:
    """One-line progress text from a Metrics object (same fields as the reference's progress bar,
    src/utils.py:128-137)."""
    m, n = metrics.compute(), metrics.name
    g = lambda k: m.get(f"{n}/{k}/current") or 0.0
    return (f"{prefix} Step: {int(g('step'))} - Time: {g('time'):.1f}s - Loss: {g('loss'):.4f} - "
            f"Norm: {g('norm'):.4f} - Perplexity: {g('perplexity'):.1f} - Throughput: {g('throughput'):.1f}")


def get_eval_pbar_description(metrics, prefix: str) -> str:
    m, n = metrics.compute(), metrics.name
    return (f"{prefix} Avg. Loss: {m.get(f'{n}/loss/average') or 0.0:.4f}, "
            f"Avg. Perplexity: {m.get(f'{n}/perplexity/average') or 0.0:.1f}")
