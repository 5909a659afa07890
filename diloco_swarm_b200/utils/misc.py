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
