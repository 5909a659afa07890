"""Python entry points of the sm_100a kernels (csrc/*.cu).

Each function takes torch CUDA tensors, checks shapes/dtypes on the host and
launches on the current stream.  None of them synchronises or allocates beyond
its outputs.  The docstrings name the reference call site each one replaces.
"""
from __future__ import annotations

import functools
import math
import os
from typing import Optional, Tuple

import torch

from ._lib import Status, check, cuda_lib, ptr, stream_ptr

BF16, F32 = torch.bfloat16, torch.float32

EPI_STORE, EPI_GELU, EPI_RESID, EPI_MUL, EPI_ATOMIC_F32, EPI_STORE_F32 = range(6)

_NUM_SMS = 148


_USE_PAIR = os.environ.get("DSWARM_GEMM_PAIR", "1") != "0"
# Cap on the CTAs of every GEMM launch (0 = all SMs): leaves SMs to kernels that sit on the device while
# the GEMMs run, such as a pipeline transfer waiting for its peer.
_MAX_CTAS = int(os.environ.get("DSWARM_GEMM_MAX_CTAS", "0"))


def _efficiency(M: int, N: int, splits: int, bm: int, bn: int, units: int) -> float:
    """Fraction of the machine busy with real tiles when the grid runs in whole waves."""
    tiles = math.ceil(M / bm) * math.ceil(N / bn) * splits
    waves = math.ceil(tiles / units)
    useful = (M * N) / (math.ceil(M / bm) * bm * math.ceil(N / bn) * bn)
    return useful * tiles / (waves * units)


@functools.lru_cache(maxsize=None)          # a training run asks for a handful of shapes, thousands of times a step
def _pick_bn(M: int, N: int, splits: int = 1) -> int:
    """Tile choice: 512 = 256x256 on a CTA pair (least operand traffic per FLOP),
    256 = 128x256 on one CTA, 128 = 128x128.  A wider tile wins unless a
    narrower one fills the SMs clearly better."""
    if N <= 128:
        return 128
    e128 = _efficiency(M, N, splits, 128, 128, _NUM_SMS)
    e256 = _efficiency(M, N, splits, 128, 256, _NUM_SMS)
    best = 256 if e256 >= e128 * 0.93 else 128
    if _USE_PAIR and M >= 256:
        epair = _efficiency(M, N, splits, 256, 256, _NUM_SMS // 2)
        if epair >= max(e128 * 0.8, e256 * 0.9):
            best = 512
    return best


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = True, mode: int = EPI_STORE,
         out: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
         resid: Optional[torch.Tensor] = None, aux_out: Optional[torch.Tensor] = None,
         aux_in: Optional[torch.Tensor] = None, split_k: int = 1, bn: int = 0, max_ctas: int = 0,
         status: Optional[Status] = None) -> torch.Tensor:
    """D = op(A) @ op(B) on tcgen05 (replaces nn.Linear's GEMMs and their
    backward, src/model.py:44-45,83-84,118).

    ``a`` is [M,K] (or [K,M] with ``a_t``), ``b`` is [N,K] with ``b_t`` (the
    nn.Linear weight layout) or [K,N] without.  bf16 in, fp32 accumulate.
    Epilogues: EPI_GELU returns gelu(acc + bias) (exact erf form) and, when
    ``aux_out`` is given, also stores gelu'(acc + bias) there; EPI_MUL returns
    acc * ``aux_in``, which with that saved derivative is the GELU backward.
    """
    assert a.dtype == BF16 and b.dtype == BF16 and a.dim() == 2 and b.dim() == 2
    assert a.stride(1) == 1 and b.stride(1) == 1
    if a_t:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_t:
        N, Kb = b.shape
    else:
        Kb, N = b.shape
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    f32_out = mode in (EPI_ATOMIC_F32, EPI_STORE_F32)
    if out is None:
        assert mode != EPI_ATOMIC_F32
        out = torch.empty(M, N, dtype=F32 if f32_out else BF16, device=a.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype == (F32 if f32_out else BF16)
    if mode == EPI_GELU and aux_out is not None:      # aux_out receives gelu'(a @ b + bias) for the backward
        assert aux_out.shape == (M, N) and aux_out.dtype == BF16
    if mode == EPI_MUL:
        assert aux_in is not None and aux_in.shape == (M, N) and aux_in.dtype == BF16
    if mode == EPI_RESID:
        assert resid is not None and resid.shape == (M, N) and resid.dtype == BF16
    if bias is not None:
        assert bias.dtype == F32 and bias.numel() == N
    kb_total = math.ceil(K / 64)
    split_k = max(1, min(split_k, kb_total))
    if split_k > 1:
        assert mode == EPI_ATOMIC_F32, "split-K needs the accumulating epilogue"
        per = math.ceil(kb_total / split_k)
        split_k = math.ceil(kb_total / per)       # no empty split
    if bn == 0:
        bn = _pick_bn(M, N, split_k)
    if max_ctas == 0:
        max_ctas = _MAX_CTAS
    aux = aux_out if aux_out is not None else aux_in
    rc = cuda_lib().dsw_gemm_bf16(
        a.data_ptr(), a.stride(0), 1 if a_t else 0, b.data_ptr(), b.stride(0), 0 if b_t else 1, M, N, K, mode,
        split_k, out.data_ptr(), out.stride(0), ptr(bias), ptr(resid), resid.stride(0) if resid is not None else 0,
        ptr(aux_out), ptr(aux_in), aux.stride(0) if aux is not None else 0, bn, max_ctas,
        status.ptr if status is not None else None, stream_ptr())
    check(rc, "dsw_gemm_bf16")
    return out


_DETERMINISTIC = False


def set_deterministic(on: bool) -> None:
    """Fixed order of floating-point additions in the gradient kernels that
    otherwise use atomics: the token-embedding scatter goes through a stable
    sort with one writer per row, and weight gradients are not split along K
    (each output tile then has one writer per launch, and launches are ordered
    by the stream).  Slower; meant for debugging and regression runs."""
    global _DETERMINISTIC
    _DETERMINISTIC = bool(on)


def wgrad_split(M: int, N: int, K: int) -> int:
    """Split-K factor for dW[M,N] = dy^T x with K = tokens: the weight gradients
    of a block have few output tiles, so K is split until the SMs are full."""
    return 1 if _DETERMINISTIC else _wgrad_split(M, N, K)


@functools.lru_cache(maxsize=None)
def _wgrad_split(M: int, N: int, K: int) -> int:
    bm, units = (256, _NUM_SMS // 2) if (_USE_PAIR and M >= 256) else (128, _NUM_SMS)
    tiles = math.ceil(M / bm) * math.ceil(N / 256)
    if tiles >= 4 * units:
        return 1
    kb = math.ceil(K / 64)
    best, best_eff = 1, 0.0
    for s in range(1, 17):
        if kb // s < 4:
            break
        waves = math.ceil(tiles * s / units)
        eff = tiles * s / (waves * units) - 0.01 * (s - 1)      # small price per extra split (atomics)
        if eff > best_eff + 1e-9:
            best, best_eff = s, eff
    return best


def layernorm_fwd(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float = 1e-5
                  ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """y, mean, rstd of F.layer_norm (src/model.py:31); bf16 in/out, fp32 statistics."""
    M, d = x.shape
    assert x.dtype == BF16 and x.is_contiguous() and gamma.dtype == F32
    y = torch.empty_like(x)
    mean = torch.empty(M, dtype=F32, device=x.device)
    rstd = torch.empty(M, dtype=F32, device=x.device)
    check(cuda_lib().dsw_layernorm_fwd(x.data_ptr(), gamma.data_ptr(), ptr(beta), y.data_ptr(), mean.data_ptr(),
                                       rstd.data_ptr(), M, d, eps, stream_ptr()), "dsw_layernorm_fwd")
    return y, mean, rstd


_ln_scratch = {}


def layernorm_bwd(dy: torch.Tensor, x: torch.Tensor, gamma: torch.Tensor, mean: torch.Tensor, rstd: torch.Tensor,
                  dgamma: torch.Tensor, dbeta: Optional[torch.Tensor], dres: Optional[torch.Tensor] = None,
                  dres_sum: Optional[torch.Tensor] = None) -> torch.Tensor:
    """dx of LayerNorm plus ``dres`` (the gradient arriving on the residual
    branch); accumulates dgamma / dbeta (fp32) in place and, when ``dres_sum``
    is given, adds the column sum of ``dres`` to it (the bias gradient of the
    projection whose output was added to the residual stream)."""
    M, d = x.shape
    assert dy.shape == x.shape and dy.is_contiguous() and x.is_contiguous()
    dx = torch.empty_like(x)
    lib = cuda_lib()
    nblk = lib.dsw_layernorm_bwd_blocks(M)
    key = (x.device.index, nblk, d)
    scratch = _ln_scratch.get(key)
    if scratch is None:
        # per-block partial column sums; reused by every call of this shape (same stream order)
        scratch = torch.empty(nblk * 3 * d, dtype=F32, device=x.device)
        _ln_scratch[key] = scratch
    check(lib.dsw_layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                ptr(dres), dx.data_ptr(), dgamma.data_ptr(), ptr(dbeta), ptr(dres_sum),
                                scratch.data_ptr(), M, d, stream_ptr()), "dsw_layernorm_bwd")
    return dx


def colsum_accum(x: torch.Tensor, out: torch.Tensor) -> None:
    """out[n] += sum_m x[m,n] (bias gradients)."""
    M, N = x.shape
    assert x.dtype == BF16 and x.stride(1) == 1 and out.dtype == F32 and out.numel() == N
    check(cuda_lib().dsw_colsum_accum(x.data_ptr(), x.stride(0), out.data_ptr(), M, N, stream_ptr()), "dsw_colsum_accum")


def embedding_fwd(ids: torch.Tensor, wte: torch.Tensor, wpe: torch.Tensor, status: Optional[Status] = None
                  ) -> torch.Tensor:
    """bf16(wte[ids] + wpe[pos]) from the fp32 tables (src/model.py:134-139)."""
    B, T = ids.shape
    V, d = wte.shape
    assert ids.dtype == torch.long and ids.is_contiguous() and wte.dtype == F32 and wpe.dtype == F32
    y = torch.empty(B * T, d, dtype=BF16, device=ids.device)
    check(cuda_lib().dsw_embedding_fwd(ids.data_ptr(), wte.data_ptr(), wpe.data_ptr(), y.data_ptr(), B, T, d, V,
                                       status.ptr if status else None, stream_ptr()), "dsw_embedding_fwd")
    return y


def embedding_bwd(ids: torch.Tensor, dx: torch.Tensor, dwte: torch.Tensor, dwpe: torch.Tensor) -> None:
    B, T = ids.shape
    V, d = dwte.shape
    assert dx.dtype == BF16 and dx.is_contiguous() and dwte.dtype == F32
    if _DETERMINISTIC:
        srt, perm = torch.sort(ids.reshape(-1), stable=True)
        check(cuda_lib().dsw_embedding_bwd_sorted(srt.data_ptr(), perm.data_ptr(), dx.data_ptr(), dwte.data_ptr(),
                                                  dwpe.data_ptr(), B, T, d, V, stream_ptr()), "dsw_embedding_bwd_sorted")
        return
    check(cuda_lib().dsw_embedding_bwd(ids.data_ptr(), dx.data_ptr(), dwte.data_ptr(), dwpe.data_ptr(), B, T, d, V,
                                       stream_ptr()), "dsw_embedding_bwd")


def count_kept_rows(mask: Optional[torch.Tensor], M: int, count_buf: torch.Tensor) -> None:
    """``count_buf[0]`` = number of rows the loss is averaged over (mask != 0, or all M without a mask)."""
    if mask is not None:
        assert mask.dtype == torch.long and mask.numel() == M
        count_buf.zero_()
        check(cuda_lib().dsw_mask_count(mask.data_ptr(), M, count_buf.data_ptr(), stream_ptr()), "dsw_mask_count")
    else:
        count_buf.fill_(float(M))


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor, mask: Optional[torch.Tensor], scale: float,
                  loss_acc: torch.Tensor, count_buf: torch.Tensor, write_grad: bool = True,
                  status: Optional[Status] = None, count_ready: bool = False) -> None:
    """Masked mean cross-entropy times ``scale`` added to ``loss_acc``; with
    ``write_grad`` the logits are overwritten by their gradient (reference:
    filter_logits_targets + CrossEntropyLoss, src/utils.py:184-193).  With ``count_ready`` the
    divisor already stands in ``count_buf`` (``count_kept_rows`` over all rows of the microbatch)
    and ``logits`` may be a slice of its rows."""
    M, V = logits.shape
    assert logits.dtype == BF16 and logits.stride(1) == 1
    assert targets.dtype == torch.long and targets.numel() == M
    lib = cuda_lib()
    if mask is not None:
        assert mask.dtype == torch.long and mask.numel() == M
    if not count_ready:
        count_kept_rows(mask, M, count_buf)
    cnt = count_buf.data_ptr()
    check(lib.dsw_cross_entropy(logits.data_ptr(), logits.stride(0), targets.data_ptr(), ptr(mask), cnt, scale,
                                loss_acc.data_ptr(), M, V, 1 if write_grad else 0,
                                status.ptr if status else None, stream_ptr()), "dsw_cross_entropy")


def cast_to_bf16(src: torch.Tensor, dst: torch.Tensor) -> None:
    assert src.dtype == F32 and dst.dtype == BF16 and src.numel() == dst.numel()
    check(cuda_lib().dsw_cast_f32_bf16(src.data_ptr(), dst.data_ptr(), src.numel(), stream_ptr()), "dsw_cast_f32_bf16")


def grad_norm_and_clip(grad: torch.Tensor, stats: torch.Tensor, max_norm: float) -> None:
    """stats = [sum of squares, norm, clip coefficient] on the device
    (clip_grad_norm_ over the stage shard, src/train.py:255)."""
    stats.zero_()
    lib = cuda_lib()
    check(lib.dsw_sumsq(grad.data_ptr(), grad.numel(), stats.data_ptr(), stream_ptr()), "dsw_sumsq")
    check(lib.dsw_clip_coef(stats.data_ptr(), max_norm, stream_ptr()), "dsw_clip_coef")


def adamw_step(p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, p16: Optional[torch.Tensor],
               lr: float, betas, eps: float, wd: float, step: int, coef: Optional[torch.Tensor],
               zero_grad: bool = True) -> None:
    """Fused clip-scale + AdamW + bf16 weight refresh + gradient clear (src/utils.py:61)."""
    check(cuda_lib().dsw_adamw(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), ptr(p16), p.numel(), lr,
                               betas[0], betas[1], eps, wd, step, coef[2:].data_ptr() if coef is not None else None,
                               1 if zero_grad else 0, stream_ptr()), "dsw_adamw")


def sgd_step(p, g, buf, p16, lr: float, mu: float, nesterov: bool, coef, zero_grad: bool = True) -> None:
    check(cuda_lib().dsw_sgd(p.data_ptr(), g.data_ptr(), ptr(buf), ptr(p16), p.numel(), lr, mu, 1 if nesterov else 0,
                             coef[2:].data_ptr() if coef is not None else None, 1 if zero_grad else 0, stream_ptr()),
          "dsw_sgd")
