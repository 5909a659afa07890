"""Causal self-attention over a packed QKV activation.

``qkv`` is the [B*T, 3*d] output of the fused QKV projection; heads are
interleaved as in the reference (src/model.py:60-63): columns [0,d) are Q,
[d,2d) K, [2d,3d) V, head h at columns h*hs..(h+1)*hs of each.  Scale is
1/sqrt(hs), mask is purely causal (the attention mask only filters the loss,
src/model.py:67).

Two implementations behind one interface:
  * the sm_100a flash-attention kernels (csrc/attention.cu), used when the
    library exports them and the head size is supported;
  * PyTorch SDPA (a library kernel) otherwise.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from ._lib import Status, check, cuda_lib, stream_ptr

BF16 = torch.bfloat16


def _native_available(hs: int, T: int) -> bool:
    """The sm_100a kernels cover head size 64 (GPT-2 small to xl) and 32 (the
    4-head, 128-wide test model) at sequence lengths that are multiples of 128;
    other shapes use the library kernel."""
    if os.environ.get("DSWARM_ATTENTION", "native") == "sdpa":
        return False
    lib = cuda_lib()
    return hs in (32, 64) and T % 128 == 0 and hasattr(lib, "dsw_attention_fwd") and hasattr(lib, "dsw_attention_bwd")


class AttnCtx:
    __slots__ = ("qkv", "out", "lse", "B", "T", "nh", "native", "q", "k", "v", "o", "status")


def attention_fwd(qkv: torch.Tensor, B: int, T: int, nh: int, need_ctx: bool = True,
                  status: Optional[Status] = None) -> Tuple[torch.Tensor, Optional[AttnCtx]]:
    """``status``: the engine's status word; an mbarrier wait that runs out inside the kernel (forward
    or the backward that uses the returned context) is reported there instead of passing silently."""
    M, d3 = qkv.shape
    d = d3 // 3
    hs = d // nh
    ctx = AttnCtx() if need_ctx else None
    if _native_available(hs, T):
        out = torch.empty(M, d, dtype=BF16, device=qkv.device)
        lse = torch.empty(B * nh * T, dtype=torch.float32, device=qkv.device)
        check(cuda_lib().dsw_attention_fwd(qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, nh, hs,
                                           1.0 / math.sqrt(hs), status.ptr if status is not None else None,
                                           stream_ptr()), "dsw_attention_fwd")
        if ctx is not None:
            ctx.native, ctx.qkv, ctx.out, ctx.lse, ctx.B, ctx.T, ctx.nh = True, qkv, out, lse, B, T, nh
            ctx.status = status
        return out, ctx
    q, k, v = (qkv[:, i * d:(i + 1) * d].view(B, T, nh, hs).transpose(1, 2) for i in range(3))
    if ctx is not None:
        q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
        with torch.enable_grad():
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
        ctx.native, ctx.q, ctx.k, ctx.v, ctx.o, ctx.status = False, q, k, v, o, None
    else:
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    return o.detach().transpose(1, 2).reshape(M, d), ctx


def attention_bwd(dout: torch.Tensor, ctx: AttnCtx) -> torch.Tensor:
    """Gradient w.r.t. the packed qkv, [B*T, 3*d]."""
    if ctx.native:
        B, T, nh = ctx.B, ctx.T, ctx.nh
        d = ctx.out.shape[1]
        hs = d // nh
        dqkv = torch.empty_like(ctx.qkv)
        dq_acc = torch.empty(B * T, d, dtype=torch.float32, device=dout.device)     # fp32 accumulator of dQ
        dvec = torch.empty(B * nh * T, dtype=torch.float32, device=dout.device)     # rowsum(dO * O)
        dout = dout.contiguous()
        check(cuda_lib().dsw_attention_bwd(ctx.qkv.data_ptr(), ctx.out.data_ptr(), dout.data_ptr(), ctx.lse.data_ptr(),
                                           dqkv.data_ptr(), dq_acc.data_ptr(), dvec.data_ptr(), B, T, nh, hs,
                                           1.0 / math.sqrt(hs), ctx.status.ptr if ctx.status is not None else None,
                                           stream_ptr()), "dsw_attention_bwd")
        return dqkv
    q, k, v, o = ctx.q, ctx.k, ctx.v, ctx.o
    B, nh, T, hs = q.shape
    do = dout.view(B, T, nh, hs).transpose(1, 2)
    dq, dk, dv = torch.autograd.grad(o, (q, k, v), do)
    return torch.cat([t.transpose(1, 2).reshape(B * T, nh * hs) for t in (dq, dk, dv)], dim=1)
