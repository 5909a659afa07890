"""tcgen05 flash attention (forward and backward) against fp32 PyTorch attention."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(qkv, B, T, nh):
    d = qkv.shape[1] // 3
    hs = d // nh
    q, k, v = (qkv[:, i * d:(i + 1) * d].float().view(B, T, nh, hs).transpose(1, 2) for i in range(3))
    att = (q @ k.transpose(-1, -2)) / math.sqrt(hs)
    mask = torch.ones(T, T, device=qkv.device, dtype=torch.bool).tril()
    att = att.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(att, dim=-1)
    o = torch.softmax(att, dim=-1) @ v
    return o.transpose(1, 2).reshape(B * T, d), lse


# The last three give every persistent CTA several work items (more items than SMs), which is where the
# double-buffered K / V, the hand-over between items and the staged dK / dV stores are exercised.
SHAPES = [(1, 128, 1, 64), (2, 256, 3, 64), (1, 1024, 2, 64), (1, 128, 1, 32), (2, 384, 4, 32), (1, 1024, 3, 32),
          (4, 1024, 12, 64), (16, 256, 12, 64), (6, 512, 12, 32)]


@pytest.mark.parametrize("B,T,nh,hs", SHAPES)
def test_attention_forward(B, T, nh, hs, monkeypatch):
    monkeypatch.setenv("DSWARM_ATTENTION", "native")
    from diloco_swarm_b200.ops.attention import attention_fwd
    torch.manual_seed(0)
    qkv = (torch.randn(B * T, 3 * nh * hs, device="cuda")).to(torch.bfloat16)
    out, ctx = attention_fwd(qkv, B, T, nh)
    torch.cuda.synchronize()
    assert ctx.native
    ref, lse = _ref(qkv, B, T, nh)
    assert (out.float() - ref).abs().max() < 2e-2 * ref.abs().max() + 2e-3
    assert (ctx.lse.view(B, nh, T) - lse).abs().max() < 2e-2


@pytest.mark.parametrize("B,T,nh,hs", SHAPES)
def test_attention_backward(B, T, nh, hs, monkeypatch):
    monkeypatch.setenv("DSWARM_ATTENTION", "native")
    from diloco_swarm_b200.ops.attention import attention_bwd, attention_fwd
    torch.manual_seed(1)
    qkv = (torch.randn(B * T, 3 * nh * hs, device="cuda")).to(torch.bfloat16)
    dout = (torch.randn(B * T, nh * hs, device="cuda")).to(torch.bfloat16)
    out, ctx = attention_fwd(qkv, B, T, nh)
    dqkv = attention_bwd(dout, ctx)
    torch.cuda.synchronize()
    x = qkv.float().requires_grad_(True)
    ref, _ = _ref(x, B, T, nh)
    ref.backward(dout.float())
    d = nh * hs
    for name, sl in (("dq", slice(0, d)), ("dk", slice(d, 2 * d)), ("dv", slice(2 * d, 3 * d))):
        got, want = dqkv[:, sl].float(), x.grad[:, sl]
        err = (got - want).abs().max().item()
        assert err < 3e-2 * want.abs().max().item() + 3e-3, f"{name}: {err} vs scale {want.abs().max().item()}"
