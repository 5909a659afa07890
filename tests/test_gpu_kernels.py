"""Memory-bound and optimiser kernels against fp32 PyTorch references."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _bf(x):
    return x.to(torch.bfloat16)


@pytest.mark.parametrize("M,d", [(64, 128), (1000, 768), (257, 1024), (96, 1600)])
def test_layernorm_fwd_bwd(M, d):
    from diloco_swarm_b200.ops import kernels as K
    torch.manual_seed(0)
    x = _bf(torch.randn(M, d, device=DEV) * 2 + 0.5)
    g = torch.randn(d, device=DEV)
    b = torch.randn(d, device=DEV)
    y, mean, rstd = K.layernorm_fwd(x, g, b)
    xr = x.float().requires_grad_(True)
    gr, br = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    yr = F.layer_norm(xr, (d,), gr, br, 1e-5)
    assert (y.float() - yr).abs().max() < 3e-2 * yr.abs().max()
    assert torch.allclose(mean, xr.mean(1), atol=1e-4)
    dy = _bf(torch.randn(M, d, device=DEV))
    dres = _bf(torch.randn(M, d, device=DEV))
    yr.backward(dy.float())
    dg, db = torch.zeros(d, device=DEV), torch.zeros(d, device=DEV)
    rs = torch.ones(d, device=DEV)
    dx = K.layernorm_bwd(dy, x, g, mean, rstd, dg, db, dres=dres, dres_sum=rs)
    ref_rs = 1 + dres.float().sum(0)
    assert (rs - ref_rs).abs().max() < 1e-2 * ref_rs.abs().max() + 1e-2
    ref_dx = xr.grad + dres.float()
    assert (dx.float() - ref_dx).abs().max() < 3e-2 * ref_dx.abs().max()
    assert (dg - gr.grad).abs().max() < 2e-2 * gr.grad.abs().max() + 1e-2
    assert (db - br.grad).abs().max() < 2e-2 * br.grad.abs().max() + 1e-2


def test_colsum():
    from diloco_swarm_b200.ops import kernels as K
    x = _bf(torch.randn(5000, 776, device=DEV))
    out = torch.ones(776, device=DEV)
    K.colsum_accum(x, out)
    ref = 1 + x.float().sum(0)
    assert (out - ref).abs().max() < 1e-2 * ref.abs().max()


def test_embedding():
    from diloco_swarm_b200.ops import kernels as K
    B, T, d, V = 3, 40, 128, 1000
    ids = torch.randint(0, V, (B, T), device=DEV)
    wte, wpe = torch.randn(V, d, device=DEV), torch.randn(64, d, device=DEV)
    y = K.embedding_fwd(ids, wte, wpe)
    ref = wte[ids] + wpe[:T]
    assert (y.float().view(B, T, d) - ref).abs().max() < 2e-2 * ref.abs().max()
    dx = _bf(torch.randn(B * T, d, device=DEV))
    dwte, dwpe = torch.zeros_like(wte), torch.zeros_like(wpe)
    K.embedding_bwd(ids, dx, dwte, dwpe)
    rte = torch.zeros_like(wte).index_add_(0, ids.view(-1), dx.float())
    rpe = torch.zeros_like(wpe)
    rpe[:T] = dx.float().view(B, T, d).sum(0)
    assert torch.allclose(dwte, rte, atol=1e-3) and torch.allclose(dwpe, rpe, atol=1e-3)


@pytest.mark.parametrize("M,V", [(64, 1000), (300, 50304)])
def test_cross_entropy(M, V):
    from diloco_swarm_b200.ops import kernels as K
    torch.manual_seed(1)
    logits = _bf(torch.randn(M, V, device=DEV) * 3)
    tg = torch.randint(0, V, (M,), device=DEV)
    mask = (torch.rand(M, device=DEV) > 0.3).long()
    scale = 0.25
    lr = logits.float().requires_grad_(True)
    ref = F.cross_entropy(lr[mask.bool()], tg[mask.bool()]) * scale
    ref.backward()
    loss = torch.zeros((), device=DEV)
    cnt = torch.zeros(1, device=DEV)
    work = logits.clone()
    K.cross_entropy(work, tg, mask, scale, loss, cnt, write_grad=True)
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item()) + 1e-4
    assert (work.float() - lr.grad).abs().max() < 2e-2 * lr.grad.abs().max() + 1e-7
    loss2 = torch.zeros((), device=DEV)
    work2 = logits.clone()
    K.cross_entropy(work2, tg, mask, scale, loss2, cnt, write_grad=False)
    # the rows' terms reach the loss through fp32 atomics, so two launches add them in different orders: the
    # two sums of some 200 terms around 0.02 agree to a few units in the last place of 3.9, not bit for bit
    assert torch.equal(work2, logits) and abs(loss2.item() - loss.item()) < 1e-5


def test_adamw_and_clip():
    from diloco_swarm_b200.ops import kernels as K
    n = 1_000_003 // 8 * 8
    torch.manual_seed(2)
    p = torch.randn(n, device=DEV)
    g = torch.randn(n, device=DEV) * 0.01
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    p16 = torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    stats = torch.zeros(4, device=DEV)
    for step in range(1, 4):
        gi = g * step
        ref_p.grad = gi.clone()
        norm = torch.nn.utils.clip_grad_norm_([ref_p], 1.0)
        opt.step()
        gw = gi.clone()
        K.grad_norm_and_clip(gw, stats, 1.0)
        K.adamw_step(p, gw, m, v, p16, 1e-3, (0.9, 0.95), 1e-8, 0.1, step, stats, zero_grad=True)
        assert abs(stats[1].item() - norm.item()) < 1e-3 * norm.item()
        assert gw.abs().max().item() == 0.0
    assert torch.allclose(p, ref_p.data, atol=2e-6, rtol=1e-5)
    assert torch.allclose(p16.float(), p, atol=1e-2, rtol=1e-2)


def test_sgd_nesterov():
    from diloco_swarm_b200.ops import kernels as K
    n = 4096
    p = torch.randn(n, device=DEV)
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.SGD([ref_p], lr=0.1, momentum=0.9, nesterov=True)
    buf = torch.zeros(n, device=DEV)
    for step in range(3):
        g = torch.randn(n, device=DEV)
        ref_p.grad = g.clone()
        opt.step()
        K.sgd_step(p, g.clone(), buf, None, 0.1, 0.9, True, None, zero_grad=False)
    assert torch.allclose(p, ref_p.data, atol=1e-5)


def test_embedding_bwd_deterministic_mode():
    """The sorted scatter (one writer per row, rows added in their original order) gives the same
    gradient as a plain fp32 index_add, twice in a row bit for bit."""
    from diloco_swarm_b200.ops import kernels as K
    torch.manual_seed(5)
    B, T, d, V = 4, 256, 128, 512
    ids = torch.randint(0, 40, (B, T), device="cuda")            # few distinct ids: long runs
    ids[0, :7] = V - 1
    dx = torch.randn(B * T, d, device="cuda").to(torch.bfloat16)
    outs = []
    K.set_deterministic(True)
    try:
        for _ in range(2):
            dwte = torch.zeros(V, d, device="cuda")
            dwpe = torch.zeros(T, d, device="cuda")
            K.embedding_bwd(ids, dx, dwte, dwpe)
            torch.cuda.synchronize()
            outs.append((dwte, dwpe))
        assert K.wgrad_split(768, 768, 16384) == 1
    finally:
        K.set_deterministic(False)
    ref_wte = torch.zeros(V, d, device="cuda").index_add_(0, ids.view(-1), dx.float())
    ref_wpe = dx.float().view(B, T, d).sum(0)
    assert torch.allclose(outs[0][0], ref_wte, atol=1e-3, rtol=1e-4)
    assert torch.allclose(outs[0][1], ref_wpe, atol=1e-3, rtol=1e-4)
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
