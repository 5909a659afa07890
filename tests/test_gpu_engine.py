"""The sm_100a stage engine against the autograd engine on the same weights."""
import pytest
import torch

from helpers import make_config, single_world

pytestmark = pytest.mark.gpu


def _engines(**over):
    from diloco_swarm_b200.models.engine_b200 import B200Engine
    from diloco_swarm_b200.models.engine_torch import TorchEngine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    cfg = make_config(**over)
    mc = cfg.model
    g = GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                   n_embd=mc.n_embd)
    w = single_world()
    dev = torch.device("cuda", 0)
    return cfg, B200Engine(g, w, cfg, dev), TorchEngine(g, w, cfg, dev)


def _batch(cfg, B=4, T=64, seed=0):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, 500, (B, T + 1), generator=g).cuda()
    mask = (torch.rand(B, T, generator=g) > 0.1).long().cuda()
    return ids[:, :-1].contiguous(), ids[:, 1:].contiguous(), mask


@pytest.mark.parametrize("attn", ["native", "sdpa"])
def test_forward_backward_matches_autograd(attn, monkeypatch):
    monkeypatch.setenv("DSWARM_ATTENTION", attn)
    cfg, eb, et = _engines()
    ids, tg, mask = _batch(cfg)
    lb, _ = eb.forward_backward(0, ids, None, tg, mask, 0.5)
    lt, _ = et.forward_backward(0, ids, None, tg, mask, 0.5)
    torch.cuda.synchronize()
    eb.check_status()
    assert abs(lb.item() - lt.item()) < 2e-2 * abs(lt.item())
    ref = dict(et.model.named_parameters())
    worst = 1.0
    for key, _, _ in eb.specs:
        gb, gt = eb.g32(key).flatten(), ref[key].grad.flatten()
        cos = torch.nn.functional.cosine_similarity(gb, gt, dim=0).item()
        worst = min(worst, cos)
        assert cos > 0.98, f"gradient of {key}: cosine {cos}"
        assert abs(gb.norm().item() / (gt.norm().item() + 1e-12) - 1) < 0.05, key


def test_training_reduces_loss_and_tracks_autograd():
    cfg, eb, et = _engines()
    ids, tg, mask = _batch(cfg)
    lb0 = lt0 = None
    for step in range(8):
        lb, _ = eb.forward_backward(0, ids, None, tg, mask, 1.0)
        lt, _ = et.forward_backward(0, ids, None, tg, mask, 1.0)
        nb = eb.optimizer_step(1e-3, 1.0)
        nt = et.optimizer_step(1e-3, 1.0)
        et.zero_grad()
        if step == 0:
            lb0, lt0 = lb.item(), lt.item()
            assert abs(float(nb) - nt) < 0.05 * nt
    eb.check_status()
    assert lb.item() < lb0 - 0.3
    assert abs(lb.item() - lt.item()) < 0.05 * lt.item()


def test_pipeline_split_equals_whole():
    """Two stage engines chained by hand reproduce the single-stage loss and input gradient path."""
    from diloco_swarm_b200.models.engine_b200 import B200Engine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    from diloco_swarm_b200.world import World
    import os
    cfg = make_config(swarm={"num_stages": 2})
    mc = cfg.model
    g = GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                   n_embd=mc.n_embd)
    dev = torch.device("cuda", 0)
    os.environ.update(RANK="0", WORLD_SIZE="2")
    w0 = World(2, init=False)
    os.environ.update(RANK="1", WORLD_SIZE="2")
    w1 = World(2, init=False)
    os.environ.pop("RANK"); os.environ.pop("WORLD_SIZE")
    w0.num_replicas = w1.num_replicas = 1
    e0, e1 = B200Engine(g, w0, cfg, dev), B200Engine(g, w1, cfg, dev)
    cfg1 = make_config()
    whole = B200Engine(g, single_world(), cfg1, dev)
    ids, tg, mask = _batch(cfg)
    y = e0.forward(0, ids, None)
    loss, dx = e1.forward_backward(0, None, y, tg, mask, 1.0)
    e0.backward(0, dx)
    lw, _ = whole.forward_backward(0, ids, None, tg, mask, 1.0)
    assert abs(loss.item() - lw.item()) < 1e-3 * abs(lw.item())
    a = e0.g32("transformer.h.0.attn.c_attn.weight").flatten()
    b = whole.g32("transformer.h.0.attn.c_attn.weight").flatten()
    assert torch.nn.functional.cosine_similarity(a, b, dim=0).item() > 0.999


def test_diloco_outer_step_single_replica():
    cfg, eb, _ = _engines(train={"outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}})
    ids, tg, mask = _batch(cfg)
    theta0 = eb.theta.clone()
    for _ in range(3):
        eb.forward_backward(0, ids, None, tg, mask, 1.0)
        eb.optimizer_step(1e-3, 1.0)
    inner = eb.theta.clone()
    eb.outer_step()
    torch.cuda.synchronize()
    eb.check_status()
    delta = theta0 - inner
    want = theta0 - 0.7 * (delta + 0.9 * delta)     # first Nesterov step: buf = delta
    assert torch.allclose(eb.theta, want, atol=1e-6)
    assert torch.allclose(eb.w16.float(), eb.theta, atol=1e-2, rtol=1e-2)


def test_checkpoint_roundtrip_restores_the_training_state(tmp_path):
    """state_dict / optimiser / outer state of the flat-buffer engine: a fresh engine loaded from them
    continues exactly like the original."""
    from diloco_swarm_b200.models.engine_b200 import B200Engine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    cfg = make_config(train={"outer_optimizer": {"type": "SGD", "lr": 0.7, "momentum": 0.9, "nesterov": True}})
    mc = cfg.model
    g = GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                   n_embd=mc.n_embd)
    dev = torch.device("cuda", 0)
    a = B200Engine(g, single_world(), cfg, dev)
    ids, tg, mask = _batch(cfg)
    for _ in range(3):
        a.forward_backward(0, ids, None, tg, mask, 1.0)
        a.optimizer_step(1e-3, 1.0)
    a.outer_step()
    sd, opt, outer = a.state_dict(), a.optim_state(), a.outer_state()
    assert set(sd) == {k for k, _, _ in a.specs} and sd["lm_head.weight"].shape == (mc.vocab_size, mc.n_embd)
    torch.save(sd, tmp_path / "model.pt")
    b = B200Engine(g, single_world(), cfg, dev)
    b.load_state_dict(torch.load(tmp_path / "model.pt", weights_only=True))
    b.load_optim_state(opt)
    b.load_outer_state(outer)
    for eng in (a, b):
        eng.forward_backward(0, ids, None, tg, mask, 1.0)
        eng.optimizer_step(1e-3, 1.0)
        eng.outer_step()
    torch.cuda.synchronize()
    assert torch.allclose(a.theta, b.theta, atol=1e-6)
    la, _ = a.forward_backward(1, ids, None, tg, mask, 1.0)
    lb, _ = b.forward_backward(1, ids, None, tg, mask, 1.0)
    assert abs(la.item() - lb.item()) < 1e-4


def test_sgd_inner_optimizer_and_explicit_layer_split():
    from diloco_swarm_b200.models.engine_b200 import B200Engine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    cfg = make_config(train={"inner_optimizer": {"type": "SGD", "lr": 0.05, "momentum": 0.9, "nesterov": True}},
                      swarm={"layer_split": "2"})
    mc = cfg.model
    g = GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                   n_embd=mc.n_embd)
    eng = B200Engine(g, single_world(), cfg, torch.device("cuda", 0))
    ids, tg, mask = _batch(cfg)
    first = None
    for _ in range(6):
        loss, _ = eng.forward_backward(0, ids, None, tg, mask, 1.0)
        eng.optimizer_step(0.05, 1.0)
        first = first if first is not None else loss.item()
    eng.check_status()
    assert loss.item() < first


def test_chunked_lm_head_matches_the_whole_one():
    """train.lm_head_chunks = 4: logits, cross-entropy and the head's gradients over four slices of the token
    rows give the loss and the gradients of the one-piece head (the divisor is the microbatch's kept-row count,
    not a slice's)."""
    _, whole, _ = _engines()
    cfg4, sliced, _ = _engines(train={"lm_head_chunks": 4})
    assert sliced.head_chunks == 4 and whole.head_chunks == 1
    ids, tg, mask = _batch(cfg4, B=16, T=64)
    l1, _ = whole.forward_backward(0, ids, None, tg, mask, 0.5)
    l4, _ = sliced.forward_backward(0, ids, None, tg, mask, 0.5)
    e1 = whole.forward_loss(ids, None, tg, mask, 0.5)
    e4 = sliced.forward_loss(ids, None, tg, mask, 0.5)
    torch.cuda.synchronize()
    whole.check_status()
    sliced.check_status()
    assert abs(l1.item() - l4.item()) < 1e-4 * abs(l1.item())
    assert abs(e1.item() - e4.item()) < 1e-4 * abs(e1.item())
    for key, _, _ in whole.specs:
        a, b = whole.g32(key).flatten(), sliced.g32(key).flatten()
        assert torch.allclose(a, b, rtol=2e-2, atol=2e-3 * a.abs().max().item() + 1e-8), key
        assert abs(a.norm().item() - b.norm().item()) <= 2e-3 * a.norm().item() + 1e-8, key
