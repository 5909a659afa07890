"""The sm_100a engine against the reference's own model on the GPU, from the reference's initial weights.

The reference's ``GPT2`` (installed unmodified under ``baseline/_ref``) is built with its own initialisation,
its state dict is loaded into ``B200Engine`` (the key names are the same), and both train on the same seeded
Zipf(1.0) batches: the reference the way its ``train_step`` does (bf16 autocast over fp32 parameters, mean
cross-entropy over the kept tokens, ``clip_grad_norm_`` at 1.0, AdamW with its defaults: src/train.py:199-258,
src/utils.py:61), this engine through its kernels.  GPT-2 small width (d = 768, 12 heads, vocabulary 50304,
sequence length 1024), three blocks.  The curves must stay within 0.2 % of each other at every step, and at the
first step every gradient tensor must agree to 2 % in relative L2 error.
"""
import pytest
import torch

from helpers import make_config, single_world
from test_reference_parity import _import_reference

pytestmark = pytest.mark.gpu

D, HEADS, LAYERS, VOCAB, T, B = 768, 12, 3, 50304, 1024, 4
LR, STEPS = 6e-4, 20


def _setup():
    from diloco_swarm_b200.models.engine_b200 import B200Engine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    from diloco_swarm_b200.utils.data import zipf_tokens
    ref = _import_reference()
    dev = torch.device("cuda", 0)
    kw = dict(block_size=T, vocab_size=VOCAB, n_layer=LAYERS, n_head=HEADS, n_embd=D, dropout=0.0, bias=True,
              parameter_sharing=False)
    torch.manual_seed(1234)
    theirs = ref.model.GPT2(ref.model.GPT2Config(**kw)).to(dev)
    cfg = make_config(model={"n_layer": LAYERS, "n_head": HEADS, "n_embd": D, "vocab_size": VOCAB, "block_size": T},
                      data={"path": "synthetic:zipf", "seq_length": T},
                      train={"inner_optimizer": {"type": "AdamW", "lr": LR}, "outer_optimizer": {"type": "None", "lr": 0.0}})
    eng = B200Engine(GPT2Config(**kw), single_world(), cfg, dev)
    sd = {k: v.detach().float() for k, v in theirs.state_dict().items()}
    eng.load_state_dict(sd)
    tokens = zipf_tokens(B * STEPS, T + 1, VOCAB, 1.0, seed=7).to(dev)
    return ref, theirs, eng, tokens


def _reference_step(theirs, opt, ids, targets):
    opt.zero_grad(set_to_none=False)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        logits = theirs(ids)
    loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.size(-1)).float(), targets.reshape(-1))
    loss.backward()
    torch.nn.utils.clip_grad_norm_(theirs.parameters(), 1.0)
    return loss


def test_loss_curve_and_first_gradients_match_the_reference_model():
    ref, theirs, eng, tokens = _setup()
    opt = torch.optim.AdamW(theirs.parameters(), lr=LR, weight_decay=0.1, betas=(0.9, 0.95))    # src/utils.py:61
    mask = torch.ones(B, T, dtype=torch.long, device=tokens.device)
    ours, refs = [], []
    for step in range(STEPS):
        chunk = tokens[step * B:(step + 1) * B]
        ids, targets = chunk[:, :-1].contiguous(), chunk[:, 1:].contiguous()
        lr_ = _reference_step(theirs, opt, ids, targets)
        lo, _ = eng.forward_backward(0, ids, None, targets, mask, 1.0)
        if step == 0:
            # gradients before clipping on our side, after clipping on theirs: compare directions and, through
            # the common clip coefficient, sizes
            torch.cuda.synchronize()
            gn_ref = torch.sqrt(sum((p.grad.float() ** 2).sum() for p in theirs.parameters()))
            named = dict(theirs.named_parameters())
            total = torch.sqrt(sum((eng.g32(k).float() ** 2).sum() for k, _, _ in eng.specs))
            coef = min(1.0, 1.0 / (total.item() + 1e-6))
            worst = {}
            for key, _, _ in eng.specs:
                g_o, g_r = eng.g32(key).float().flatten() * coef, named[key].grad.float().flatten()
                rel = ((g_o - g_r).norm() / (g_r.norm() + 1e-12)).item()
                cls = key.split(".")[-2] + "." + key.split(".")[-1]
                worst[cls] = max(worst.get(cls, 0.0), rel)
            print("relative gradient error by tensor class:", {k: round(v, 4) for k, v in sorted(worst.items())})
            print("clipped gradient norm, reference:", gn_ref.item(), "total norm, engine:", total.item())
            for cls, rel in worst.items():
                assert rel <= 2e-2, f"{cls}: relative gradient error {rel:.4f}"
        opt.step()
        eng.optimizer_step(LR, 1.0)
        ours.append(lo.item())
        refs.append(lr_.item())
    torch.cuda.synchronize()
    eng.check_status()
    print("reference:", [round(x, 4) for x in refs])
    print("engine:   ", [round(x, 4) for x in ours])
    assert refs[-1] < refs[0] - 0.5, "the reference did not learn on these batches"
    for i, (a, b) in enumerate(zip(ours, refs)):
        assert abs(a - b) <= 2e-3 * abs(b), f"step {i}: engine {a:.4f} vs reference {b:.4f}"
