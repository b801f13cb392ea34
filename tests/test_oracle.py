"""The oracle's own pins: its Adam arithmetic is torch.optim.Adam's, its loop is plain
gradient accumulation, its init recipe is deterministic."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import gpt_ref  # noqa: E402

CFG = gpt_ref.RefConfig(layers=2, hidden=32, heads=2, ffn=64, seq=8, vocab=50)


def test_adam_update_is_torch_adam():
    torch.manual_seed(0)
    p = torch.randn(1000)
    ref = p.clone().requires_grad_(True)
    opt = torch.optim.Adam([ref], lr=1e-3)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    for step in range(1, 6):
        g = torch.randn(1000)
        ref.grad = g.clone()
        opt.step()
        gpt_ref.adam_update(p, g, m, v, step, 1e-3)
    assert torch.allclose(p, ref.detach(), rtol=1e-5, atol=1e-7)


def test_train_batch_is_accumulation_over_micro_batches():
    data = gpt_ref.synthetic_batches(CFG, 2, 4, 1, seed=1)[0]
    a = gpt_ref.RefTrainer(CFG, seed=0, lr=1e-3, micro_batches=4)
    loss = a.train_batch(data)
    # same thing as one big batch (all sequences have the same number of valid labels)
    P = {k: v.clone().requires_grad_(True) for k, v in gpt_ref.init_params(CFG, 0).items()}
    tok = torch.cat([t for t, _ in data]); lab = torch.cat([l for _, l in data])
    big = gpt_ref.forward_loss(CFG, P, tok, lab)
    big.backward()
    assert loss == pytest.approx(float(big), rel=1e-5)
    for k in P:
        assert torch.allclose(a.last_grads[k], P[k].grad, rtol=1e-4, atol=1e-6), k


def test_init_is_deterministic_and_layerwise():
    a, b = gpt_ref.init_params(CFG, 0), gpt_ref.init_params(CFG, 0)
    assert all(torch.equal(a[k], b[k]) for k in a)
    c = gpt_ref.init_params(CFG, 1)
    assert not torch.equal(a["wte"], c["wte"])
    assert abs(float(a["b0.qkv_w"].std()) - 0.02) < 0.004
    assert float(a["b0.qkv_b"].abs().sum()) == 0 and float(a["lnf_w"].mean()) == 1


def test_product_init_recipe_matches_oracle():
    """The product's layer constructors draw the same values as the oracle (checked on CPU
    before any arena adoption)."""
    from bamboo_b200 import layers
    P = gpt_ref.init_params(CFG, 0)
    emb = layers.TokenEmbedding(CFG.vocab, CFG.hidden, CFG.seq, seed=0)
    assert torch.equal(emb.wte.data, P["wte"]) and torch.equal(emb.wpe.data, P["wpe"])
    blk = layers.TransformerBlock(CFG.hidden, CFG.heads, CFG.ffn, seed=2)
    for n in ("qkv_w", "proj_w", "fc1_w", "fc2_w"):
        assert torch.equal(getattr(blk, n).data, P[f"b1.{n}"]), n
    head = layers.Linear(CFG.hidden, CFG.vocab, bias=False, pad_to=128, seed=CFG.layers + 2)
    assert torch.equal(head.weight.data[: CFG.vocab], P["head_w"]) and head.weight.shape[0] == 128


def test_masked_lm_batches_and_loss():
    """15 % of every sequence is chosen, labels elsewhere are ignored, about 80 % of the chosen
    inputs carry the mask id; the product's vectorised masking draws the same batch; the loss is
    the mean over the chosen positions only."""
    import torch.nn.functional as F
    from bamboo_b200 import models
    cfg = gpt_ref.RefConfig(layers=1, hidden=64, heads=2, ffn=128, seq=128, vocab=1000, causal=False, mlm=True)
    (inp, lab), = gpt_ref.synthetic_mlm_batches(cfg, 8, 1, 1, seed=3)[0]
    chosen = lab != -100
    assert chosen.sum(1).tolist() == [round(0.15 * cfg.seq)] * 8
    frac_mask = (inp[chosen] == 103).float().mean().item()
    assert 0.7 < frac_mask < 0.9
    assert torch.equal(inp[~chosen], inp[~chosen]) and (inp[~chosen] != 103).float().mean() > 0.99
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, cfg.vocab, (8, cfg.seq), generator=g)
    inp2, lab2 = models.mlm_mask(tok, g, cfg.vocab)
    assert torch.equal(inp, inp2) and torch.equal(lab, lab2)
    P = gpt_ref.init_params(cfg, 0)
    loss = gpt_ref.forward_loss(cfg, P, inp, lab)
    # same loss from per-position terms averaged over the chosen positions by hand
    full = gpt_ref.forward_loss(cfg, P, inp, torch.where(chosen, lab, torch.zeros_like(lab)))  # all positions labelled
    assert loss.item() != pytest.approx(full.item(), rel=1e-6)
    x = P["wte"][inp] + P["wpe"][: cfg.seq].unsqueeze(0)
    x = gpt_ref.block_forward(cfg, P, "b0.", x)
    x = F.layer_norm(x, (cfg.hidden,), P["lnf_w"], P["lnf_b"], 1e-5)
    x = F.layer_norm(F.gelu(F.linear(x, P["mlm_w"], P["mlm_b"]), approximate="tanh"), (cfg.hidden,), P["mlm_ln_w"], P["mlm_ln_b"], 1e-5)
    logp = F.log_softmax(F.linear(x, P["head_w"]), -1)
    manual = -(logp[chosen].gather(1, lab[chosen].unsqueeze(1))).mean()
    assert loss.item() == pytest.approx(manual.item(), rel=1e-5)
