"""ORACLE - test infrastructure only, never imported by the product package.

Single-process fp32 restatement, in plain PyTorch, of what one Bamboo pipeline step
computes for the benchmark transformer, so that the CUDA path can be checked for
per-step loss and gradient parity.  What it follows in the reference:

* micro-batch loop, loss accumulation and returned loss = mean of the micro-batch losses:
  ``deepspeed/runtime/pipe/engine.py:1626-1727`` (``_exec_forward_pass`` /
  ``_exec_backward_pass``) and ``:1550-1553`` (``_aggregate_total_loss``);
* every micro-batch back-propagates ``loss / gradient_accumulation_steps``:
  ``deepspeed/runtime/engine.py:1317-1335,1416-1478``;
* one optimizer step per batch, then gradients cleared: ``deepspeed/runtime/engine.py:1526-1573``;
* Adam arithmetic of FusedAdam in its default ``adam_w_mode`` with weight decay 0:
  ``deepspeed/ops/adam/fused_adam.py:107-180`` and ``csrc/adam/multi_tensor_adam.cu:100-108``
  (identical to ``torch.optim.Adam`` up to rounding);
* layers applied in list order: ``deepspeed/runtime/pipe/module.py:516-553``.

The model itself (token + learned position embedding, pre-LN blocks with tanh-GeLU MLP,
final LayerNorm, untied vocabulary head, mean token cross entropy) is specified by the
benchmark configuration, not by the reference, whose examples train on random activations
(``DeepSpeedExamples/pipeline_parallelism/gpt2.py:20-154``).  The stage maths lives in
PyTorch (the reference pins torch 1.10; 2.11 is installed here).

Parity pin: the *instruction streams* are pinned by golden vectors generated from the
reference's own schedule code (tests/golden).  For the numbers there is nothing in the
reference to pin against (it has no such model, no CPU path and cannot be constructed
without etcd): numerical parity is "unpinned" beyond this restatement's agreement with
``torch.optim.Adam`` / ``torch.nn.functional`` semantics, which tests/test_oracle.py checks.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F


@dataclass
class RefConfig:
    layers: int
    hidden: int
    heads: int
    ffn: int
    seq: int
    vocab: int
    causal: bool = True
    mlm: bool = False       # BERT-style head: dense + GeLU + LayerNorm before the vocabulary decoder


def _normal(shape, gen):
    return torch.randn(shape, generator=gen, dtype=torch.float32) * 0.02


def init_params(cfg: RefConfig, seed: int = 0):
    """Layer i draws N(0, 0.02) from Generator(seed*1000 + i) in the order wte, wpe /
    qkv, proj, fc1, fc2 / head; biases 0, LayerNorm gain 1."""
    h, P = cfg.hidden, {}
    g = torch.Generator().manual_seed(seed * 1000)
    P["wte"] = _normal((cfg.vocab, h), g)
    P["wpe"] = _normal((cfg.seq, h), g)
    for i in range(cfg.layers):
        g = torch.Generator().manual_seed(seed * 1000 + 1 + i)
        p = f"b{i}."
        P[p + "ln1_w"], P[p + "ln1_b"] = torch.ones(h), torch.zeros(h)
        P[p + "qkv_w"], P[p + "qkv_b"] = _normal((3 * h, h), g), torch.zeros(3 * h)
        P[p + "proj_w"], P[p + "proj_b"] = _normal((h, h), g), torch.zeros(h)
        P[p + "ln2_w"], P[p + "ln2_b"] = torch.ones(h), torch.zeros(h)
        P[p + "fc1_w"], P[p + "fc1_b"] = _normal((cfg.ffn, h), g), torch.zeros(cfg.ffn)
        P[p + "fc2_w"], P[p + "fc2_b"] = _normal((h, cfg.ffn), g), torch.zeros(h)
    P["lnf_w"], P["lnf_b"] = torch.ones(h), torch.zeros(h)
    nxt = seed * 1000 + cfg.layers + 2
    if cfg.mlm:
        g = torch.Generator().manual_seed(nxt)
        P["mlm_w"], P["mlm_b"] = _normal((h, h), g), torch.zeros(h)
        P["mlm_ln_w"], P["mlm_ln_b"] = torch.ones(h), torch.zeros(h)
        nxt += 1
    g = torch.Generator().manual_seed(nxt)
    P["head_w"] = _normal((cfg.vocab, h), g)
    return P


def block_forward(cfg: RefConfig, P, prefix, x):
    B, S, h = x.shape
    H, D = cfg.heads, h // cfg.heads
    y = F.layer_norm(x, (h,), P[prefix + "ln1_w"], P[prefix + "ln1_b"], 1e-5)
    qkv = F.linear(y, P[prefix + "qkv_w"], P[prefix + "qkv_b"]).view(B, S, 3, H, D)
    q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
    s = (q @ k.transpose(-1, -2)) / math.sqrt(D)
    if cfg.causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device=x.device), 1), float("-inf"))
    a = (torch.softmax(s, dim=-1) @ v).transpose(1, 2).reshape(B, S, h)
    x = x + F.linear(a, P[prefix + "proj_w"], P[prefix + "proj_b"])
    y = F.layer_norm(x, (h,), P[prefix + "ln2_w"], P[prefix + "ln2_b"], 1e-5)
    y = F.gelu(F.linear(y, P[prefix + "fc1_w"], P[prefix + "fc1_b"]), approximate="tanh")
    return x + F.linear(y, P[prefix + "fc2_w"], P[prefix + "fc2_b"])


def forward_loss(cfg: RefConfig, P, tokens, labels, ignore_index=-100):
    B, S = tokens.shape
    x = P["wte"][tokens] + P["wpe"][:S].unsqueeze(0)
    for i in range(cfg.layers):
        x = block_forward(cfg, P, f"b{i}.", x)
    x = F.layer_norm(x, (cfg.hidden,), P["lnf_w"], P["lnf_b"], 1e-5)
    if cfg.mlm:
        x = F.gelu(F.linear(x, P["mlm_w"], P["mlm_b"]), approximate="tanh")
        x = F.layer_norm(x, (cfg.hidden,), P["mlm_ln_w"], P["mlm_ln_b"], 1e-5)
    logits = F.linear(x, P["head_w"])
    return F.cross_entropy(logits.view(-1, cfg.vocab), labels.reshape(-1), ignore_index=ignore_index)


def adam_update(p, g, m, v, step, lr, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, adam_w_mode=True):
    """In-place FusedAdam arithmetic (reference functor, both modes)."""
    if not adam_w_mode:
        g = g + weight_decay * p
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    update = (m / bc1) / ((v / bc2).sqrt() + eps)
    if adam_w_mode:
        update = update + weight_decay * p
    p.add_(update, alpha=-lr)


class RefTrainer:
    """Runs ``train_batch`` the way the pipeline engine does, on one process."""

    def __init__(self, cfg: RefConfig, seed=0, lr=1e-4, micro_batches=4, device="cpu", dtype=torch.float32):
        self.cfg, self.lr, self.micro_batches = cfg, lr, micro_batches
        self.P = {k: v.to(device=device, dtype=dtype).requires_grad_(True) for k, v in init_params(cfg, seed).items()}
        self.m = {k: torch.zeros_like(v) for k, v in self.P.items()}
        self.v = {k: torch.zeros_like(v) for k, v in self.P.items()}
        self.steps = 0
        self.last_grads = None

    def train_batch(self, batches):
        """``batches``: list of (tokens, labels), one per micro-batch.  Returns the mean loss;
        ``last_grads`` holds the accumulated gradients the optimizer consumed."""
        assert len(batches) == self.micro_batches
        total = 0.0
        for tokens, labels in batches:
            loss = forward_loss(self.cfg, self.P, tokens, labels)
            (loss / self.micro_batches).backward()
            total += float(loss.detach())
        self.steps += 1
        self.last_grads = {k: p.grad.detach().clone() for k, p in self.P.items()}
        with torch.no_grad():
            for k, p in self.P.items():
                adam_update(p, p.grad, self.m[k], self.v[k], self.steps, self.lr)
                p.grad = None
        return total / self.micro_batches


def synthetic_batches(cfg: RefConfig, micro_batch, micro_batches, steps, seed=1):
    """Uniform token ids from Generator(seed); labels are the tokens shifted left by one
    (next-token prediction), last position ignored."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(steps):
        step = []
        for _ in range(micro_batches):
            tok = torch.randint(0, cfg.vocab, (micro_batch, cfg.seq), generator=g)
            lab = torch.full_like(tok, -100)
            lab[:, :-1] = tok[:, 1:]
            step.append((tok, lab))
        out.append(step)
    return out


def synthetic_mlm_batches(cfg: RefConfig, micro_batch, micro_batches, steps, seed=1, mask_id=103):
    """Masked-LM micro-batches: uniform token ids from Generator(seed); per sequence 15 % of the
    positions are chosen (the first round(0.15 S) of a random permutation); labels hold the
    original token there and -100 elsewhere; chosen inputs become ``mask_id`` with probability
    0.8, a random token with 0.1 and stay with 0.1.  Draw order per micro-batch: tokens,
    permutation keys, the 80/10/10 roll, the replacement tokens."""
    g = torch.Generator().manual_seed(seed)
    n = max(1, int(round(0.15 * cfg.seq)))
    out = []
    for _ in range(steps):
        step = []
        for _ in range(micro_batches):
            tok = torch.randint(0, cfg.vocab, (micro_batch, cfg.seq), generator=g)
            pos = torch.rand(micro_batch, cfg.seq, generator=g).argsort(dim=1)[:, :n]
            roll = torch.rand(micro_batch, cfg.seq, generator=g)
            rnd = torch.randint(0, cfg.vocab, (micro_batch, cfg.seq), generator=g)
            lab = torch.full_like(tok, -100)
            inp = tok.clone()
            for b in range(micro_batch):
                for p_ in pos[b].tolist():
                    lab[b, p_] = tok[b, p_]
                    if roll[b, p_] < 0.8:
                        inp[b, p_] = mask_id
                    elif roll[b, p_] < 0.9:
                        inp[b, p_] = rnd[b, p_]
            step.append((inp, lab))
        out.append(step)
    return out
