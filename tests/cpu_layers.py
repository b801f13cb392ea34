"""Plain-PyTorch fp32 layers built from the oracle's functions, used to drive the engine's
host logic (schedules, transport, redundancy, failover) on CPU ranks."""
import os
import sys

import torch
from torch import nn

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from oracle import gpt_ref  # noqa: E402


class RefEmbedding(nn.Module):
    def __init__(self, cfg, seed):
        super().__init__()
        P = gpt_ref.init_params(cfg, seed)
        self.wte, self.wpe = nn.Parameter(P["wte"]), nn.Parameter(P["wpe"])

    def forward(self, tokens):
        return self.wte[tokens] + self.wpe[: tokens.shape[1]].unsqueeze(0)


class RefBlock(nn.Module):
    NAMES = ["ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b"]

    def __init__(self, cfg, seed, index):
        super().__init__()
        self.cfg = cfg
        P = gpt_ref.init_params(cfg, seed)
        for n in self.NAMES:
            setattr(self, n, nn.Parameter(P[f"b{index}.{n}"]))

    def forward(self, x):
        return gpt_ref.block_forward(self.cfg, {"." + n: getattr(self, n) for n in self.NAMES}, ".", x)


class RefNorm(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.weight, self.bias = nn.Parameter(torch.ones(cfg.hidden)), nn.Parameter(torch.zeros(cfg.hidden))

    def forward(self, x):
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), self.weight, self.bias, 1e-5)


class RefHead(nn.Module):
    def __init__(self, cfg, seed):
        super().__init__()
        self.weight = nn.Parameter(gpt_ref.init_params(cfg, seed)["head_w"])

    def forward(self, x):
        return torch.nn.functional.linear(x, self.weight)


def ref_layer_specs(cfg, seed=0):
    from bamboo_b200.module import LayerSpec
    specs = [LayerSpec(RefEmbedding, cfg, seed)]
    specs += [LayerSpec(RefBlock, cfg, seed, i) for i in range(cfg.layers)]
    specs += [LayerSpec(RefNorm, cfg), LayerSpec(RefHead, cfg, seed)]
    return specs


def ref_loss(cfg):
    def loss_fn(logits, labels):
        return torch.nn.functional.cross_entropy(logits.view(-1, cfg.vocab), labels.reshape(-1), ignore_index=-100)
    return loss_fn
