"""ORACLE - test infrastructure only, never imported by the product package.

Single-process fp32 restatement, in plain PyTorch (NCHW, ``torch.nn.functional``), of one
pipeline step over a bottleneck ResNet, for loss / gradient parity of the channels-last CUDA
layers.  The step logic is the one ``oracle/gpt_ref.py`` restates (micro-batch loop with
``loss / gradient_accumulation_steps``, mean reported loss, one FusedAdam-equivalent update:
``deepspeed/runtime/pipe/engine.py:1626-1727``, ``deepspeed/runtime/engine.py:1416-1478,1526-1573``).
The network is torchvision's ``resnet152`` as the reference pipelines it
(``DeepSpeedExamples/osdi22-cv/resnet-exp.py:69-83``): 7 x 7 / 2 stem convolution, batch norm
(training mode: batch statistics, biased variance), ReLU, 3 x 3 / 2 max pooling, bottleneck
blocks [3, 8, 36, 3] with the stride on the 3 x 3 convolution and a projected shortcut in the
first block of every stage, global average pooling, fully connected classifier, cross entropy.
torchvision is not installed here and the reference pins torch 1.10 / torchvision 0.11: the
architecture is restated from its published definition; **parity unpinned** against the
reference's own run (it needs CUDA and etcd).

Parameters are drawn exactly like the product layers draw them (``bamboo_b200/resnet.py``):
layer ``i`` uses ``Generator(seed * 1000 + i)``; a convolution draws ``[Cout, k, k, Cin]``
(Kaiming normal, fan-out) and is permuted to ``[Cout, Cin, k, k]`` here; the stem draws 8 input
channels of which the image uses the first 3.
"""
import math

import torch
import torch.nn.functional as F

from .gpt_ref import adam_update


def _conv_w(g, cin, cout, k):
    std = math.sqrt(2.0 / (cout * k * k))
    w = torch.randn(cout, k, k, cin, generator=g, dtype=torch.float32) * std
    return w.permute(0, 3, 1, 2).contiguous()


def init_params(blocks=(3, 8, 36, 3), classes=1000, width=64, seed=0):
    """Ordered ``{name: tensor}``; names ``<layer>.<conv>.{weight,bn_weight,bn_bias}`` and ``<last>.fc.{weight,bias}``."""
    P = {}
    base = seed * 1000
    g = torch.Generator().manual_seed(base)
    P["0.conv.weight"] = _conv_w(g, 8, width, 7)
    P["0.conv.bn_weight"], P["0.conv.bn_bias"] = torch.ones(width), torch.zeros(width)
    cin, i = width, 1
    for stage, n in enumerate(blocks):
        mid = width * (2 ** stage)
        for b in range(n):
            g = torch.Generator().manual_seed(base + i)
            for name, (ci, co, k) in (("conv1", (cin, mid, 1)), ("conv2", (mid, mid, 3)), ("conv3", (mid, mid * 4, 1))):
                P[f"{i}.{name}.weight"] = _conv_w(g, ci, co, k)
                P[f"{i}.{name}.bn_weight"], P[f"{i}.{name}.bn_bias"] = torch.ones(co), torch.zeros(co)
            if b == 0:
                P[f"{i}.down.weight"] = _conv_w(g, cin, mid * 4, 1)
                P[f"{i}.down.bn_weight"], P[f"{i}.down.bn_bias"] = torch.ones(mid * 4), torch.zeros(mid * 4)
            cin, i = mid * 4, i + 1
    g = torch.Generator().manual_seed(base + i)
    P[f"{i}.fc.weight"] = torch.randn(classes, cin, generator=g, dtype=torch.float32) * 0.02
    P[f"{i}.fc.bias"] = torch.zeros(classes)
    return P


def _conv_bn(P, prefix, x, stride, k, relu, residual=None, eps=1e-5):
    w = P[f"{prefix}.weight"]
    if prefix == "0.conv":
        w = w[:, :3]                                    # the product carries 5 zero input planes
    y = F.conv2d(x, w, None, stride=stride, padding=(k - 1) // 2)
    y = F.batch_norm(y, None, None, P[f"{prefix}.bn_weight"], P[f"{prefix}.bn_bias"], training=True, eps=eps)
    if residual is not None:
        y = y + residual
    return F.relu(y) if relu else y


def forward_loss(P, images, labels, blocks=(3, 8, 36, 3)):
    """``images``: [N, 3, H, W] fp32; returns the mean cross entropy."""
    x = _conv_bn(P, "0.conv", images, 2, 7, True)
    x = F.max_pool2d(x, 3, 2, 1)
    i = 1
    for stage, n in enumerate(blocks):
        for b in range(n):
            stride = 2 if (b == 0 and stage > 0) else 1
            identity = _conv_bn(P, f"{i}.down", x, stride, 1, False) if b == 0 else x
            y = _conv_bn(P, f"{i}.conv1", x, 1, 1, True)
            y = _conv_bn(P, f"{i}.conv2", y, stride, 3, True)
            x = _conv_bn(P, f"{i}.conv3", y, 1, 1, True, residual=identity)
            i += 1
    x = F.adaptive_avg_pool2d(x, 1).flatten(1)
    logits = F.linear(x, P[f"{i}.fc.weight"], P[f"{i}.fc.bias"])
    return F.cross_entropy(logits, labels)


class RefTrainer:
    def __init__(self, blocks=(3, 8, 36, 3), classes=1000, width=64, seed=0, lr=1e-4, micro_batches=2):
        self.blocks, self.lr, self.micro_batches = tuple(blocks), lr, micro_batches
        self.P = {k: v.requires_grad_(True) for k, v in init_params(blocks, classes, width, seed).items()}
        self.m = {k: torch.zeros_like(v) for k, v in self.P.items()}
        self.v = {k: torch.zeros_like(v) for k, v in self.P.items()}
        self.steps = 0
        self.last_grads = None

    def train_batch(self, batches):
        assert len(batches) == self.micro_batches
        total = 0.0
        for images, labels in batches:
            loss = forward_loss(self.P, images, labels, self.blocks)
            (loss / self.micro_batches).backward()
            total += float(loss.detach())
        self.steps += 1
        self.last_grads = {k: (p.grad.detach().clone() if p.grad is not None else torch.zeros_like(p)) for k, p in self.P.items()}
        with torch.no_grad():
            for k, p in self.P.items():
                if p.grad is None:
                    continue
                adam_update(p, p.grad, self.m[k], self.v[k], self.steps, self.lr)
                p.grad = None
        return total / self.micro_batches


def synthetic_batches(micro_batch, micro_batches, steps, size=224, classes=1000, seed=1):
    """N(0, 1) images [N, 3, size, size] and uniform labels from ``Generator(seed)``."""
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(steps):
        step = []
        for _ in range(micro_batches):
            step.append((torch.randn(micro_batch, 3, size, size, generator=g),
                         torch.randint(0, classes, (micro_batch,), generator=g)))
        out.append(step)
    return out


def to_channels_last_8(images):
    """[N, 3, H, W] fp32 -> [N, H, W, 8] bf16 with five zero planes (the product's input layout)."""
    n, c, h, w = images.shape
    x = torch.zeros(n, h, w, 8, dtype=torch.bfloat16)
    x[..., :c] = images.permute(0, 2, 3, 1).to(torch.bfloat16)
    return x
