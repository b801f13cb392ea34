"""Flat per-stage parameter storage and the Adam step over it.

The reference keeps one tensor per parameter, lets autograd fill ``param.grad``, flattens
gradients into buckets for the all-reduce (``deepspeed/runtime/engine.py:1728-1771``,
``csrc/utils/flatten_unflatten.cpp:11-25``) and steps with FusedAdam
(``deepspeed/ops/adam/fused_adam.py:85-182``).  Here a stage's parameters live in flat
buffers from the start, so the all-reduce and the optimizer see one contiguous tensor and
nothing is flattened per step:

* ``master`` fp32 weights, ``grad`` fp32 gradient accumulator, ``exp_avg``/``exp_avg_sq``;
* ``lp``: the working copy the layers read - bf16 for the sm_100a kernels, or the master
  buffer itself for fp32 modules.

``flatten``/``unflatten`` keep the reference's two-function interface for callers that
still hold tensor lists.
"""
from typing import Iterable, List

import torch
from torch import nn


def flatten(tensors):
    """Concatenate dense tensors into one 1-D tensor (reference ``utils_op.flatten``)."""
    return torch.cat([t.reshape(-1) for t in tensors]) if len(tensors) else torch.empty(0)


def unflatten(flat, tensors):
    """Views of ``flat`` shaped like ``tensors`` (reference ``utils_op.unflatten``)."""
    out, off = [], 0
    for t in tensors:
        n = t.numel()
        out.append(flat[off:off + n].view(t.shape))
        off += n
    return out


class ParamArena:
    ALIGN = 8  # elements; keeps every parameter 16-byte aligned in the bf16 buffer

    def __init__(self, params: Iterable[nn.Parameter], device, lp_dtype=torch.bfloat16, with_optimizer_state=True):
        self.params: List[nn.Parameter] = list(params)
        self.device = torch.device(device)
        self.lp_dtype = lp_dtype
        self.offsets, total = [], 0
        for p in self.params:
            self.offsets.append(total)
            total += (p.numel() + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        self.numel = max(total, self.ALIGN)
        self.master = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        for p, off in zip(self.params, self.offsets):
            self.master[off:off + p.numel()].copy_(p.data.detach().reshape(-1).to(self.device, torch.float32))
        if lp_dtype == torch.float32:
            self.lp = self.master
        else:
            self.lp = self.master.to(lp_dtype)
        self.grad = self.exp_avg = self.exp_avg_sq = None
        for p, off in zip(self.params, self.offsets):
            p.data = self.lp[off:off + p.numel()].view(p.shape)
            p.grad = None
        if with_optimizer_state:
            self.allocate_optimizer_state()
        self.step_count = 0

    def allocate_optimizer_state(self):
        if self.grad is not None:
            return
        self.grad = torch.zeros(self.numel, dtype=torch.float32, device=self.device)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        for p, off in zip(self.params, self.offsets):
            p.main_grad = self.grad[off:off + p.numel()].view(p.shape)

    def named_slices(self):
        """(index, offset, numel) of every parameter in the flat buffers."""
        for i, (p, off) in enumerate(zip(self.params, self.offsets)):
            yield i, off, p.numel()

    def fold_autograd_grads(self):
        """Generic torch layers leave their gradient in ``param.grad``; accumulate it into
        the fp32 arena (the sm_100a layers write there directly and leave ``grad`` None)."""
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    def refresh_lp(self):
        """lp = cast(master) after the master copy was overwritten (weight sync, promotion)."""
        if self.lp is self.master:
            return
        if self.master.is_cuda and self.lp_dtype == torch.bfloat16:
            from . import lib as L
            L.cast_f32_to_bf16(self.master, self.lp)
        else:
            self.lp.copy_(self.master)

    def state_tensors(self):
        """What a shadow copy of this stage needs: weights and both Adam moments."""
        return [self.master, self.exp_avg, self.exp_avg_sq]

    def adam_step(self, *, lr, beta1, beta2, eps, weight_decay, adam_w_mode, bias_correction, grad_scale=1.0):
        """One Adam step; clears the gradient.  CUDA arenas use the fused kernel; CPU arenas
        (plumbing runs) evaluate the same formula (csrc/adam/multi_tensor_adam.cu:72-108 of
        the reference) with tensor ops."""
        self.step_count += 1
        step = self.step_count
        if self.master.is_cuda:
            from . import lib as L
            L.adam_step(self.master, self.grad, self.exp_avg, self.exp_avg_sq,
                        None if self.lp is self.master else self.lp, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                        step=step, adam_w_mode=adam_w_mode, bias_correction=bias_correction,
                        weight_decay=weight_decay, grad_scale=grad_scale, zero_grad=True)
            return
        g = self.grad * grad_scale if grad_scale != 1.0 else self.grad
        bc1 = 1.0 - beta1 ** step if bias_correction else 1.0
        bc2 = 1.0 - beta2 ** step if bias_correction else 1.0
        if not adam_w_mode and weight_decay:
            g = g + weight_decay * self.master
        self.exp_avg.mul_(beta1).add_(g, alpha=1.0 - beta1)
        self.exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
        update = (self.exp_avg / bc1) / ((self.exp_avg_sq / bc2).sqrt_().add_(eps))
        if adam_w_mode and weight_decay:
            update.add_(self.master, alpha=weight_decay)
        self.master.add_(update, alpha=-lr)
        self.grad.zero_()
        self.refresh_lp()
