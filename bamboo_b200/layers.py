"""Transformer stage layers whose forward and backward run on the sm_100a kernels.

Each layer is an ``nn.Module`` (so it can sit in a ``PipelineModule`` layer list like the
reference's example layers, ``DeepSpeedExamples/pipeline_parallelism/gpt2.py:20-150``) whose
computation is a ``torch.autograd.Function`` calling the C ABI: tcgen05 GEMMs with fused
bias / GeLU / residual epilogues, fused attention, LayerNorm, embedding, cross entropy.
``BackwardPass`` therefore stays ``torch.autograd.backward`` as in the reference engine
(``deepspeed/runtime/pipe/engine.py:1680-1727``).

Weights are bf16 views into a :class:`ParamArena` (fp32 master copy, fp32 gradient, Adam
moments, bf16 working copy - one flat buffer each per stage).  Weight gradients are
accumulated by the kernels straight into the fp32 gradient arena (``param.main_grad``);
autograd only carries activation gradients.

There is no fallback: these modules raise on CPU tensors.
"""
import ctypes
import math
from typing import Iterable, List, Optional

import torch
from torch import nn

from . import lib as L
from .arena import ParamArena  # noqa: F401  (re-exported)


def _require_cuda(t, what):
    if not t.is_cuda:
        raise L.BambooNativeError(f"{what}: expected a CUDA tensor; the sm_100a kernels have no CPU fallback")


def _main_grad(p):
    g = getattr(p, "main_grad", None)
    if g is None:
        raise L.BambooNativeError("parameter has no main_grad: adopt the module into a ParamArena first "
                                  "(deepspeed.initialize does this)")
    return g


# ----------------------------------------------------------------------------------- functions
_side_streams = {}
# False: weight-gradient work stays on the launching stream (used when kernels are timed one by
# one with events, which concurrent work on a second stream would distort)
WGRAD_SIDE_STREAM = True


def _wgrad_stream(device):
    """Per-device side stream for weight-gradient work.  Weight gradients are off the backward
    critical path (nothing downstream reads them before the optimizer step), so their GEMMs and
    bias column sums run beside the input-gradient chain and fill the SMs that the tail of each
    persistent GEMM leaves idle."""
    st = _side_streams.get(device.index)
    if st is None:
        # one level below the highest priority: above redundant computation, below the chain of
        # input gradients it runs beside
        lo, hi = torch.cuda.Stream.priority_range()
        st = torch.cuda.Stream(device=device, priority=min(hi + 1, lo))
        _side_streams[device.index] = st
    return st


def wgrad_sync(device):
    """Make the current stream wait for all weight-gradient work issued so far on ``device``."""
    st = _side_streams.get(device.index if device.index is not None else torch.cuda.current_device())
    if st is not None:
        torch.cuda.current_stream(device).wait_stream(st)


def _wgrad(dy2d, x2d, weight, bias, stream=None):
    """dW += dy^T x ; db += colsum(dy), into the fp32 gradient arena."""
    L.gemm(dy2d, x2d, _main_grad(weight), a_mn=True, b_mn=True, epilogue=L.EPI_ACCUM_F32,
           M=dy2d.shape[1], N=weight.shape[1], K=dy2d.shape[0], stream=stream)
    if bias is not None:
        L.colsum_accum(dy2d, _main_grad(bias), tag="wgrad", stream=stream)


def flush_wgrads(pending):
    """Launch the deferred weight-gradient work `[(dy, x, weight, bias), ...]`: on the side stream
    (one fork per call, all operands already produced on the current stream), or in place when
    the side stream is switched off."""
    if not pending:
        return
    if not WGRAD_SIDE_STREAM:
        for item in pending:
            _wgrad(*item)
        return
    dev = pending[0][0].device
    side = _wgrad_stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    raw = side.cuda_stream
    for dy2d, x2d, weight, bias in pending:
        _wgrad(dy2d, x2d, weight, bias, stream=raw)
        # the caching allocator must not hand these buffers out again before the side stream is done
        dy2d.record_stream(side)
        x2d.record_stream(side)


def _linear_backward(dy2d, x2d, weight, bias, dx_out=None, dx_epilogue=L.EPI_STORE, aux=None, need_dx=True, defer=None):
    """dx = dy @ W (optionally through a fused epilogue); the weight and bias gradients are
    launched right away, or appended to `defer` for one `flush_wgrads` call per layer."""
    T, n_out = dy2d.shape
    n_in = weight.shape[1]
    if defer is None:
        flush_wgrads([(dy2d, x2d, weight, bias)])
    else:
        defer.append((dy2d, x2d, weight, bias))
    dx = None
    if need_dx:
        dx = dx_out if dx_out is not None else torch.empty(T, n_in, dtype=torch.bfloat16, device=dy2d.device)
        L.gemm(dy2d, weight, dx, b_mn=True, epilogue=dx_epilogue, aux=aux, M=T, N=n_in, K=n_out)
    return dx


class _BlockFn(torch.autograd.Function):
    """Pre-LN transformer block: x + Attn(LN1(x)) then + MLP(LN2(.))."""

    @staticmethod
    def forward(ctx, x, blk, *params):
        _require_cuda(x, "TransformerBlock")
        shape = x.shape
        h = shape[-1]
        x2 = x.reshape(-1, h)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        B, S = (shape[0], shape[1]) if x.dim() == 3 else (1, T)
        H, D = blk.heads, h // blk.heads
        dev, bf = x.device, torch.bfloat16
        f32 = torch.float32
        mean1, rstd1 = torch.empty(T, dtype=f32, device=dev), torch.empty(T, dtype=f32, device=dev)
        mean2, rstd2 = torch.empty(T, dtype=f32, device=dev), torch.empty(T, dtype=f32, device=dev)
        h1 = torch.empty(T, h, dtype=bf, device=dev)
        L.layernorm_fwd(x2, blk.ln1_w, blk.ln1_b, h1, mean1, rstd1, blk.eps)
        qkv = torch.empty(T, 3 * h, dtype=bf, device=dev)
        L.gemm(h1, blk.qkv_w, qkv, epilogue=L.EPI_BIAS, bias=blk.qkv_b)
        att = torch.empty(T, h, dtype=bf, device=dev)
        lse = torch.empty(B, H, S, dtype=f32, device=dev)
        L.attention_fwd(qkv, att, lse, B, H, S, D, blk.causal)
        x1 = torch.empty(T, h, dtype=bf, device=dev)
        L.gemm(att, blk.proj_w, x1, epilogue=L.EPI_BIAS_RESIDUAL, bias=blk.proj_b, aux=x2)
        h2 = torch.empty(T, h, dtype=bf, device=dev)
        L.layernorm_fwd(x1, blk.ln2_w, blk.ln2_b, h2, mean2, rstd2, blk.eps)
        ffn = blk.fc1_w.shape[0]
        pre = torch.empty(T, ffn, dtype=bf, device=dev)
        act = torch.empty(T, ffn, dtype=bf, device=dev)
        L.gemm(h2, blk.fc1_w, act, epilogue=L.EPI_BIAS_GELU, bias=blk.fc1_b, out2=pre)
        out = torch.empty(T, h, dtype=bf, device=dev)
        L.gemm(act, blk.fc2_w, out, epilogue=L.EPI_BIAS_RESIDUAL, bias=blk.fc2_b, aux=x1)
        ctx.blk, ctx.dims, ctx.shape = blk, (B, S, H, D), shape
        ctx.save_for_backward(x2, h1, qkv, att, lse, x1, h2, pre, act, mean1, rstd1, mean2, rstd2)
        return out.view(shape)

    @staticmethod
    def backward(ctx, dout):
        blk = ctx.blk
        B, S, H, D = ctx.dims
        x2, h1, qkv, att, lse, x1, h2, pre, act, mean1, rstd1, mean2, rstd2 = ctx.saved_tensors
        h = x2.shape[1]
        dev, bf = x2.device, torch.bfloat16
        d2 = dout.reshape(-1, h)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        T = d2.shape[0]
        # MLP: d(pre) = (d2 @ W2) * gelu'(pre) fused in the dgrad epilogue
        wg = []          # the block's four weight gradients go to the side stream in one batch
        dpre = _linear_backward(d2, act, blk.fc2_w, blk.fc2_b, dx_epilogue=L.EPI_MUL_DGELU, aux=pre, defer=wg)
        dh2 = _linear_backward(dpre, h2, blk.fc1_w, blk.fc1_b, defer=wg)
        flush_wgrads(wg)
        wg = []
        dx1 = torch.empty(T, h, dtype=bf, device=dev)
        L.layernorm_bwd(dh2, x1, blk.ln2_w, mean2, rstd2, d2, dx1, _main_grad(blk.ln2_w), _main_grad(blk.ln2_b))
        # attention
        datt = _linear_backward(dx1, att, blk.proj_w, blk.proj_b, defer=wg)
        dqkv = torch.empty_like(qkv)
        L.attention_bwd(qkv, att, datt, lse, dqkv, B, H, S, D, blk.causal)
        dh1 = _linear_backward(dqkv, h1, blk.qkv_w, blk.qkv_b, defer=wg)
        flush_wgrads(wg)
        dx = torch.empty(T, h, dtype=bf, device=dev)
        L.layernorm_bwd(dh1, x2, blk.ln1_w, mean1, rstd1, dx1, dx, _main_grad(blk.ln1_w), _main_grad(blk.ln1_b))
        return (dx.view(ctx.shape), None) + (None,) * 12


class _AttnHalfFn(torch.autograd.Function):
    """First half of a pre-LN block as a layer of its own: x + proj(attention(LN1(x)))."""

    @staticmethod
    def forward(ctx, x, blk, *params):
        _require_cuda(x, "AttentionHalf")
        shape = x.shape
        h = shape[-1]
        x2 = x.reshape(-1, h)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        B, S = (shape[0], shape[1]) if x.dim() == 3 else (1, T)
        H, D = blk.heads, h // blk.heads
        dev, bf, f32 = x.device, torch.bfloat16, torch.float32
        mean1, rstd1 = torch.empty(T, dtype=f32, device=dev), torch.empty(T, dtype=f32, device=dev)
        h1 = torch.empty(T, h, dtype=bf, device=dev)
        L.layernorm_fwd(x2, blk.ln1_w, blk.ln1_b, h1, mean1, rstd1, blk.eps)
        qkv = torch.empty(T, 3 * h, dtype=bf, device=dev)
        L.gemm(h1, blk.qkv_w, qkv, epilogue=L.EPI_BIAS, bias=blk.qkv_b)
        att = torch.empty(T, h, dtype=bf, device=dev)
        lse = torch.empty(B, H, S, dtype=f32, device=dev)
        L.attention_fwd(qkv, att, lse, B, H, S, D, blk.causal)
        x1 = torch.empty(T, h, dtype=bf, device=dev)
        L.gemm(att, blk.proj_w, x1, epilogue=L.EPI_BIAS_RESIDUAL, bias=blk.proj_b, aux=x2)
        ctx.blk, ctx.dims, ctx.shape = blk, (B, S, H, D), shape
        ctx.save_for_backward(x2, h1, qkv, att, lse, mean1, rstd1)
        return x1.view(shape)

    @staticmethod
    def backward(ctx, dout):
        blk = ctx.blk
        B, S, H, D = ctx.dims
        x2, h1, qkv, att, lse, mean1, rstd1 = ctx.saved_tensors
        h = x2.shape[1]
        dx1 = dout.reshape(-1, h)
        if not dx1.is_contiguous():
            dx1 = dx1.contiguous()
        wg = []
        datt = _linear_backward(dx1, att, blk.proj_w, blk.proj_b, defer=wg)
        dqkv = torch.empty_like(qkv)
        L.attention_bwd(qkv, att, datt, lse, dqkv, B, H, S, D, blk.causal)
        dh1 = _linear_backward(dqkv, h1, blk.qkv_w, blk.qkv_b, defer=wg)
        flush_wgrads(wg)
        dx = torch.empty(dx1.shape[0], h, dtype=torch.bfloat16, device=x2.device)
        L.layernorm_bwd(dh1, x2, blk.ln1_w, mean1, rstd1, dx1, dx, _main_grad(blk.ln1_w), _main_grad(blk.ln1_b))
        return (dx.view(ctx.shape), None) + (None,) * 6


class _MLPHalfFn(torch.autograd.Function):
    """Second half of a pre-LN block as a layer of its own: x + fc2(gelu(fc1(LN2(x))))."""

    @staticmethod
    def forward(ctx, x, blk, *params):
        _require_cuda(x, "MLPHalf")
        shape = x.shape
        h = shape[-1]
        x1 = x.reshape(-1, h)
        if not x1.is_contiguous():
            x1 = x1.contiguous()
        T = x1.shape[0]
        dev, bf, f32 = x.device, torch.bfloat16, torch.float32
        mean2, rstd2 = torch.empty(T, dtype=f32, device=dev), torch.empty(T, dtype=f32, device=dev)
        h2 = torch.empty(T, h, dtype=bf, device=dev)
        L.layernorm_fwd(x1, blk.ln2_w, blk.ln2_b, h2, mean2, rstd2, blk.eps)
        ffn = blk.fc1_w.shape[0]
        pre = torch.empty(T, ffn, dtype=bf, device=dev)
        act = torch.empty(T, ffn, dtype=bf, device=dev)
        L.gemm(h2, blk.fc1_w, act, epilogue=L.EPI_BIAS_GELU, bias=blk.fc1_b, out2=pre)
        out = torch.empty(T, h, dtype=bf, device=dev)
        L.gemm(act, blk.fc2_w, out, epilogue=L.EPI_BIAS_RESIDUAL, bias=blk.fc2_b, aux=x1)
        ctx.blk, ctx.shape = blk, shape
        ctx.save_for_backward(x1, h2, pre, act, mean2, rstd2)
        return out.view(shape)

    @staticmethod
    def backward(ctx, dout):
        blk = ctx.blk
        x1, h2, pre, act, mean2, rstd2 = ctx.saved_tensors
        h = x1.shape[1]
        d2 = dout.reshape(-1, h)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        wg = []
        dpre = _linear_backward(d2, act, blk.fc2_w, blk.fc2_b, dx_epilogue=L.EPI_MUL_DGELU, aux=pre, defer=wg)
        dh2 = _linear_backward(dpre, h2, blk.fc1_w, blk.fc1_b, defer=wg)
        flush_wgrads(wg)
        dx1 = torch.empty(d2.shape[0], h, dtype=torch.bfloat16, device=x1.device)
        L.layernorm_bwd(dh2, x1, blk.ln2_w, mean2, rstd2, d2, dx1, _main_grad(blk.ln2_w), _main_grad(blk.ln2_b))
        return (dx1.view(ctx.shape), None) + (None,) * 6


# One foreign call per half block (bb_block_half_fwd / bb_block_half_bwd) instead of one per
# kernel.  False, or an active lib.gemm_hook (per-GEMM timing), selects the per-kernel Functions
# above; both issue the same kernels in the same order.
NATIVE_BLOCKS = True


def _half_desc(mod, half, T, B, S, need_grads):
    """The module's cached bb_block_desc for this geometry; rebuilt when its parameters moved
    (another arena) or the GEMM CTA budget changed."""
    names = ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "proj_w", "proj_b") if half == L.HALF_ATTENTION else \
            ("ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")
    params = [getattr(mod, n) for n in names]
    key = (half, T, B, S, L.GEMM_MAX_CTAS, params[2].data_ptr(), need_grads)
    cache = mod.__dict__.setdefault("_desc_cache", {})
    d = cache.get(key)
    if d is not None:
        return d
    h = params[2].shape[1]
    heads = getattr(mod, "heads", 1)
    d = L.BlockDesc(tokens=T, batch=B, seq=S, heads=heads, head_dim=h // heads, hidden=h,
                    ffn=params[2].shape[0] if half == L.HALF_MLP else 0, causal=int(getattr(mod, "causal", True)),
                    eps=mod.eps, max_ctas=L.GEMM_MAX_CTAS,
                    ln_w=params[0].data_ptr(), ln_b=params[1].data_ptr(), w1=params[2].data_ptr(), b1=params[3].data_ptr(),
                    w2=params[4].data_ptr(), b2=params[5].data_ptr())
    if need_grads:
        g = [_main_grad(p).data_ptr() for p in params]
        d.g_ln_w, d.g_ln_b, d.g_w1, d.g_b1, d.g_w2, d.g_b2 = g
    lib = L.load()
    d._saved_bytes = lib.bb_block_saved_bytes(ctypes.byref(d), half)
    d._scratch_bytes = lib.bb_block_scratch_bytes(ctypes.byref(d), half)
    if d._saved_bytes < 0:
        raise L.BambooNativeError("bb_block_saved_bytes rejected the block geometry")
    if len(cache) > 16:
        cache.clear()
    cache[key] = d
    return d


class _HalfFn(torch.autograd.Function):
    """Half a pre-LN block through one native call each way: x + proj(attention(LN1(x))) or
    x + fc2(gelu(fc1(LN2(x))))."""

    @staticmethod
    def forward(ctx, x, mod, half, *params):
        _require_cuda(x, "transformer block")
        shape = x.shape
        h = shape[-1]
        x2 = x.reshape(-1, h)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        B, S = (shape[0], shape[1]) if x.dim() == 3 else (1, T)
        d = _half_desc(mod, half, T, B, S, False)
        saved = torch.empty(d._saved_bytes, dtype=torch.uint8, device=x.device)
        out = torch.empty(T, h, dtype=torch.bfloat16, device=x.device)
        L.block_half_fwd(d, half, x2, saved, out)
        ctx.mod, ctx.half, ctx.geom, ctx.shape = mod, half, (T, B, S), shape
        ctx.save_for_backward(x2, saved)
        return out.view(shape)

    @staticmethod
    def backward(ctx, dout):
        x2, saved = ctx.saved_tensors
        T, B, S = ctx.geom
        h = x2.shape[1]
        d2 = dout.reshape(-1, h)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        d = _half_desc(ctx.mod, ctx.half, T, B, S, True)
        scratch = torch.empty(d._scratch_bytes, dtype=torch.uint8, device=x2.device)
        dx = torch.empty(T, h, dtype=torch.bfloat16, device=x2.device)
        side = None
        if WGRAD_SIDE_STREAM:
            st = _wgrad_stream(x2.device)
            side = st.cuda_stream
            # operands of the weight-gradient kernels: not to be handed out again before that stream is done
            for t in (d2, saved, scratch):
                t.record_stream(st)
        L.block_half_bwd(d, ctx.half, x2, saved, d2, dx, scratch, side)
        return (dx.view(ctx.shape), None, None) + (None,) * 6


def _use_native_blocks():
    return NATIVE_BLOCKS and L.gemm_hook is None


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, tokens, mod, wte, wpe):
        _require_cuda(tokens, "TokenEmbedding")
        B, S = tokens.shape
        tok = tokens.contiguous()
        out = torch.empty(B * S, wte.shape[1], dtype=torch.bfloat16, device=tokens.device)
        L.embedding_fwd(tok, wte, wpe, out, S)
        ctx.mod, ctx.S = mod, S
        ctx.save_for_backward(tok)
        return out.view(B, S, -1)

    @staticmethod
    def backward(ctx, dout):
        (tok,) = ctx.saved_tensors
        mod = ctx.mod
        d2 = dout.reshape(-1, dout.shape[-1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        L.embedding_bwd(tok, d2, _main_grad(mod.wte), _main_grad(mod.wpe), ctx.S)
        return None, None, None, None


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mod, w, b):
        _require_cuda(x, "LayerNorm")
        h = x.shape[-1]
        x2 = x.reshape(-1, h)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        mean = torch.empty(T, dtype=torch.float32, device=x.device)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        y = torch.empty_like(x2)
        L.layernorm_fwd(x2, w, b, y, mean, rstd, mod.eps)
        ctx.mod, ctx.shape = mod, x.shape
        ctx.save_for_backward(x2, mean, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, mean, rstd = ctx.saved_tensors
        mod = ctx.mod
        d2 = dy.reshape(-1, x2.shape[1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dx = torch.empty_like(x2)
        L.layernorm_bwd(d2, x2, mod.weight, mean, rstd, None, dx, _main_grad(mod.weight), _main_grad(mod.bias))
        return dx.view(ctx.shape), None, None, None


class _LinearFn(torch.autograd.Function):
    """y = x @ W^T (+ b); W may be row-padded (only ``mod.out_features`` rows are real)."""

    @staticmethod
    def forward(ctx, x, mod, w, b):
        _require_cuda(x, "Linear")
        k = x.shape[-1]
        x2 = x.reshape(-1, k)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = torch.empty(x2.shape[0], w.shape[0], dtype=torch.bfloat16, device=x.device)
        L.gemm(x2, w, y, epilogue=L.EPI_BIAS if b is not None else L.EPI_STORE, bias=b)
        ctx.mod, ctx.shape = mod, x.shape
        ctx.save_for_backward(x2)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        mod = ctx.mod
        d2 = dy.reshape(-1, dy.shape[-1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dx = _linear_backward(d2, x2, mod.weight, mod.bias)
        return dx.view(ctx.shape), None, None, None


class _MLMTransformFn(torch.autograd.Function):
    """y = LayerNorm(gelu(x W^T + b)): the masked-LM head transform.  Forward: one GEMM with the
    bias+GeLU epilogue (keeps the pre-activation) and a LayerNorm; backward: LayerNorm backward,
    stand-alone GeLU backward, then the usual input / weight gradients."""

    @staticmethod
    def forward(ctx, x, mod, w, b, ln_w, ln_b):
        _require_cuda(x, "MLMTransform")
        h = x.shape[-1]
        x2 = x.reshape(-1, h)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T, dev = x2.shape[0], x.device
        pre = torch.empty(T, h, dtype=torch.bfloat16, device=dev)
        act = torch.empty(T, h, dtype=torch.bfloat16, device=dev)
        L.gemm(x2, w, act, epilogue=L.EPI_BIAS_GELU, bias=b, out2=pre)
        mean = torch.empty(T, dtype=torch.float32, device=dev)
        rstd = torch.empty(T, dtype=torch.float32, device=dev)
        y = torch.empty(T, h, dtype=torch.bfloat16, device=dev)
        L.layernorm_fwd(act, ln_w, ln_b, y, mean, rstd, mod.eps)
        ctx.mod, ctx.shape = mod, x.shape
        ctx.save_for_backward(x2, pre, act, mean, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, pre, act, mean, rstd = ctx.saved_tensors
        mod = ctx.mod
        d2 = dy.reshape(-1, x2.shape[1])
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dact = torch.empty_like(act)
        L.layernorm_bwd(d2, act, mod.ln_weight, mean, rstd, None, dact, _main_grad(mod.ln_weight), _main_grad(mod.ln_bias))
        dpre = torch.empty_like(pre)
        L.gelu_bwd(dact, pre, dpre)
        dx = _linear_backward(dpre, x2, mod.weight, mod.bias)
        return dx.view(ctx.shape), None, None, None, None, None


class _CrossEntropyFn(torch.autograd.Function):
    """Mean token cross entropy; the gradient overwrites the logits buffer in place."""

    @staticmethod
    def forward(ctx, logits, targets, vocab, ignore_index):
        _require_cuda(logits, "cross_entropy")
        cols = logits.shape[-1]
        lg = logits.reshape(-1, cols)
        tg = targets.reshape(-1).contiguous()
        rows = lg.shape[0]
        dev = logits.device
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        row_loss = torch.empty(rows, dtype=torch.float32, device=dev)
        loss_out = torch.empty(2, dtype=torch.float32, device=dev)
        L.cross_entropy_fwd(lg, tg, lse, row_loss, loss_out, vocab, ignore_index)
        ctx.vocab, ctx.ignore_index, ctx.shape = vocab, ignore_index, logits.shape
        ctx.save_for_backward(lg, tg, lse, loss_out)
        return loss_out[0].clone()

    @staticmethod
    def backward(ctx, gloss):
        lg, tg, lse, loss_out = ctx.saved_tensors
        g = gloss.reshape(1).to(torch.float32).contiguous()
        L.cross_entropy_bwd(lg, tg, lse, loss_out, lg, ctx.vocab, grad_scale=1.0, grad_scale_dev=g,
                            ignore_index=ctx.ignore_index)
        return lg.view(ctx.shape), None, None, None


# ----------------------------------------------------------------------------------- modules
def _normal(shape, gen, std=0.02):
    return torch.randn(shape, generator=gen, dtype=torch.float32) * std


class TokenEmbedding(nn.Module):
    """tokens [B,S] int64 -> [B,S,h]: token embedding + learned position embedding."""

    def __init__(self, vocab, hidden, max_seq, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.wte = nn.Parameter(_normal((vocab, hidden), g))
        self.wpe = nn.Parameter(_normal((max_seq, hidden), g))

    def forward(self, tokens):
        return _EmbeddingFn.apply(tokens, self, self.wte, self.wpe)


class TransformerBlock(nn.Module):
    """Pre-LayerNorm block: multi-head attention (causal or bidirectional) and a 4x GeLU MLP."""

    def __init__(self, hidden, heads, ffn, causal=True, eps=1e-5, seed=0):
        super().__init__()
        assert hidden % heads == 0
        g = torch.Generator().manual_seed(seed)
        self.heads, self.causal, self.eps = heads, causal, eps
        self.ln1_w = nn.Parameter(torch.ones(hidden)); self.ln1_b = nn.Parameter(torch.zeros(hidden))
        self.qkv_w = nn.Parameter(_normal((3 * hidden, hidden), g)); self.qkv_b = nn.Parameter(torch.zeros(3 * hidden))
        self.proj_w = nn.Parameter(_normal((hidden, hidden), g)); self.proj_b = nn.Parameter(torch.zeros(hidden))
        self.ln2_w = nn.Parameter(torch.ones(hidden)); self.ln2_b = nn.Parameter(torch.zeros(hidden))
        self.fc1_w = nn.Parameter(_normal((ffn, hidden), g)); self.fc1_b = nn.Parameter(torch.zeros(ffn))
        self.fc2_w = nn.Parameter(_normal((hidden, ffn), g)); self.fc2_b = nn.Parameter(torch.zeros(hidden))

    def forward(self, x):
        if _use_native_blocks():
            x1 = _HalfFn.apply(x, self, L.HALF_ATTENTION, self.ln1_w, self.ln1_b, self.qkv_w, self.qkv_b, self.proj_w,
                               self.proj_b)
            return _HalfFn.apply(x1, self, L.HALF_MLP, self.ln2_w, self.ln2_b, self.fc1_w, self.fc1_b, self.fc2_w,
                                 self.fc2_b)
        return _BlockFn.apply(x, self, self.ln1_w, self.ln1_b, self.qkv_w, self.qkv_b, self.proj_w, self.proj_b,
                              self.ln2_w, self.ln2_b, self.fc1_w, self.fc1_b, self.fc2_w, self.fc2_b)


class AttentionHalf(nn.Module):
    """The attention half of a ``TransformerBlock`` as its own pipeline layer (finer stage
    boundaries); with ``MLPHalf(..., seed=same)`` after it the pair equals the fused block,
    weights included: both draw from ``Generator(seed)`` in the block's order qkv, proj, fc1, fc2."""

    def __init__(self, hidden, heads, ffn, causal=True, eps=1e-5, seed=0):
        super().__init__()
        assert hidden % heads == 0
        g = torch.Generator().manual_seed(seed)
        self.heads, self.causal, self.eps = heads, causal, eps
        self.ln1_w = nn.Parameter(torch.ones(hidden)); self.ln1_b = nn.Parameter(torch.zeros(hidden))
        self.qkv_w = nn.Parameter(_normal((3 * hidden, hidden), g)); self.qkv_b = nn.Parameter(torch.zeros(3 * hidden))
        self.proj_w = nn.Parameter(_normal((hidden, hidden), g)); self.proj_b = nn.Parameter(torch.zeros(hidden))

    def forward(self, x):
        if _use_native_blocks():
            return _HalfFn.apply(x, self, L.HALF_ATTENTION, self.ln1_w, self.ln1_b, self.qkv_w, self.qkv_b, self.proj_w,
                                 self.proj_b)
        return _AttnHalfFn.apply(x, self, self.ln1_w, self.ln1_b, self.qkv_w, self.qkv_b, self.proj_w, self.proj_b)


class MLPHalf(nn.Module):
    """The MLP half of a ``TransformerBlock`` as its own pipeline layer; see ``AttentionHalf``."""

    def __init__(self, hidden, heads, ffn, causal=True, eps=1e-5, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        _normal((3 * hidden, hidden), g); _normal((hidden, hidden), g)      # the attention half's draws
        self.eps = eps
        self.ln2_w = nn.Parameter(torch.ones(hidden)); self.ln2_b = nn.Parameter(torch.zeros(hidden))
        self.fc1_w = nn.Parameter(_normal((ffn, hidden), g)); self.fc1_b = nn.Parameter(torch.zeros(ffn))
        self.fc2_w = nn.Parameter(_normal((hidden, ffn), g)); self.fc2_b = nn.Parameter(torch.zeros(hidden))

    def forward(self, x):
        if _use_native_blocks():
            return _HalfFn.apply(x, self, L.HALF_MLP, self.ln2_w, self.ln2_b, self.fc1_w, self.fc1_b, self.fc2_w, self.fc2_b)
        return _MLPHalfFn.apply(x, self, self.ln2_w, self.ln2_b, self.fc1_w, self.fc1_b, self.fc2_w, self.fc2_b)


class LayerNorm(nn.Module):
    def __init__(self, hidden, eps=1e-5):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden)); self.bias = nn.Parameter(torch.zeros(hidden))

    def forward(self, x):
        return _LayerNormFn.apply(x, self, self.weight, self.bias)


class Linear(nn.Module):
    """y = x W^T + b.  ``pad_to`` rounds the stored output rows up (zero rows) so that a
    vocabulary projection satisfies the kernels' 8-element leading-dimension rule."""

    def __init__(self, in_features, out_features, bias=True, pad_to=1, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.in_features, self.out_features = in_features, out_features
        rows = (out_features + pad_to - 1) // pad_to * pad_to
        w = torch.zeros(rows, in_features)
        w[:out_features] = _normal((out_features, in_features), g)
        self.weight = nn.Parameter(w)
        self.bias = nn.Parameter(torch.zeros(rows)) if bias else None

    def forward(self, x):
        return _LinearFn.apply(x, self, self.weight, self.bias)


class MLMTransform(nn.Module):
    """Masked-LM head transform: dense (hidden -> hidden) + tanh-GeLU + LayerNorm; the vocabulary
    decoder is the ``Linear`` that follows it in the layer list."""

    def __init__(self, hidden, eps=1e-5, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.eps = eps
        self.weight = nn.Parameter(_normal((hidden, hidden), g))
        self.bias = nn.Parameter(torch.zeros(hidden))
        self.ln_weight = nn.Parameter(torch.ones(hidden)); self.ln_bias = nn.Parameter(torch.zeros(hidden))

    def forward(self, x):
        return _MLMTransformFn.apply(x, self, self.weight, self.bias, self.ln_weight, self.ln_bias)


class CrossEntropyLoss:
    """``loss_fn(logits, labels)`` for the last stage: mean CE over labels != ignore_index.
    ``vocab`` is the number of real logit columns (the rest is padding)."""

    def __init__(self, vocab, ignore_index=-100):
        self.vocab, self.ignore_index = vocab, ignore_index

    def __call__(self, logits, labels):
        return _CrossEntropyFn.apply(logits, labels, self.vocab, self.ignore_index)
