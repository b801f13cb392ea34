"""ResNet-152 stage layers (bottleneck blocks [3, 8, 36, 3]) in channels-last bf16 on the sm_100a
kernels, as a ``PipelineModule`` layer list.

The reference pipelines torchvision's ``resnet152`` split by ``join_resnet_layers``
(``DeepSpeedExamples/osdi22-cv/resnet-exp.py:69-83``: conv1, bn1, relu, maxpool, the 50 bottleneck
blocks, avgpool, flatten, fc).  Here the list is ``ResNetStem`` (conv1 + bn1 + relu + maxpool),
50 x ``Bottleneck``, ``ResNetHead`` (avgpool + flatten + fc): the same boundaries between blocks,
with the stem's four and the head's three entries each fused into one layer.

Every convolution is the library's tcgen05 GEMM over a patch matrix (rows = output pixels,
columns = taps x input channels; a 1 x 1 / stride 1 convolution reads the activation tensor
itself), followed by batch norm with batch statistics, the residual add and ReLU in one
element-wise pass.  Weights are stored ``[Cout, k, k, Cin]`` (flattened to 2-D), activations
``[N, H, W, C]``; channel counts are multiples of 8, so the 3-channel input is carried in 8
channels with five zero planes.  Batch-norm running statistics are not kept: they do not enter a
training step.

There is no fallback: these modules raise on CPU tensors.
"""
import ctypes
import math

import torch
from torch import nn

from . import lib as L
from .layers import CrossEntropyLoss, Linear, _main_grad, _require_cuda
from .module import LayerSpec

IN_CHANNELS = 8            # 3 image channels + 5 zero planes (16-byte channel vectors)


def _conv_desc(mod, N, H, W, Cin, need_grads):
    """The layer's cached bb_conv_desc for this input geometry (rebuilt when its parameters moved)."""
    key = (N, H, W, L.GEMM_MAX_CTAS, mod.weight.data_ptr(), need_grads)
    cache = mod.__dict__.setdefault("_desc_cache", {})
    d = cache.get(key)
    if d is not None:
        return d
    d = L.ConvDesc(N=N, H=H, W=W, Cin=Cin, Cout=mod.weight.shape[0], k=mod.k, stride=mod.stride, pad=mod.pad,
                   relu=int(mod.relu), eps=mod.eps, max_ctas=L.GEMM_MAX_CTAS,
                   w=mod.weight.data_ptr(), gamma=mod.bn_weight.data_ptr(), beta=mod.bn_bias.data_ptr())
    if need_grads:
        d.g_w, d.g_gamma, d.g_beta = (_main_grad(p).data_ptr() for p in (mod.weight, mod.bn_weight, mod.bn_bias))
    lib = L.load()
    d._fwd_scratch = lib.bb_conv_bn_scratch_bytes(ctypes.byref(d), 0, 0)
    d._bwd_scratch = (lib.bb_conv_bn_scratch_bytes(ctypes.byref(d), 1, 0), lib.bb_conv_bn_scratch_bytes(ctypes.byref(d), 1, 1))
    if d._fwd_scratch < 0:
        raise L.BambooNativeError("bb_conv_bn_scratch_bytes rejected the layer geometry "
                                  "(channels: multiples of 8; batch norm: 8 x a power of two <= 2048)")
    if len(cache) > 8:
        cache.clear()
    cache[key] = d
    return d


class _ConvBNNativeFn(torch.autograd.Function):
    """z = [relu]( batchnorm(conv(x)) [+ residual] ) through one native call each way."""

    @staticmethod
    def forward(ctx, x, residual, mod, w, gamma, beta):
        _require_cuda(x, "ConvBN")
        if not x.is_contiguous():
            x = x.contiguous()
        N, H, W, Cin = x.shape
        Ho, Wo = (H + 2 * mod.pad - mod.k) // mod.stride + 1, (W + 2 * mod.pad - mod.k) // mod.stride + 1
        P, Cout = N * Ho * Wo, w.shape[0]
        dev = x.device
        d = _conv_desc(mod, N, H, W, Cin, False)
        y = torch.empty(P, Cout, dtype=torch.bfloat16, device=dev)
        z = torch.empty(N, Ho, Wo, Cout, dtype=torch.bfloat16, device=dev)
        stats = torch.empty(2, Cout, dtype=torch.float32, device=dev)
        scratch = torch.empty(max(d._fwd_scratch, 16), dtype=torch.uint8, device=dev)
        if residual is not None and not residual.is_contiguous():
            residual = residual.contiguous()
        L.conv_bn_fwd(d, x, residual, y, z, stats[0], stats[1], scratch)
        ctx.mod, ctx.geom, ctx.has_res = mod, (N, H, W, Cin), residual is not None
        ctx.save_for_backward(x, y, z, stats)
        return z

    @staticmethod
    def backward(ctx, dz):
        x, y, z, stats = ctx.saved_tensors
        mod = ctx.mod
        N, H, W, Cin = ctx.geom
        dev = x.device
        if not dz.is_contiguous():
            dz = dz.contiguous()
        need_dx = ctx.needs_input_grad[0]
        d = _conv_desc(mod, N, H, W, Cin, True)
        dx = torch.empty(N, H, W, Cin, dtype=torch.bfloat16, device=dev) if need_dx else None
        dres = torch.empty_like(z) if ctx.has_res else None
        scratch = torch.empty(d._bwd_scratch[1 if need_dx else 0], dtype=torch.uint8, device=dev)
        L.conv_bn_bwd(d, x, y, z, stats[0], stats[1], dz, dx, dres, scratch)
        return dx, dres, None, None, None, None


# One foreign call per layer and direction (False, or an active lib.gemm_hook: one call per kernel)
NATIVE_LAYERS = True


class _ConvBNFn(torch.autograd.Function):
    """z = [relu]( batchnorm(conv(x)) [+ residual] )"""

    @staticmethod
    def forward(ctx, x, residual, mod, w, gamma, beta):
        _require_cuda(x, "ConvBN")
        if not x.is_contiguous():
            x = x.contiguous()
        N, H, W, Cin = x.shape
        k, s, pad = mod.k, mod.stride, mod.pad
        Ho, Wo = (H + 2 * pad - k) // s + 1, (W + 2 * pad - k) // s + 1
        P, Cout = N * Ho * Wo, w.shape[0]
        dev, bf = x.device, torch.bfloat16
        col = mod.patches(x, Ho, Wo)
        y = torch.empty(P, Cout, dtype=bf, device=dev)
        L.gemm(col, w, y)
        mean = torch.empty(Cout, dtype=torch.float32, device=dev)
        rstd = torch.empty(Cout, dtype=torch.float32, device=dev)
        L.bn_stats(y, mean, rstd, mod.eps)
        z = torch.empty(P, Cout, dtype=bf, device=dev)
        res2d = None
        if residual is not None:
            res2d = residual.reshape(P, Cout)
            if not res2d.is_contiguous():
                res2d = res2d.contiguous()
        L.bn_apply(y, mean, rstd, gamma, beta, res2d, z, mod.relu)
        ctx.mod, ctx.geom, ctx.has_res = mod, (N, H, W, Cin, Ho, Wo), residual is not None
        ctx.save_for_backward(x, y, z, mean, rstd)
        return z.view(N, Ho, Wo, Cout)

    @staticmethod
    def backward(ctx, dz):
        x, y, z, mean, rstd = ctx.saved_tensors
        mod = ctx.mod
        N, H, W, Cin, Ho, Wo = ctx.geom
        P, Cout = y.shape
        K = mod.k * mod.k * Cin
        dev, bf = x.device, torch.bfloat16
        dz2 = dz.reshape(P, Cout)
        if not dz2.is_contiguous():
            dz2 = dz2.contiguous()
        dy = torch.empty(P, Cout, dtype=bf, device=dev)
        dres = torch.empty(P, Cout, dtype=bf, device=dev) if ctx.has_res else None
        L.bn_bwd(dz2, z, y, mean, rstd, mod.bn_weight, dy, dres, _main_grad(mod.bn_weight), _main_grad(mod.bn_bias), mod.relu)
        # weight gradient: dW[Cout, K] += dy^T patches (the patch matrix is gathered again, not kept)
        col = mod.patches(x, Ho, Wo)
        L.gemm(dy, col, _main_grad(mod.weight), a_mn=True, b_mn=True, epilogue=L.EPI_ACCUM_F32, M=Cout, N=K, K=P)
        dx = None
        if ctx.needs_input_grad[0]:
            dcol = torch.empty(P, K, dtype=bf, device=dev)
            L.gemm(dy, mod.weight, dcol, b_mn=True, M=P, N=K, K=Cout)
            if mod.k == 1 and mod.stride == 1:
                dx = dcol.view(N, H, W, Cin)
            else:
                dx = torch.empty(N, H, W, Cin, dtype=bf, device=dev)
                L.col2im(dcol, dx, mod.k, mod.stride, mod.pad, Ho, Wo)
        return dx, (dres.view(N, Ho, Wo, Cout) if dres is not None else None), None, None, None, None


class ConvBN(nn.Module):
    """k x k convolution (no bias) + batch norm (batch statistics, affine) [+ residual] [+ ReLU]."""

    def __init__(self, cin, cout, k, stride=1, relu=True, eps=1e-5, generator=None):
        super().__init__()
        assert cin % 8 == 0 and cout % 8 == 0
        self.k, self.stride, self.pad, self.relu, self.eps = k, stride, (k - 1) // 2, relu, eps
        # Kaiming normal, fan_out (torchvision's initialisation of ResNet convolutions)
        std = math.sqrt(2.0 / (cout * k * k))
        w = torch.randn(cout, k, k, cin, generator=generator, dtype=torch.float32) * std
        self.weight = nn.Parameter(w.reshape(cout, k * k * cin))
        self.bn_weight = nn.Parameter(torch.ones(cout))
        self.bn_bias = nn.Parameter(torch.zeros(cout))

    def patches(self, x, Ho, Wo):
        N, H, W, C = x.shape
        if self.k == 1 and self.stride == 1:
            return x.view(N * H * W, C)
        col = torch.empty(N * Ho * Wo, self.k * self.k * C, dtype=torch.bfloat16, device=x.device)
        return L.im2col(x, col, self.k, self.stride, self.pad, Ho, Wo)

    def forward(self, x, residual=None):
        fn = _ConvBNNativeFn if (NATIVE_LAYERS and L.gemm_hook is None) else _ConvBNFn
        return fn.apply(x, residual, self, self.weight, self.bn_weight, self.bn_bias)


class _MaxPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        _require_cuda(x, "max pooling")
        if not x.is_contiguous():
            x = x.contiguous()
        N, H, W, C = x.shape
        Ho, Wo = (H - 1) // 2 + 1, (W - 1) // 2 + 1
        y = torch.empty(N, Ho, Wo, C, dtype=x.dtype, device=x.device)
        arg = torch.empty(N, Ho, Wo, C, dtype=torch.uint8, device=x.device)
        L.maxpool_fwd(x, y, arg)
        ctx.shape = (N, H, W, C)
        ctx.save_for_backward(arg)
        return y

    @staticmethod
    def backward(ctx, dy):
        (arg,) = ctx.saved_tensors
        dx = torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        L.maxpool_bwd(dy.contiguous(), arg, dx)
        return dx


class _AvgPoolFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        _require_cuda(x, "average pooling")
        if not x.is_contiguous():
            x = x.contiguous()
        N, H, W, C = x.shape
        y = torch.empty(N, C, dtype=x.dtype, device=x.device)
        L.avgpool_fwd(x, y)
        ctx.shape = (N, H, W, C)
        return y

    @staticmethod
    def backward(ctx, dy):
        dx = torch.empty(ctx.shape, dtype=dy.dtype, device=dy.device)
        L.avgpool_bwd(dy.contiguous(), dx)
        return dx


class ResNetStem(nn.Module):
    """7 x 7 / stride 2 convolution + batch norm + ReLU + 3 x 3 / stride 2 max pooling."""

    def __init__(self, width=64, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.conv = ConvBN(IN_CHANNELS, width, 7, stride=2, relu=True, generator=g)

    def forward(self, x):
        return _MaxPoolFn.apply(self.conv(x))


class Bottleneck(nn.Module):
    """1 x 1 -> 3 x 3 (carries the stride) -> 1 x 1 (x 4 channels), identity or projected shortcut."""
    expansion = 4

    def __init__(self, cin, mid, stride=1, downsample=False, seed=0):
        super().__init__()
        g = torch.Generator().manual_seed(seed)
        self.conv1 = ConvBN(cin, mid, 1, relu=True, generator=g)
        self.conv2 = ConvBN(mid, mid, 3, stride=stride, relu=True, generator=g)
        self.conv3 = ConvBN(mid, mid * 4, 1, relu=True, generator=g)          # ReLU after the residual add
        self.down = ConvBN(cin, mid * 4, 1, stride=stride, relu=False, generator=g) if downsample else None

    def forward(self, x):
        identity = self.down(x) if self.down is not None else x
        return self.conv3(self.conv2(self.conv1(x)), residual=identity)


class ResNetHead(nn.Module):
    """Global average pooling, flatten, fully connected classifier."""

    def __init__(self, cin, classes, seed=0):
        super().__init__()
        self.fc = Linear(cin, classes, bias=True, pad_to=8, seed=seed)

    def forward(self, x):
        return self.fc(_AvgPoolFn.apply(x))


def resnet_layer_specs(blocks=(3, 8, 36, 3), classes=1000, width=64, seed=0):
    """Layer list of a bottleneck ResNet: ``blocks`` = (3, 8, 36, 3) is ResNet-152.  Layer ``i``
    draws its weights from ``Generator(seed * 1000 + i)`` in definition order, so a stage or its
    shadow copy built on any rank holds identical values."""
    base = seed * 1000
    specs = [LayerSpec(ResNetStem, width, seed=base)]
    cin, i = width, 1
    for stage, n in enumerate(blocks):
        mid = width * (2 ** stage)
        for b in range(n):
            stride = 2 if (b == 0 and stage > 0) else 1
            specs.append(LayerSpec(Bottleneck, cin, mid, stride=stride, downsample=(b == 0), seed=base + i))
            cin, i = mid * 4, i + 1
    specs.append(LayerSpec(ResNetHead, cin, classes, seed=base + i))
    return specs


def resnet_loss(classes=1000):
    return CrossEntropyLoss(classes)


def conv_flops_per_image(blocks=(3, 8, 36, 3), size=224, classes=1000, width=64):
    """Forward multiply-add FLOPs (2 x MACs) of one image: every convolution 2 Cin Cout k^2 Ho Wo
    with the real 3 input channels, plus the classifier."""
    def out(n, k, s):
        return (n + 2 * ((k - 1) // 2) - k) // s + 1
    total = 0
    hw = out(size, 7, 2)
    total += 2 * 3 * width * 49 * hw * hw
    hw = out(hw, 3, 2)
    cin = width
    for stage, n in enumerate(blocks):
        mid = width * (2 ** stage)
        for b in range(n):
            stride = 2 if (b == 0 and stage > 0) else 1
            total += 2 * cin * mid * hw * hw
            ho = out(hw, 3, stride)
            total += 2 * mid * mid * 9 * ho * ho + 2 * mid * mid * 4 * ho * ho
            if b == 0:
                total += 2 * cin * mid * 4 * ho * ho
            hw, cin = ho, mid * 4
    return total + 2 * cin * classes
