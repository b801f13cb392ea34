"""ctypes binding of libbamboo_b200.so (the C ABI declared in include/bamboo_b200.h).

There is no Python or CPU fallback behind these calls: if the shared library is missing
or a call fails, an exception is raised.
"""
import ctypes
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbamboo_b200.so")

STATUS_PEER_TIMEOUT, STATUS_KERNEL_WAIT_TIMEOUT = 1, 2
EPI_STORE, EPI_BIAS, EPI_BIAS_GELU, EPI_ACCUM_F32, EPI_STORE_F32, EPI_MUL_DGELU, EPI_BIAS_RESIDUAL = range(7)


class BambooNativeError(RuntimeError):
    """A native entry point returned a negative status."""


class GemmDesc(ctypes.Structure):
    _fields_ = [
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
        ("A", ctypes.c_void_p), ("lda", ctypes.c_longlong), ("a_mn_major", ctypes.c_int),
        ("B", ctypes.c_void_p), ("ldb", ctypes.c_longlong), ("b_mn_major", ctypes.c_int),
        ("D", ctypes.c_void_p), ("ldd", ctypes.c_longlong),
        ("epilogue", ctypes.c_int),
        ("bias", ctypes.c_void_p),
        ("D2", ctypes.c_void_p),
        ("aux", ctypes.c_void_p), ("ld_aux", ctypes.c_longlong),
        ("tile_n", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
        ("split_k", ctypes.c_int),
        ("cta_pair", ctypes.c_int),
        ("epi_warps", ctypes.c_int),
    ]


class BlockDesc(ctypes.Structure):
    """bb_block_desc: one half of a transformer block (see include/bamboo_b200.h)."""
    _fields_ = [
        ("tokens", ctypes.c_int), ("batch", ctypes.c_int), ("seq", ctypes.c_int), ("heads", ctypes.c_int),
        ("head_dim", ctypes.c_int), ("hidden", ctypes.c_int), ("ffn", ctypes.c_int), ("causal", ctypes.c_int),
        ("eps", ctypes.c_float), ("max_ctas", ctypes.c_int),
        ("ln_w", ctypes.c_void_p), ("ln_b", ctypes.c_void_p), ("w1", ctypes.c_void_p), ("b1", ctypes.c_void_p),
        ("w2", ctypes.c_void_p), ("b2", ctypes.c_void_p),
        ("g_ln_w", ctypes.c_void_p), ("g_ln_b", ctypes.c_void_p), ("g_w1", ctypes.c_void_p), ("g_b1", ctypes.c_void_p),
        ("g_w2", ctypes.c_void_p), ("g_b2", ctypes.c_void_p),
    ]


class ConvDesc(ctypes.Structure):
    """bb_conv_desc: convolution + batch norm layer (see include/bamboo_b200.h)."""
    _fields_ = [
        ("N", ctypes.c_int), ("H", ctypes.c_int), ("W", ctypes.c_int), ("Cin", ctypes.c_int), ("Cout", ctypes.c_int),
        ("k", ctypes.c_int), ("stride", ctypes.c_int), ("pad", ctypes.c_int), ("relu", ctypes.c_int),
        ("eps", ctypes.c_float), ("max_ctas", ctypes.c_int),
        ("w", ctypes.c_void_p), ("gamma", ctypes.c_void_p), ("beta", ctypes.c_void_p),
        ("g_w", ctypes.c_void_p), ("g_gamma", ctypes.c_void_p), ("g_beta", ctypes.c_void_p),
    ]


HALF_ATTENTION, HALF_MLP = 0, 1
# kernels behind one call of bb_block_half_fwd / bb_block_half_bwd, per half (launch accounting)
HALF_FWD_LAUNCHES = {HALF_ATTENTION: 4, HALF_MLP: 3}
HALF_BWD_LAUNCHES = {HALF_ATTENTION: 10, HALF_MLP: 7}   # attention backward: three launches for either head dimension

_lib = None
_lock = threading.Lock()
# number of kernels launched through this binding (benchmarks report it)
LAUNCHES = 0
# optional hook called as hook(name, flops, launch_fn) around GEMM launches (profiling only)
gemm_hook = None


def load():
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise BambooNativeError(
                f"{LIB_PATH} is missing: build it with `python -m bamboo_b200.csrc.build` "
                "(there is no fallback path)")
        lib = ctypes.CDLL(LIB_PATH)
        lib.bb_last_error.restype = ctypes.c_char_p
        lib.bb_version.restype = ctypes.c_int
        lib.bb_block_saved_bytes.restype = ctypes.c_longlong
        lib.bb_block_scratch_bytes.restype = ctypes.c_longlong
        lib.bb_conv_bn_scratch_bytes.restype = ctypes.c_longlong
        _lib = lib
    return _lib


def check(rc, what=""):
    if rc < 0:
        msg = load().bb_last_error().decode(errors="replace")
        raise BambooNativeError(f"{what} failed with status {rc}: {msg}")
    return rc


def read_status():
    """Synchronously read-and-clear the device status word (0 = healthy)."""
    out = ctypes.c_int(0)
    check(load().bb_read_status(ctypes.byref(out)), "bb_read_status")
    return out.value


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream(raw=None):
    """cudaStream_t of the current stream of the current device (or the given raw handle).  The
    raw getter is a single C call; `torch.cuda.current_stream()` builds a Stream object through
    several Python layers and showed up as a third of the host time per step."""
    if raw is not None:
        return ctypes.c_void_p(raw)
    import torch
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice()))


# Process-wide default for GemmDesc.cta_pair (0 = library heuristic, 1 = pairs, -1 = single CTAs);
# BB_GEMM_CTA_PAIR in the environment sets it, for A/B measurements of the two kernels.
GEMM_CTA_PAIR = int(os.environ.get("BB_GEMM_CTA_PAIR", "0"))
GEMM_EPI_WARPS = int(os.environ.get("BB_GEMM_EPI_WARPS", "0"))      # same for GemmDesc.epi_warps (0, 2 or 4)


# Default for GemmDesc.max_ctas; the engine sets it to -1 (one tile per CTA) while it issues
# redundant computation on the low-priority stream and back to 0 afterwards.
GEMM_MAX_CTAS = 0


def gemm(a, b, out, *, a_mn=False, b_mn=False, epilogue=EPI_STORE, bias=None, out2=None, aux=None,
         M=None, N=None, K=None, tile_n=0, max_ctas=0, split_k=0, cta_pair=0, epi_warps=0, stream=None):
    """out[M,N] = op(a)[M,K] @ op(b)[N,K]^T with a fused epilogue; see bb_gemm_bf16.

    ``a`` is [M,K] (or [K,M] when ``a_mn``), ``b`` is [N,K] (or [K,N] when ``b_mn``); 2-D,
    unit inner stride, bf16, on the current CUDA device.
    """
    if M is None:
        M = a.shape[1] if a_mn else a.shape[0]
    if K is None:
        K = a.shape[0] if a_mn else a.shape[1]
    if N is None:
        N = b.shape[1] if b_mn else b.shape[0]
    for t in (a, b, out, bias, out2, aux):
        if t is not None and (not t.is_cuda or t.stride(-1) != 1):
            raise BambooNativeError("gemm operands must be CUDA tensors with unit inner stride")
    d = GemmDesc(M=M, N=N, K=K, A=a.data_ptr(), lda=a.stride(0), a_mn_major=int(a_mn),
                 B=b.data_ptr(), ldb=b.stride(0), b_mn_major=int(b_mn), D=out.data_ptr(), ldd=out.stride(0),
                 epilogue=epilogue, bias=None if bias is None else bias.data_ptr(),
                 D2=None if out2 is None else out2.data_ptr(), aux=None if aux is None else aux.data_ptr(),
                 ld_aux=aux.stride(0) if aux is not None else 0, tile_n=tile_n, max_ctas=max_ctas or GEMM_MAX_CTAS, split_k=split_k,
                 cta_pair=cta_pair or GEMM_CTA_PAIR, epi_warps=epi_warps or GEMM_EPI_WARPS)
    global LAUNCHES
    LAUNCHES += 1
    if gemm_hook is not None:
        gemm_hook((M, N, K, int(a_mn), int(b_mn), epilogue), 2.0 * M * N * K,
                  lambda: check(load().bb_gemm_bf16(ctypes.byref(d), _stream(stream)), "bb_gemm_bf16"))
        return out
    check(load().bb_gemm_bf16(ctypes.byref(d), _stream(stream)), "bb_gemm_bf16")
    return out


# ---------------------------------------------------------------------------- helpers
_LL = ctypes.c_longlong
_F = ctypes.c_float
_I = ctypes.c_int
_workspaces = {}


def workspace(nbytes, tag="default", stream=None):
    """A per-device scratch buffer that only ever grows (allocated through torch so it is
    accounted in the caching allocator; the native side never allocates).  ``stream`` is the raw
    handle of the stream the buffer's kernels run on when that is not the current one: a
    buffer that is replaced by a larger one is first marked as in use on every stream that
    consumed it, so the caching allocator cannot hand its block to another tensor while
    kernels queued there still read and write it."""
    import torch
    dev = torch.cuda.current_device()
    key = (dev, tag)
    entry = _workspaces.get(key)
    buf = entry[0] if entry is not None else None
    users = entry[1] if entry is not None else set()
    if stream is not None:
        users.add(int(stream))
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            for raw in users:
                buf.record_stream(torch.cuda.ExternalStream(raw, device=f"cuda:{dev}"))
        buf = torch.empty(max(int(nbytes), 1 << 20), dtype=torch.uint8, device=f"cuda:{dev}")
    _workspaces[key] = (buf, users)
    return buf


def layernorm_fwd(x, gamma, beta, y, mean, rstd, eps=1e-5):
    global LAUNCHES
    LAUNCHES += 1
    rows, h = x.numel() // x.shape[-1], x.shape[-1]
    check(load().bb_layernorm_fwd(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(mean), _ptr(rstd),
                                  _I(rows), _I(h), _F(eps), _stream()), "bb_layernorm_fwd")
    return y


def layernorm_bwd(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta):
    global LAUNCHES
    LAUNCHES += 2
    rows, h = x.numel() // x.shape[-1], x.shape[-1]
    lib = load()
    lib.bb_layernorm_bwd_workspace_bytes.restype = _LL
    need = lib.bb_layernorm_bwd_workspace_bytes(_I(rows), _I(h))
    ws = workspace(need, "rowwise")
    check(lib.bb_layernorm_bwd(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dres), _ptr(dx),
                               _ptr(dgamma), _ptr(dbeta), _ptr(ws), _LL(ws.numel()), _I(rows), _I(h), _stream()),
          "bb_layernorm_bwd")
    return dx


def layernorm_bwd_res(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, dres_sum):
    """LayerNorm backward that also accumulates the column sums of ``dres`` into ``dres_sum`` (fp32)."""
    global LAUNCHES
    LAUNCHES += 2
    lib = load()
    rows, h = x.shape[0], x.shape[1]
    lib.bb_layernorm_bwd_res_workspace_bytes.restype = _LL
    need = lib.bb_layernorm_bwd_res_workspace_bytes(_I(rows), _I(h))
    ws = workspace(need, "rowwise")
    check(lib.bb_layernorm_bwd_res(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dres), _ptr(dx),
                                   _ptr(dgamma), _ptr(dbeta), _ptr(dres_sum), _ptr(ws), _LL(ws.numel()), _I(rows), _I(h),
                                   _stream()), "bb_layernorm_bwd_res")
    return dx


def layernorm_bwd_static(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta):
    """LayerNorm backward through the entry point that allocates nothing: its scratch is an
    array inside the library (see bb_layernorm_bwd_static in the header for the limits)."""
    global LAUNCHES
    LAUNCHES += 2
    rows, h = x.numel() // x.shape[-1], x.shape[-1]
    check(load().bb_layernorm_bwd_static(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dres), _ptr(dx),
                                         _ptr(dgamma), _ptr(dbeta), _I(rows), _I(h), _stream()),
          "bb_layernorm_bwd_static")
    return dx


def colsum_accum(dy, out, tag="rowwise", stream=None):
    """out(fp32)[n] += dy(bf16)[rows, n].sum(0); ``tag`` names the scratch buffer (calls that may
    overlap on the GPU, e.g. on different streams, need different ones)"""
    global LAUNCHES
    LAUNCHES += 1
    rows, n = dy.shape
    lib = load()
    lib.bb_colsum_workspace_bytes.restype = _LL
    need = lib.bb_colsum_workspace_bytes(_I(rows), _I(n))
    ws = workspace(need, tag, stream)
    check(lib.bb_colsum_accum(_ptr(dy), _LL(dy.stride(0)), _ptr(out), _ptr(ws), _LL(ws.numel()), _I(rows), _I(n),
                              _stream(stream)), "bb_colsum_accum")
    return out


def gelu_bwd(dy, pre, dx):
    """dx = dy * gelu'(pre), elementwise over contiguous bf16 tensors"""
    global LAUNCHES
    LAUNCHES += 1
    check(load().bb_gelu_bwd(_ptr(dy), _ptr(pre), _ptr(dx), _LL(dy.numel()), _stream()), "bb_gelu_bwd")
    return dx


def embedding_fwd(tokens, wte, wpe, out, seq):
    global LAUNCHES
    LAUNCHES += 1
    check(load().bb_embedding_fwd(_ptr(tokens), _ptr(wte), _ptr(wpe), _ptr(out), _I(tokens.numel()), _I(seq),
                                  _I(wte.shape[1]), _I(wte.shape[0]), _stream()), "bb_embedding_fwd")
    return out


def embedding_bwd(tokens, dout, dwte, dwpe, seq):
    global LAUNCHES
    LAUNCHES += 1
    check(load().bb_embedding_bwd(_ptr(tokens), _ptr(dout), _ptr(dwte), _ptr(dwpe), _I(tokens.numel()), _I(seq),
                                  _I(dwte.shape[1]), _I(dwte.shape[0]), _stream()), "bb_embedding_bwd")


def attention_fwd(qkv, out, lse, B, H, S, D, causal, scale=None):
    """qkv: [B*S, 3*H*D] packed projection output; out: [B*S, H*D]; lse: [B,H,S] fp32."""
    global LAUNCHES
    LAUNCHES += 1
    hd = H * D
    esz = qkv.element_size()
    base = qkv.data_ptr()
    scale = (1.0 / D ** 0.5) if scale is None else scale
    check(load().bb_attention_fwd(ctypes.c_void_p(base), ctypes.c_void_p(base + hd * esz),
                                  ctypes.c_void_p(base + 2 * hd * esz), _ptr(out), _ptr(lse), _I(B), _I(H), _I(S),
                                  _I(D), _LL(qkv.stride(0)), _LL(out.stride(0)), _I(int(causal)), _F(scale),
                                  _stream()), "bb_attention_fwd")
    return out


def attention_bwd(qkv, out, dout, lse, dqkv, B, H, S, D, causal, scale=None):
    global LAUNCHES
    LAUNCHES += 3
    hd = H * D
    esz = qkv.element_size()
    base, dbase = qkv.data_ptr(), dqkv.data_ptr()
    scale = (1.0 / D ** 0.5) if scale is None else scale
    lib = load()
    lib.bb_attention_bwd_workspace_bytes.restype = _LL
    need = lib.bb_attention_bwd_workspace_bytes(_I(B), _I(H), _I(S))
    ws = workspace(need, "attention")
    check(lib.bb_attention_bwd(ctypes.c_void_p(base), ctypes.c_void_p(base + hd * esz),
                               ctypes.c_void_p(base + 2 * hd * esz), _ptr(out), _ptr(dout), _ptr(lse),
                               ctypes.c_void_p(dbase), ctypes.c_void_p(dbase + hd * esz),
                               ctypes.c_void_p(dbase + 2 * hd * esz), _ptr(ws), _LL(ws.numel()), _I(B), _I(H), _I(S),
                               _I(D), _LL(qkv.stride(0)), _LL(out.stride(0)), _LL(dqkv.stride(0)), _I(int(causal)),
                               _F(scale), _stream()), "bb_attention_bwd")
    return dqkv


def cross_entropy_fwd(logits, targets, lse, row_loss, loss_out, vocab, ignore_index=-100):
    global LAUNCHES
    LAUNCHES += 2
    rows = logits.shape[0]
    check(load().bb_cross_entropy_fwd(_ptr(logits), _LL(logits.stride(0)), _ptr(targets), _ptr(lse), _ptr(row_loss),
                                      _ptr(loss_out), _I(rows), _I(vocab), _LL(ignore_index), _stream()),
          "bb_cross_entropy_fwd")
    return loss_out


def cross_entropy_bwd(logits, targets, lse, loss_out, dlogits, vocab, grad_scale=1.0, grad_scale_dev=None,
                      ignore_index=-100):
    global LAUNCHES
    LAUNCHES += 1
    rows, cols = logits.shape
    check(load().bb_cross_entropy_bwd(_ptr(logits), _LL(logits.stride(0)), _ptr(targets), _ptr(lse), _ptr(loss_out),
                                      _ptr(grad_scale_dev), _F(grad_scale), _ptr(dlogits), _LL(dlogits.stride(0)),
                                      _I(rows), _I(vocab), _I(cols), _LL(ignore_index), _stream()),
          "bb_cross_entropy_bwd")
    return dlogits


def adam_step(master, grad, exp_avg, exp_avg_sq, param_lp, *, lr, beta1=0.9, beta2=0.999, eps=1e-8, step,
              adam_w_mode=True, bias_correction=True, weight_decay=0.0, grad_scale=1.0, zero_grad=True):
    global LAUNCHES
    LAUNCHES += 1
    check(load().bb_adam_step(_ptr(master), _ptr(grad), _ptr(exp_avg), _ptr(exp_avg_sq), _ptr(param_lp),
                              _LL(master.numel()), _F(lr), _F(beta1), _F(beta2), _F(eps), _I(step),
                              _I(int(adam_w_mode)), _I(int(bias_correction)), _F(weight_decay), _F(grad_scale),
                              _I(int(zero_grad)), _stream()), "bb_adam_step")


def cast_f32_to_bf16(src, dst):
    global LAUNCHES
    LAUNCHES += 1
    check(load().bb_cast_f32_to_bf16(_ptr(src), _ptr(dst), _LL(src.numel()), _stream()), "bb_cast_f32_to_bf16")
    return dst


def block_half_fwd(desc, half, x, saved, out):
    global LAUNCHES
    LAUNCHES += HALF_FWD_LAUNCHES[half]
    check(load().bb_block_half_fwd(ctypes.byref(desc), _I(half), _ptr(x), _ptr(saved), _ptr(out), _stream()),
          "bb_block_half_fwd")
    return out


def block_half_bwd(desc, half, x, saved, dout, dx, scratch, side_stream=None):
    """``side_stream``: raw handle of the stream for the weight gradients (None: the current stream)."""
    global LAUNCHES
    LAUNCHES += HALF_BWD_LAUNCHES[half]
    main = _stream()
    side = main if side_stream is None else ctypes.c_void_p(side_stream)
    check(load().bb_block_half_bwd(ctypes.byref(desc), _I(half), _ptr(x), _ptr(saved), _ptr(dout), _ptr(dx), _ptr(scratch),
                                   _LL(scratch.numel()), main, side), "bb_block_half_bwd")
    return dx


# ---------------------------------------------------------------------------- convolutional stages
def im2col(x, col, k, stride, pad, Ho, Wo):
    """x: [N,H,W,C] bf16 -> col: [N*Ho*Wo, ld] patch matrix, columns (r, s, c)."""
    global LAUNCHES
    LAUNCHES += 1
    N, H, W, C = x.shape
    check(load().bb_im2col_nhwc(_ptr(x), _ptr(col), _I(N), _I(H), _I(W), _I(C), _I(k), _I(stride), _I(pad), _I(Ho), _I(Wo),
                                _LL(col.stride(0)), _stream()), "bb_im2col_nhwc")
    return col


def col2im(dcol, dx, k, stride, pad, Ho, Wo):
    global LAUNCHES
    LAUNCHES += 1
    N, H, W, C = dx.shape
    check(load().bb_col2im_nhwc(_ptr(dcol), _ptr(dx), _I(N), _I(H), _I(W), _I(C), _I(k), _I(stride), _I(pad), _I(Ho), _I(Wo),
                                _LL(dcol.stride(0)), _stream()), "bb_col2im_nhwc")
    return dx


def _bn_ws(rows, C):
    lib = load()
    lib.bb_bn_workspace_bytes.restype = _LL
    need = lib.bb_bn_workspace_bytes(_LL(rows), _I(C))
    if need < 0:
        raise BambooNativeError(f"batch norm over {C} channels: the channel count must be 8 x a power of two <= 2048")
    return workspace(need, "bn")


def bn_stats(y, mean, rstd, eps=1e-5):
    global LAUNCHES
    LAUNCHES += 2
    rows, C = y.shape
    ws = _bn_ws(rows, C)
    check(load().bb_bn_stats(_ptr(y), _LL(rows), _I(C), _F(eps), _ptr(mean), _ptr(rstd), _ptr(ws), _LL(ws.numel()), _stream()),
          "bb_bn_stats")


def bn_apply(y, mean, rstd, gamma, beta, residual, z, relu):
    global LAUNCHES
    LAUNCHES += 1
    rows, C = y.shape
    check(load().bb_bn_apply(_ptr(y), _ptr(mean), _ptr(rstd), _ptr(gamma), _ptr(beta), _ptr(residual), _ptr(z), _LL(rows), _I(C),
                             _I(int(relu)), _stream()), "bb_bn_apply")
    return z


def bn_bwd(dz, z, y, mean, rstd, gamma, dy, dres, dgamma, dbeta, relu):
    global LAUNCHES
    LAUNCHES += 3
    rows, C = y.shape
    ws = _bn_ws(rows, C)
    check(load().bb_bn_bwd(_ptr(dz), _ptr(z), _ptr(y), _ptr(mean), _ptr(rstd), _ptr(gamma), _ptr(dy), _ptr(dres), _ptr(dgamma),
                           _ptr(dbeta), _LL(rows), _I(C), _I(int(relu)), _ptr(ws), _LL(ws.numel()), _stream()), "bb_bn_bwd")
    return dy


def maxpool_fwd(x, y, argmax):
    global LAUNCHES
    LAUNCHES += 1
    N, H, W, C = x.shape
    check(load().bb_maxpool3x3s2_fwd(_ptr(x), _ptr(y), _ptr(argmax), _I(N), _I(H), _I(W), _I(C), _stream()), "bb_maxpool3x3s2_fwd")
    return y


def maxpool_bwd(dy, argmax, dx):
    global LAUNCHES
    LAUNCHES += 1
    N, H, W, C = dx.shape
    check(load().bb_maxpool3x3s2_bwd(_ptr(dy), _ptr(argmax), _ptr(dx), _I(N), _I(H), _I(W), _I(C), _stream()), "bb_maxpool3x3s2_bwd")
    return dx


def avgpool_fwd(x, y):
    global LAUNCHES
    LAUNCHES += 1
    N, H, W, C = x.shape
    check(load().bb_avgpool_fwd(_ptr(x), _ptr(y), _I(N), _I(H * W), _I(C), _stream()), "bb_avgpool_fwd")
    return y


def avgpool_bwd(dy, dx):
    global LAUNCHES
    LAUNCHES += 1
    N, H, W, C = dx.shape
    check(load().bb_avgpool_bwd(_ptr(dy), _ptr(dx), _I(N), _I(H * W), _I(C), _stream()), "bb_avgpool_bwd")
    return dx


def conv_bn_fwd(desc, x, residual, y, z, mean, rstd, scratch):
    global LAUNCHES
    LAUNCHES += 4 + (0 if (desc.k == 1 and desc.stride == 1) else 1)
    check(load().bb_conv_bn_fwd(ctypes.byref(desc), _ptr(x), _ptr(residual), _ptr(y), _ptr(z), _ptr(mean), _ptr(rstd),
                                _ptr(scratch), _LL(scratch.numel()), _stream()), "bb_conv_bn_fwd")
    return z


def conv_bn_bwd(desc, x, y, z, mean, rstd, dz, dx, dres, scratch):
    global LAUNCHES
    direct = desc.k == 1 and desc.stride == 1
    LAUNCHES += 4 + (0 if direct else 1) + (0 if dx is None else (1 if direct else 2))
    check(load().bb_conv_bn_bwd(ctypes.byref(desc), _ptr(x), _ptr(y), _ptr(z), _ptr(mean), _ptr(rstd), _ptr(dz), _ptr(dx),
                                _ptr(dres), _ptr(scratch), _LL(scratch.numel()), _stream()), "bb_conv_bn_bwd")
    return dx
