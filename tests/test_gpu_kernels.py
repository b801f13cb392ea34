"""Parity of every sm_100a kernel, called through the C ABI, with an fp32 PyTorch statement
of the same operation on the same seeded inputs.  Tolerance: bf16 outputs within 2e-2 of
the reference magnitude; fp32 accumulations within 1e-3."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def L():
    from bamboo_b200 import lib
    lib.load()
    return lib


def close(got, want, tol=2e-2):
    err = (got.float() - want.float()).abs().max().item()
    scale = want.float().abs().max().item()
    assert err <= tol * scale + 1e-3, (err, scale)


def gelu(x):
    return F.gelu(x, approximate="tanh")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("tile_n,cta_pair", [(128, -1), (256, -1), (0, 1)])
def test_gemm_operand_layouts(L, a_mn, b_mn, tile_n, cta_pair):
    torch.manual_seed(0)
    M, N, K = 384, 512, 320
    A = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    B = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    L.gemm(a, b, out, a_mn=a_mn, b_mn=b_mn, M=M, N=N, K=K, tile_n=tile_n, cta_pair=cta_pair)
    close(out, A.float() @ B.float().t())


@pytest.mark.parametrize("cta_pair", [-1, 1])
@pytest.mark.parametrize("shape", [(128, 128, 64), (200, 136, 72), (130, 264, 200), (8, 8, 8), (1024, 1024, 1000),
                                   (100, 260, 136), (520, 100, 72)])
def test_gemm_ragged_shapes(L, shape, cta_pair):
    """Edges: rows and columns that end inside a tile, inside a 16-byte store, or (pairs) before
    the second CTA's rows begin."""
    torch.manual_seed(1)
    M, N, K = shape
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(N, K, device="cuda").bfloat16()
    bias = torch.randn(N + 8, device="cuda").bfloat16()[:N]
    ldd = (N + 7) // 8 * 8 + 8                                       # guard columns after N
    out = torch.full((M, ldd), 7.0, device="cuda", dtype=torch.bfloat16)
    L.gemm(A, B, out[:, :N], epilogue=L.EPI_BIAS, bias=bias, cta_pair=cta_pair)
    close(out[:, :N], A.float() @ B.float().t() + bias.float())
    assert torch.all(out[:, N:] == 7)                               # nothing written past column N
    aux = torch.randn(M, ldd, device="cuda").bfloat16()[:, :N]
    L.gemm(A, B, out[:, :N], epilogue=L.EPI_BIAS_RESIDUAL, bias=bias, aux=aux, cta_pair=cta_pair)
    close(out[:, :N], A.float() @ B.float().t() + bias.float() + aux.float())
    out.fill_(7)
    L.gemm(A, B, out[:, :N], epilogue=L.EPI_BIAS_RESIDUAL, bias=bias, aux=aux, cta_pair=cta_pair, epi_warps=4)
    close(out[:, :N], A.float() @ B.float().t() + bias.float() + aux.float())
    assert torch.all(out[:, N:] == 7)
    acc = torch.full((M, ldd), 7.0, device="cuda")
    L.gemm(A, B, acc[:, :N], epilogue=L.EPI_ACCUM_F32, cta_pair=cta_pair)
    close(acc[:, :N], A.float() @ B.float().t() + 7, 1e-3)
    assert torch.all(acc[:, N:] == 7)


@pytest.mark.parametrize("epi_warps", [2, 4])
@pytest.mark.parametrize("cta_pair", [-1, 1])
def test_gemm_epilogues(L, cta_pair, epi_warps):
    """Every fused epilogue, with 8 and with 16 epilogue warps (the latter bf16 outputs only)."""
    torch.manual_seed(2)
    M, N, K = 384, 768, 320
    A = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    B = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    aux = torch.randn(M, N, device="cuda").bfloat16()
    ref = A.float() @ B.float().t()
    out = torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)
    out2 = torch.zeros_like(out)
    L.gemm(A, B, out, epilogue=L.EPI_BIAS_GELU, bias=bias, out2=out2, cta_pair=cta_pair, epi_warps=epi_warps)
    close(out2, ref + bias.float())
    close(out, gelu((ref + bias.float()).bfloat16().float()))
    L.gemm(A, B, out, epilogue=L.EPI_BIAS_RESIDUAL, bias=bias, aux=aux, cta_pair=cta_pair, epi_warps=epi_warps)
    close(out, ref + bias.float() + aux.float())
    x = aux.float().requires_grad_(True)
    gelu(x).sum().backward()
    L.gemm(A, B, out, epilogue=L.EPI_MUL_DGELU, aux=aux, cta_pair=cta_pair, epi_warps=epi_warps)
    close(out, ref * x.grad)
    acc = torch.randn(M, N, device="cuda")
    want = acc + ref
    L.gemm(A, B, acc, epilogue=L.EPI_ACCUM_F32, cta_pair=cta_pair)
    close(acc, want, 1e-3)
    L.gemm(A, B, acc, epilogue=L.EPI_STORE_F32, cta_pair=cta_pair)
    close(acc, ref, 1e-3)


def test_gemm_is_linear_and_deterministic_at_full_size(L):
    """GPT-2-medium MLP shape: two runs are bit-identical and (A1+A2)B = A1 B + A2 B in fp32 output."""
    torch.manual_seed(3)
    M, N, K = 8192, 4096, 1024
    A1 = torch.randint(-4, 5, (M, K), device="cuda").bfloat16()
    A2 = torch.randint(-4, 5, (M, K), device="cuda").bfloat16()
    B = torch.randint(-4, 5, (N, K), device="cuda").bfloat16()
    o1, o2, o12, again = (torch.empty(M, N, device="cuda") for _ in range(4))
    L.gemm(A1, B, o1, epilogue=L.EPI_STORE_F32)
    L.gemm(A2, B, o2, epilogue=L.EPI_STORE_F32)
    L.gemm((A1 + A2), B, o12, epilogue=L.EPI_STORE_F32)
    L.gemm(A1, B, again, epilogue=L.EPI_STORE_F32)
    assert torch.equal(o1, again)
    assert torch.equal(o12, o1 + o2)          # small integers: exact in bf16 x bf16 -> fp32
    assert torch.equal(o1[:256], (A1[:256].float() @ B.float().t()))


def test_gemm_cta_pairs_at_full_size(L):
    """Input-gradient shape of the MLP (long reduction, B stored [K, N]): the heuristic picks CTA
    pairs; small integers make the result exact, and single CTAs must give the same bits."""
    torch.manual_seed(13)
    M, N, K = 8192, 1024, 4096
    A = torch.randint(-3, 4, (M, K), device="cuda").bfloat16()
    B = torch.randint(-3, 4, (K, N), device="cuda").bfloat16()      # stored [K, N]
    pair = torch.empty(M, N, device="cuda")
    single = torch.empty(M, N, device="cuda")
    L.gemm(A, B, pair, b_mn=True, epilogue=L.EPI_STORE_F32, M=M, N=N, K=K)
    L.gemm(A, B, single, b_mn=True, epilogue=L.EPI_STORE_F32, M=M, N=N, K=K, cta_pair=-1)
    assert torch.equal(pair, single)
    assert torch.equal(pair[:512], A[:512].float() @ B.float())


@pytest.mark.parametrize("cta_pair", [-1, 1])
@pytest.mark.parametrize("split", [0, 1, 3, 8])
def test_gemm_split_k_accumulation(L, split, cta_pair):
    """Weight-gradient shape (few output tiles, long reduction): partial sums of the K splits
    meet in the fp32 add-reduction."""
    torch.manual_seed(11)
    M, N, K = 1024, 1024, 8192
    A = torch.randint(-3, 4, (K, M), device="cuda").bfloat16()      # stored [K, M]
    B = torch.randint(-3, 4, (K, N), device="cuda").bfloat16()      # stored [K, N]
    acc = torch.ones(M, N, device="cuda")
    L.gemm(A, B, acc, a_mn=True, b_mn=True, epilogue=L.EPI_ACCUM_F32, M=M, N=N, K=K, split_k=split, cta_pair=cta_pair)
    want = A.float().t() @ B.float() + 1
    assert torch.equal(acc, want)                                    # small integers: exact


def test_gemm_rejects_bad_arguments(L):
    A = torch.zeros(16, 12, device="cuda", dtype=torch.bfloat16)   # leading dimension not a multiple of 8
    B = torch.zeros(16, 12, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(16, 16, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(L.BambooNativeError):
        L.gemm(A, B, out)
    with pytest.raises(L.BambooNativeError):
        L.gemm(out, out, out, epilogue=L.EPI_BIAS)                 # bias missing
    with pytest.raises(L.BambooNativeError):
        L.gemm(out, out, torch.zeros(16, 16, device="cuda"), epilogue=L.EPI_STORE_F32, epi_warps=4)   # fp32 output


@pytest.mark.parametrize("rows,h", [(512, 256), (8192, 1024), (300, 768), (1000, 4096)])
def test_layernorm(L, rows, h):
    torch.manual_seed(4)
    x = torch.randn(rows, h, device="cuda").bfloat16()
    g = (1 + 0.1 * torch.randn(h, device="cuda")).bfloat16()
    b = (0.1 * torch.randn(h, device="cuda")).bfloat16()
    y = torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    L.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
    xf, gf, bf = x.float().requires_grad_(True), g.float().requires_grad_(True), b.float().requires_grad_(True)
    yr = F.layer_norm(xf, (h,), gf, bf, 1e-5)
    close(y, yr)
    dy, dres = torch.randn(rows, h, device="cuda").bfloat16(), torch.randn(rows, h, device="cuda").bfloat16()
    yr.backward(dy.float())
    dx = torch.empty_like(x)
    dg, db = torch.ones(h, device="cuda"), torch.ones(h, device="cuda")      # accumulate on top of 1
    L.layernorm_bwd(dy, x, g, mean, rstd, dres, dx, dg, db)
    close(dx, xf.grad + dres.float())
    close(dg - 1, gf.grad)
    close(db - 1, bf.grad)


@pytest.mark.parametrize("rows,h", [(8192, 1024), (777, 256), (300, 768), (1000, 2048), (515, 4096), (64, 8192), (100, 1000)])
def test_layernorm_backward_with_residual_sums(L, rows, h):
    """One pass gives dx, dgamma, dbeta and the column sums of the residual gradient; every
    column-owner instantiation (hidden sizes up to 1024, 2048, 4096, 8192) and the fallback."""
    torch.manual_seed(6)
    x = torch.randn(rows, h, device="cuda").bfloat16()
    g = (1 + 0.1 * torch.randn(h, device="cuda")).bfloat16()
    b = torch.zeros(h, device="cuda").bfloat16()
    y = torch.empty_like(x)
    mean, rstd = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda")
    L.layernorm_fwd(x, g, b, y, mean, rstd, 1e-5)
    dy, dres = torch.randn(rows, h, device="cuda").bfloat16(), torch.randn(rows, h, device="cuda").bfloat16()
    dx0, dx1 = torch.empty_like(x), torch.empty_like(x)
    dg0, db0 = torch.zeros(h, device="cuda"), torch.zeros(h, device="cuda")
    dg1, db1, ds1 = torch.zeros(h, device="cuda"), torch.zeros(h, device="cuda"), torch.ones(h, device="cuda")
    L.layernorm_bwd(dy, x, g, mean, rstd, dres, dx0, dg0, db0)
    L.layernorm_bwd_res(dy, x, g, mean, rstd, dres, dx1, dg1, db1, ds1)
    close(dx1, dx0, 1e-2)
    close(dg1, dg0, 1e-4)
    close(db1, db0, 1e-4)
    close(ds1 - 1, dres.float().sum(0), 1e-3)
    xf, gf = x.float().requires_grad_(True), g.float().requires_grad_(True)
    F.layer_norm(xf, (h,), gf, b.float(), 1e-5).backward(dy.float())
    close(dx1, xf.grad + dres.float())
    close(dg1, gf.grad)
    # in place over the residual gradient
    alias = dres.clone()
    ds2 = torch.zeros(h, device="cuda")
    L.layernorm_bwd_res(dy, x, g, mean, rstd, alias, alias, dg1, db1, ds2)
    close(alias, dx1, 1e-2)
    close(ds2, dres.float().sum(0), 1e-3)
    assert L.read_status() == 0


@pytest.mark.parametrize("rows,n", [(8192, 4096), (8192, 1024), (100, 264), (513, 1024), (1, 8), (4096, 50304), (33, 3072)])
def test_colsum(L, rows, n):
    torch.manual_seed(5)
    dy = torch.randn(rows, n, device="cuda").bfloat16()
    out = torch.ones(n, device="cuda")
    L.colsum_accum(dy, out)
    close(out - 1, dy.float().sum(0), 1e-3)
    # the ticket counters return to zero: repeated calls (also back to back on two streams, each
    # with its own scratch) give the same bits
    again = torch.ones(n, device="cuda")
    L.colsum_accum(dy, again)
    assert torch.equal(out, again)
    side = torch.cuda.Stream()
    a, b = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    torch.cuda.synchronize()
    for _ in range(3):
        L.colsum_accum(dy, a)
        with torch.cuda.stream(side):
            L.colsum_accum(dy, b, tag="test-side", stream=side.cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    close(a, 3 * dy.float().sum(0), 1e-3)


def test_gelu_backward(L):
    torch.manual_seed(4)
    pre = torch.randn(1000, 1024, device="cuda").bfloat16()
    dy = torch.randn_like(pre)
    dx = torch.empty_like(pre)
    L.gelu_bwd(dy, pre, dx)
    x = pre.float().requires_grad_(True)
    gelu(x).backward(dy.float())
    close(dx, x.grad)


def test_embedding(L):
    torch.manual_seed(6)
    V, h, B, S = 1024, 256, 4, 128
    tok = torch.randint(0, V, (B, S), device="cuda")
    tok[0, :8] = 7                                                   # collisions in the scatter
    wte, wpe = torch.randn(V, h, device="cuda").bfloat16(), torch.randn(S, h, device="cuda").bfloat16()
    out = torch.empty(B * S, h, device="cuda", dtype=torch.bfloat16)
    L.embedding_fwd(tok, wte, wpe, out, S)
    close(out, wte[tok.view(-1)].float() + wpe.float().repeat(B, 1))
    dout = torch.randn(B * S, h, device="cuda").bfloat16()
    dwte, dwpe = torch.zeros(V, h, device="cuda"), torch.zeros(S, h, device="cuda")
    L.embedding_bwd(tok, dout, dwte, dwpe, S)
    close(dwte, torch.zeros(V, h, device="cuda").index_add_(0, tok.view(-1), dout.float()), 1e-3)
    close(dwpe, dout.float().view(B, S, h).sum(0), 1e-3)


@pytest.mark.parametrize("rows,V,Vp", [(512, 1024, 1024), (1024, 50257, 50304), (100, 30522, 30528), (4, 8, 8)])
def test_cross_entropy(L, rows, V, Vp):
    torch.manual_seed(7)
    logits = torch.zeros(rows, Vp, device="cuda", dtype=torch.bfloat16)
    logits[:, :V] = (3 * torch.randn(rows, V, device="cuda")).bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[::7] = -100                                                  # ignored positions
    lse, rl, lo = torch.empty(rows, device="cuda"), torch.empty(rows, device="cuda"), torch.empty(2, device="cuda")
    L.cross_entropy_fwd(logits, tgt, lse, rl, lo, V)
    lf = logits[:, :V].float().requires_grad_(True)
    ref = F.cross_entropy(lf, tgt, ignore_index=-100)
    assert lo[0].item() == pytest.approx(ref.item(), rel=1e-4)
    assert lo[1].item() == (tgt != -100).sum().item()
    (ref * 0.25).backward()
    L.cross_entropy_bwd(logits, tgt, lse, lo, logits, V, grad_scale=0.25)       # in place
    close(logits[:, :V], lf.grad)
    assert logits[:, V:].abs().max().item() == 0 if Vp > V else True


def test_adam_matches_torch(L):
    torch.manual_seed(8)
    n = 1 << 20
    p, m, v = torch.randn(n, device="cuda"), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    g, lp = torch.empty(n, device="cuda"), torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = p.clone().requires_grad_(True)
    opt = torch.optim.Adam([pr], lr=1e-3)
    for step in (1, 2, 3):
        gg = torch.randn(n, device="cuda")
        g.copy_(gg)
        pr.grad = gg.clone()
        opt.step()
        L.adam_step(p, g, m, v, lp, lr=1e-3, step=step)
    close(p, pr.detach(), 1e-5)
    close(lp, pr.detach(), 1e-2)
    assert g.abs().max().item() == 0
    close(m, opt.state[pr]["exp_avg"], 1e-5)
    close(v, opt.state[pr]["exp_avg_sq"], 1e-5)


def _attn_ref(qkv, B, H, S, D, causal):
    q, k, v = qkv.float().view(B, S, 3, H, D).permute(2, 0, 3, 1, 4)
    return F.scaled_dot_product_attention(q, k, v, is_causal=causal).permute(0, 2, 1, 3).reshape(B * S, H * D)


@pytest.mark.parametrize("B,H,S,D,causal", [(2, 4, 128, 64, True), (2, 3, 256, 64, False), (1, 2, 1024, 64, True),
                                            (1, 2, 200, 64, True), (1, 2, 72, 64, False), (1, 2, 256, 128, True),
                                            (2, 2, 320, 128, False),
                                            # an odd number of 64-query sub-blocks (the fused backward pairs them up and
                                            # pads with a masked one that reads the next batch's rows), several key tiles
                                            (2, 2, 192, 64, True), (2, 2, 192, 64, False), (2, 1, 448, 64, True),
                                            (1, 1, 2048, 64, True), (3, 2, 640, 64, False),
                                            # head dimension 128: tcgen05 forward (two 64-column atoms per row), warp-level backward
                                            (1, 2, 1024, 128, True), (1, 2, 200, 128, True), (2, 1, 448, 128, False),
                                            (1, 1, 72, 128, False),
                                            (1, 16, 2048, 128, True)])     # enough CTAs to keep every SM and the TMA unit busy
def test_attention(L, B, H, S, D, causal):
    torch.manual_seed(9)
    qkv = torch.randn(B * S, 3 * H * D, device="cuda").bfloat16()
    out = torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, S, device="cuda")
    L.attention_fwd(qkv, out, lse, B, H, S, D, causal)
    qf = qkv.float().requires_grad_(True)
    ref = _attn_ref(qf, B, H, S, D, causal)
    close(out, ref)
    do = torch.randn_like(out)
    ref.backward(do.float())
    dqkv = torch.empty_like(qkv)
    L.attention_bwd(qkv, out, do, lse, dqkv, B, H, S, D, causal)
    close(dqkv, qf.grad)


def test_attention_backward_with_fixed_summation_order(L):
    """BB_ATTENTION_BWD=split selects the two-role backward kernels (dK/dV and dQ by different CTAs, no
    reductions into an accumulator): same gradients, and bit-identical from run to run.  The switch is read
    once per process, so the check runs in a child process."""
    import os
    import subprocess
    import sys
    code = """
import sys, torch
sys.path.insert(0, %r)
import torch.nn.functional as F
from bamboo_b200 import lib as L
L.load()
B, H, S, D = 2, 2, 448, 64
torch.manual_seed(3)
qkv = torch.randn(B * S, 3 * H * D, device="cuda").bfloat16()
out = torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16)
lse = torch.empty(B, H, S, device="cuda")
L.attention_fwd(qkv, out, lse, B, H, S, D, True)
qf = qkv.float().requires_grad_(True)
q, k, v = qf.view(B, S, 3, H, D).permute(2, 0, 3, 1, 4)
ref = F.scaled_dot_product_attention(q, k, v, is_causal=True).permute(0, 2, 1, 3).reshape(B * S, H * D)
do = torch.randn_like(out)
ref.backward(do.float())
a, b = torch.empty_like(qkv), torch.empty_like(qkv)
L.attention_bwd(qkv, out, do, lse, a, B, H, S, D, True)
L.attention_bwd(qkv, out, do, lse, b, B, H, S, D, True)
torch.cuda.synchronize()
err = (a.float() - qf.grad).abs().max().item()
assert err <= 2e-2 * qf.grad.abs().max().item() + 1e-3, err
assert torch.equal(a, b)
assert L.read_status() == 0
print("split backward ok")
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, BB_ATTENTION_BWD="split")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "split backward ok" in r.stdout, r.stdout + r.stderr


def test_attention_rows_sum_to_one_at_full_size(L):
    """GPT-2-medium attention shape: with V = 1 every output element must be 1."""
    B, H, S, D = 8, 16, 1024, 64
    torch.manual_seed(10)
    qkv = torch.randn(B * S, 3 * H * D, device="cuda").bfloat16()
    qkv[:, 2 * H * D:] = 1
    out = torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, S, device="cuda")
    L.attention_fwd(qkv, out, lse, B, H, S, D, True)
    assert (out.float() - 1).abs().max().item() < 1e-2
    assert torch.isfinite(lse).all()


def test_attention_backward_checksums_at_full_size(L):
    """GPT-2-medium attention shape, properties that hold at any size: every probability row sums
    to one, so the V-gradient summed over keys equals dO summed over queries; and the score
    gradient of a row sums to zero, so with all keys equal the Q-gradient vanishes."""
    B, H, S, D = 8, 16, 1024, 64
    torch.manual_seed(12)
    qkv = (torch.randn(B * S, 3 * H * D, device="cuda") * 0.5).bfloat16()
    qkv[:, H * D:2 * H * D] = qkv[0, H * D:2 * H * D]               # the same key vector at every position
    out = torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16)
    lse = torch.empty(B, H, S, device="cuda")
    L.attention_fwd(qkv, out, lse, B, H, S, D, True)
    do = torch.randn_like(out)
    dqkv = torch.empty_like(qkv)
    L.attention_bwd(qkv, out, do, lse, dqkv, B, H, S, D, True)
    dq, dv = dqkv[:, :H * D].float(), dqkv[:, 2 * H * D:].float()
    want = do.float().view(B, S, H * D).sum(1)
    got = dv.view(B, S, H * D).sum(1)
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item() + 0.5   # bf16 rounding of 1024 addends
    assert dq.abs().max().item() <= 2e-2 * do.float().abs().max().item()
    assert L.read_status() == 0


def test_ping_counter_may_run_ahead_of_the_receiver(L):
    """A liveness ping carries no payload: its flag is a counter.  A receiver that waits for ping
    1 after the sender already signalled ping 3 has its answer (lazy redundancy on more than two
    stages does exactly that); a payload slot whose flag moved on is an error, and a ping that
    never comes ends the bounded wait with the peer-timeout status.  All on this GPU's own memory."""
    import ctypes
    lib = L.load()
    flag = torch.zeros(1, dtype=torch.int64, device="cuda")
    stream = L._stream()
    fp = ctypes.c_void_p(flag.data_ptr())
    assert lib.bb_p2p_signal(fp, ctypes.c_ulonglong(3), stream) == 0
    assert lib.bb_p2p_wait_copy(None, None, ctypes.c_longlong(0), fp, ctypes.c_ulonglong(1),
                                ctypes.c_ulonglong(200_000_000), None, stream) == 0
    torch.cuda.synchronize()
    assert L.read_status() == 0
    src = torch.ones(64, device="cuda"); dst = torch.zeros(64, device="cuda")
    assert lib.bb_p2p_wait_copy(ctypes.c_void_p(src.data_ptr()), ctypes.c_void_p(dst.data_ptr()), ctypes.c_longlong(256), fp,
                                ctypes.c_ulonglong(1), ctypes.c_ulonglong(200_000_000), None, stream) == 0
    torch.cuda.synchronize()
    assert L.read_status() == -1 and float(dst.sum()) == 0          # overwritten slot: reported, nothing copied
    assert lib.bb_p2p_wait_copy(None, None, ctypes.c_longlong(0), fp, ctypes.c_ulonglong(9),
                                ctypes.c_ulonglong(50_000_000), None, stream) == 0
    torch.cuda.synchronize()
    assert L.read_status() == L.STATUS_PEER_TIMEOUT                   # the wait ran out, the context lives on
    assert L.read_status() == 0


def test_status_word_is_clean(L):
    torch.cuda.synchronize()
    assert L.read_status() == 0
