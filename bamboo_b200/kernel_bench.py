"""Stand-alone timings of the library's kernels through the C ABI bindings (CUDA events, one GPU).

    python -m bamboo_b200.kernel_bench attention     # tcgen05 attention forward / backward
    python -m bamboo_b200.kernel_bench rowwise       # LayerNorm backward, bias-gradient column sums
    python -m bamboo_b200.kernel_bench gemm          # the GEMM shapes of a GPT-2-medium step, beside torch.matmul

Every measurement rotates over operand sets larger than the 126 MB L2.  The row-wise kernels are
short enough for the host to be the bottleneck of a launch loop, so their calls are captured into
a CUDA graph and the graph is replayed; the fixed cost of a call in that harness is reported from
a tiny shape.
"""
import sys

import torch

from . import lib as L


def _events(fn, iters):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(iters):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters * 1e3            # us per call


def _graph_us(fn, sets, passes=3, replays=10):
    """us per call of fn(i), i over `sets` operand sets, from replays of a captured graph."""
    for i in range(sets):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(passes):
            for i in range(sets):
                fn(i)
    g.replay()
    return _events(lambda _i: g.replay(), replays) / (passes * sets)


def attention():
    for (B, H, S, D, causal) in [(8, 16, 1024, 64, True), (8, 16, 1024, 64, False), (4, 16, 512, 64, False),
                                 (2, 32, 2048, 128, True)]:
        sets = 4
        qkv = [(torch.randn(B * S, 3 * H * D, device="cuda") * 0.5).bfloat16() for _ in range(sets)]
        out = [torch.empty(B * S, H * D, device="cuda", dtype=torch.bfloat16) for _ in range(sets)]
        lse = [torch.empty(B, H, S, device="cuda") for _ in range(sets)]
        do = [torch.randn_like(out[0]) for _ in range(sets)]
        dqkv = torch.empty_like(qkv[0])

        def fwd(i):
            L.attention_fwd(qkv[i % sets], out[i % sets], lse[i % sets], B, H, S, D, causal)

        def bwd(i):
            L.attention_bwd(qkv[i % sets], out[i % sets], do[i % sets], lse[i % sets], dqkv, B, H, S, D, causal)
        for i in range(sets):
            fwd(i)
            bwd(i)
        torch.cuda.synchronize()
        if L.read_status() != 0:
            print(f"attention B{B} H{H} S{S} D{D} causal={causal}: device status {L.read_status()} after the warm-up calls, not timed", flush=True)
            return
        tf, tb = _events(fwd, 40), _events(bwd, 40)
        half = 0.5 if causal else 1.0
        print(f"attention B{B} H{H} S{S} D{D} causal={causal}: forward {tf:.1f} us ({2 * 2 * B * H * S * S * D * half / tf / 1e6:.0f} TFLOP/s), "
              f"backward {tb:.1f} us ({5 * 2 * B * H * S * S * D * half / tb / 1e6:.0f} TFLOP/s useful), device status {L.read_status()}", flush=True)


def rowwise():
    def ln_case(rows, h, sets):
        x = [torch.randn(rows, h, device="cuda").bfloat16() for _ in range(sets)]
        dy = [torch.randn(rows, h, device="cuda").bfloat16() for _ in range(sets)]
        dres = [torch.randn(rows, h, device="cuda").bfloat16() for _ in range(sets)]
        g = torch.ones(h, device="cuda", dtype=torch.bfloat16)
        mean = [t.float().mean(1) for t in x]
        rstd = [1.0 / t.float().std(1) for t in x]
        dx = torch.empty(rows, h, device="cuda", dtype=torch.bfloat16)
        dg, db, ds = (torch.zeros(h, device="cuda") for _ in range(3))
        plain = _graph_us(lambda i: L.layernorm_bwd(dy[i], x[i], g, mean[i], rstd[i], dres[i], dx, dg, db), sets)
        fused = _graph_us(lambda i: L.layernorm_bwd_res(dy[i], x[i], g, mean[i], rstd[i], dres[i], dx, dg, db, ds), sets)
        return plain, fused
    fixed, _ = ln_case(16, 1024, 4)
    print(f"layernorm_bwd 16 x 1024 (fixed cost of a call: two launches): {fixed:.1f} us", flush=True)
    for rows, h, sets in [(8192, 1024, 8), (4096, 4096, 4)]:
        plain, fused = ln_case(rows, h, sets)
        print(f"layernorm_bwd {rows} x {h}: {plain:.1f} us per call, net of the fixed cost {4 * 2 * rows * h / (plain - fixed) / 1e6:.2f} TB/s; "
              f"with the residual column sums {fused:.1f} us", flush=True)
    for rows, n in [(64, 256), (8192, 1024), (8192, 3072), (8192, 4096)]:
        k = max(2, int(500e6 / (rows * n * 2))) if rows > 64 else 4
        src = [torch.randn(rows, n, device="cuda").bfloat16() for _ in range(k)]
        out = torch.zeros(n, device="cuda")
        t = _graph_us(lambda i: L.colsum_accum(src[i], out), k)
        print(f"colsum {rows} x {n}: {t:.1f} us per call ({2 * rows * n / t / 1e6:.2f} TB/s including the fixed cost)", flush=True)
        del src


def gemm():
    T = 8192
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timed(fn, iters=30):
        for _ in range(3):
            fn()
        total = 0.0
        for _ in range(iters):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); fn(); b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters * 1e3
    shapes = [(T, 3072, 1024, 0, 0, L.EPI_BIAS), (T, 1024, 1024, 0, 0, L.EPI_BIAS_RESIDUAL), (T, 4096, 1024, 0, 0, L.EPI_BIAS_GELU),
              (T, 1024, 4096, 0, 0, L.EPI_BIAS_RESIDUAL), (T, 4096, 1024, 0, 1, L.EPI_MUL_DGELU), (T, 1024, 4096, 0, 1, L.EPI_STORE),
              (T, 1024, 1024, 0, 1, L.EPI_STORE), (T, 1024, 3072, 0, 1, L.EPI_STORE), (1024, 4096, T, 1, 1, L.EPI_ACCUM_F32),
              (4096, 1024, T, 1, 1, L.EPI_ACCUM_F32), (1024, 1024, T, 1, 1, L.EPI_ACCUM_F32), (3072, 1024, T, 1, 1, L.EPI_ACCUM_F32),
              (T, 50304, 1024, 0, 0, L.EPI_STORE), (T, 1024, 50304, 0, 1, L.EPI_STORE), (50304, 1024, T, 1, 1, L.EPI_ACCUM_F32),
              (8192, 8192, 8192, 0, 0, L.EPI_STORE)]
    for (M, N, K, am, bm, epi) in shapes:
        A = torch.randn(M, K, device="cuda").bfloat16()
        B = torch.randn(N, K, device="cuda").bfloat16()
        a = A.t().contiguous() if am else A
        b = B.t().contiguous() if bm else B
        f32 = epi in (L.EPI_ACCUM_F32, L.EPI_STORE_F32)
        out = torch.zeros(M, N, device="cuda", dtype=torch.float32 if f32 else torch.bfloat16)
        out2 = torch.zeros_like(out)
        bias = torch.zeros(N, device="cuda").bfloat16()
        aux = torch.zeros(M, N, device="cuda").bfloat16()
        ours = timed(lambda: L.gemm(a, b, out, a_mn=bool(am), b_mn=bool(bm), epilogue=epi, bias=bias, out2=out2, aux=aux, M=M, N=N, K=K))
        Bt = B.t()
        ref = timed(lambda: torch.matmul(A, Bt))
        print(f"gemm M{M} N{N} K{K} a_mn{am} b_mn{bm} epilogue {epi}: {ours:.1f} us {2 * M * N * K / ours / 1e6:.0f} TFLOP/s | "
              f"torch.matmul (plain) {ref:.1f} us {2 * M * N * K / ref / 1e6:.0f} TFLOP/s | ratio {ours / ref:.2f}", flush=True)
        del A, B, a, b, out, out2, aux
    print("device status", L.read_status())


if __name__ == "__main__":
    L.load()
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    if which in ("attention", "all"):
        attention()
    if which in ("rowwise", "all"):
        rowwise()
    if which in ("gemm", "all"):
        gemm()
