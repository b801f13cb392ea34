// Channels-last (NHWC, bf16) pieces of the ResNet stages around the tensor-core GEMM: patch
// gathering for k x k convolutions and its adjoint, batch normalisation with batch statistics
// (forward and backward, ReLU and the residual add folded in), 3 x 3 / stride 2 max pooling and
// global average pooling.  All of these are HBM-bound: 16-byte vectors over the channel
// dimension, consecutive threads on consecutive channel chunks of a pixel, fp32 arithmetic.
// A convolution itself is the library's GEMM: output pixels x (taps * input channels) times the
// [Cout, k, k, Cin] weight matrix.
#include "common.cuh"
#include "bamboo_b200.h"

namespace {

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  f[0] = bb::bf16_lo(q.x); f[1] = bb::bf16_hi(q.x); f[2] = bb::bf16_lo(q.y); f[3] = bb::bf16_hi(q.y);
  f[4] = bb::bf16_lo(q.z); f[5] = bb::bf16_hi(q.z); f[6] = bb::bf16_lo(q.w); f[7] = bb::bf16_hi(q.w);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 q;
  q.x = bb::pack_bf16x2(f[0], f[1]); q.y = bb::pack_bf16x2(f[2], f[3]);
  q.z = bb::pack_bf16x2(f[4], f[5]); q.w = bb::pack_bf16x2(f[6], f[7]);
  return q;
}

int flat_grid(long long work_items, int per_thread = 1) {
  long long blocks = (work_items + 256LL * per_thread - 1) / (256LL * per_thread);
  const long long cap = (long long)bb_num_sms() * 16;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

struct ConvGeom {
  int N, H, W, C, k, stride, pad, Ho, Wo;
  long long ld_col;      // elements between consecutive rows of the patch matrix (>= k*k*C)
};

// col[(n, ho, wo), (r, s, c)] = x[n, ho*stride - pad + r, wo*stride - pad + s, c]  (0 outside)
__global__ void __launch_bounds__(256)
im2col_kernel(const uint4* __restrict__ x, uint4* __restrict__ col, const ConvGeom g) {
  const int chunks = g.C >> 3;                       // 16-byte chunks per pixel
  const int row_chunks = g.k * g.k * chunks;
  const long long total = (long long)g.N * g.Ho * g.Wo * row_chunks;
  const long long ld16 = g.ld_col >> 3;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const long long p = e / row_chunks;
    const int within = (int)(e - p * row_chunks);
    const int tap = within / chunks, cc = within - tap * chunks;
    const int r = tap / g.k, s = tap - r * g.k;
    const int wo = (int)(p % g.Wo);
    const long long t = p / g.Wo;
    const int ho = (int)(t % g.Ho), n = (int)(t / g.Ho);
    const int h = ho * g.stride - g.pad + r, w = wo * g.stride - g.pad + s;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (h >= 0 && h < g.H && w >= 0 && w < g.W) v = __ldg(x + (((long long)n * g.H + h) * g.W + w) * chunks + cc);
    col[p * ld16 + within] = v;
  }
}

// Adjoint of the gather: dx[n, h, w, c] = sum over the (output pixel, tap) pairs that read it.
// Gather form (one thread owns an input pixel's chunk): no atomics, fixed summation order.
__global__ void __launch_bounds__(256)
col2im_kernel(const uint4* __restrict__ dcol, uint4* __restrict__ dx, const ConvGeom g) {
  const int chunks = g.C >> 3;
  const long long total = (long long)g.N * g.H * g.W * chunks;
  const long long ld16 = g.ld_col >> 3;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int cc = (int)(e % chunks);
    const long long pix = e / chunks;
    const int w = (int)(pix % g.W);
    const long long t = pix / g.W;
    const int h = (int)(t % g.H), n = (int)(t / g.H);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < g.k; ++r) {
      const int hs = h + g.pad - r;
      if (hs < 0 || hs % g.stride) continue;
      const int ho = hs / g.stride;
      if (ho >= g.Ho) continue;
      for (int s = 0; s < g.k; ++s) {
        const int ws = w + g.pad - s;
        if (ws < 0 || ws % g.stride) continue;
        const int wo = ws / g.stride;
        if (wo >= g.Wo) continue;
        const long long p = ((long long)n * g.Ho + ho) * g.Wo + wo;
        float f[8];
        unpack8(__ldg(dcol + p * ld16 + (r * g.k + s) * chunks + cc), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
    dx[e] = pack8(acc);
  }
}

bool bad_geom(const ConvGeom& g) {
  return g.N <= 0 || g.H <= 0 || g.W <= 0 || g.C <= 0 || (g.C & 7) || g.k <= 0 || g.stride <= 0 || g.pad < 0 ||
         g.Ho != (g.H + 2 * g.pad - g.k) / g.stride + 1 || g.Wo != (g.W + 2 * g.pad - g.k) / g.stride + 1 ||
         g.ld_col < (long long)g.k * g.k * g.C || (g.ld_col & 7);
}

}  // namespace

extern "C" int bb_im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                              long long ld_col, void* stream) {
  const ConvGeom g = {N, H, W, C, k, stride, pad, Ho, Wo, ld_col};
  if (!x || !col || bad_geom(g) || ((uintptr_t)x & 15) || ((uintptr_t)col & 15)) {
    bb_set_last_error_msg("bb_im2col_nhwc: null/unaligned pointer or inconsistent geometry (channels and ld_col multiples of 8)");
    return BB_ERR_INVALID_ARG;
  }
  const long long total = (long long)N * Ho * Wo * k * k * (C >> 3);
  im2col_kernel<<<flat_grid(total, 4), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)col, g);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_col2im_nhwc(const void* dcol, void* dx, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                              long long ld_col, void* stream) {
  const ConvGeom g = {N, H, W, C, k, stride, pad, Ho, Wo, ld_col};
  if (!dcol || !dx || bad_geom(g) || ((uintptr_t)dcol & 15) || ((uintptr_t)dx & 15)) {
    bb_set_last_error_msg("bb_col2im_nhwc: null/unaligned pointer or inconsistent geometry (channels and ld_col multiples of 8)");
    return BB_ERR_INVALID_ARG;
  }
  const long long total = (long long)N * H * W * (C >> 3);
  col2im_kernel<<<flat_grid(total, 2), 256, 0, (cudaStream_t)stream>>>((const uint4*)dcol, (uint4*)dx, g);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

// ---------------------------------------------------------------------------------- batch norm
namespace {

// Per-channel sums over the rows of a [rows, C] bf16 matrix, two quantities at a time.  Thread g
// owns channel chunk g % chunks (chunks = C / 8 divides 256) and walks rows g / chunks,
// + threads / chunks, ...; a block combines its threads through shared memory and writes one
// partial row [2, C] to the workspace; bn_finish_* adds the partial rows in block order.
enum { RED_STATS = 0, RED_BWD = 1 };

template <int MODE>
__global__ void __launch_bounds__(256)
bn_reduce_kernel(const uint4* __restrict__ a, const uint4* __restrict__ zz, const uint4* __restrict__ yy,
                 const float* __restrict__ mean, const float* __restrict__ rstd, int relu, long long rows, int C,
                 float* __restrict__ ws) {
  __shared__ float sm[256 * 16];
  const int chunks = C >> 3;
  const long long gthreads = (long long)gridDim.x * blockDim.x;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cc = (int)(g % chunks);
  const long long row_step = gthreads / chunks;
  float s1[8], s2[8], mu[8], rs[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { s1[i] = 0.f; s2[i] = 0.f; mu[i] = 0.f; rs[i] = 0.f; }
  if (MODE == RED_BWD) {
#pragma unroll
    for (int i = 0; i < 8; ++i) { mu[i] = mean[cc * 8 + i]; rs[i] = rstd[cc * 8 + i]; }
  }
  for (long long r = g / chunks; r < rows; r += row_step) {
    float v[8];
    unpack8(__ldg(a + r * chunks + cc), v);
    if (MODE == RED_STATS) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { s1[i] += v[i]; s2[i] += v[i] * v[i]; }
    } else {
      float y[8];
      unpack8(__ldg(yy + r * chunks + cc), y);
      if (relu) {
        float z[8];
        unpack8(__ldg(zz + r * chunks + cc), z);
#pragma unroll
        for (int i = 0; i < 8; ++i) if (!(z[i] > 0.f)) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) { s1[i] += v[i]; s2[i] += v[i] * ((y[i] - mu[i]) * rs[i]); }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) { sm[threadIdx.x * 16 + i] = s1[i]; sm[threadIdx.x * 16 + 8 + i] = s2[i]; }
  __syncthreads();
  // 256 % chunks == 0: the chunk of thread t is (blockIdx.x * 256 + t) % chunks = t % chunks
  if ((int)threadIdx.x < chunks) {
    float t1[8], t2[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { t1[i] = 0.f; t2[i] = 0.f; }
    for (int j = threadIdx.x; j < 256; j += chunks) {
#pragma unroll
      for (int i = 0; i < 8; ++i) { t1[i] += sm[j * 16 + i]; t2[i] += sm[j * 16 + 8 + i]; }
    }
    float* out = ws + (long long)blockIdx.x * 2 * C;
#pragma unroll
    for (int i = 0; i < 8; ++i) { out[threadIdx.x * 8 + i] = t1[i]; out[C + threadIdx.x * 8 + i] = t2[i]; }
  }
}

// mean / rstd per channel from the partial rows (biased variance, as batch norm normalises with)
__global__ void bn_finish_stats_kernel(const float* __restrict__ ws, int parts, int C, float inv_rows, float eps,
                                       float* __restrict__ mean, float* __restrict__ rstd) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s1 = 0.f, s2 = 0.f;
  for (int p = 0; p < parts; ++p) { s1 += ws[(long long)p * 2 * C + c]; s2 += ws[(long long)p * 2 * C + C + c]; }
  const float m = s1 * inv_rows;
  const float var = fmaxf(s2 * inv_rows - m * m, 0.f);
  mean[c] = m;
  rstd[c] = rsqrtf(var + eps);
}

// sums[0][c] = sum dz', sums[1][c] = sum dz' * yhat; dbeta += sums[0], dgamma += sums[1]
__global__ void bn_finish_bwd_kernel(const float* __restrict__ ws, int parts, int C, float* __restrict__ sums,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s1 = 0.f, s2 = 0.f;
  for (int p = 0; p < parts; ++p) { s1 += ws[(long long)p * 2 * C + c]; s2 += ws[(long long)p * 2 * C + C + c]; }
  sums[c] = s1; sums[C + c] = s2;
  dbeta[c] += s1; dgamma[c] += s2;
}

// z = (y - mean) * rstd * gamma + beta (+ residual) (ReLU)
__global__ void __launch_bounds__(256)
bn_apply_kernel(const uint4* __restrict__ y, const float* __restrict__ mean, const float* __restrict__ rstd,
                const __nv_bfloat16* __restrict__ gamma, const __nv_bfloat16* __restrict__ beta,
                const uint4* __restrict__ residual, uint4* __restrict__ z, long long rows, int C, int relu) {
  const int chunks = C >> 3;
  const long long gthreads = (long long)gridDim.x * blockDim.x;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cc = (int)(g % chunks);
  float sc[8], sh[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float ga = __bfloat162float(gamma[cc * 8 + i]), r = rstd[cc * 8 + i];
    sc[i] = ga * r;
    sh[i] = __bfloat162float(beta[cc * 8 + i]) - mean[cc * 8 + i] * ga * r;
  }
  const long long total = rows * chunks;
  for (long long e = g; e < total; e += gthreads) {      // gthreads % chunks == 0: the chunk stays cc
    float v[8];
    unpack8(__ldg(y + e), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = v[i] * sc[i] + sh[i];
    if (residual) {
      float rr[8];
      unpack8(__ldg(residual + e), rr);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += rr[i];
    }
    if (relu) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = fmaxf(v[i], 0.f);
    }
    z[e] = pack8(v);
  }
}

// dy = gamma * rstd * (dz' - s1 / rows - yhat * s2 / rows); dres = dz' (the masked gradient that
// also flows into the residual branch)
__global__ void __launch_bounds__(256)
bn_bwd_apply_kernel(const uint4* __restrict__ dz, const uint4* __restrict__ zz, const uint4* __restrict__ yy,
                    const float* __restrict__ mean, const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ gamma,
                    const float* __restrict__ sums, uint4* __restrict__ dy, uint4* __restrict__ dres, long long rows, int C,
                    int relu, float inv_rows) {
  const int chunks = C >> 3;
  const long long gthreads = (long long)gridDim.x * blockDim.x;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int cc = (int)(g % chunks);
  float mu[8], rs[8], k0[8], m1[8], m2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    mu[i] = mean[cc * 8 + i]; rs[i] = rstd[cc * 8 + i];
    k0[i] = __bfloat162float(gamma[cc * 8 + i]) * rs[i];
    m1[i] = sums[cc * 8 + i] * inv_rows; m2[i] = sums[C + cc * 8 + i] * inv_rows;
  }
  const long long total = rows * chunks;
  for (long long e = g; e < total; e += gthreads) {
    float v[8], y[8];
    unpack8(__ldg(dz + e), v);
    unpack8(__ldg(yy + e), y);
    if (relu) {
      float z[8];
      unpack8(__ldg(zz + e), z);
#pragma unroll
      for (int i = 0; i < 8; ++i) if (!(z[i] > 0.f)) v[i] = 0.f;
    }
    if (dres) dres[e] = pack8(v);
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = k0[i] * (v[i] - m1[i] - (y[i] - mu[i]) * rs[i] * m2[i]);
    dy[e] = pack8(o);
  }
}

bool bad_bn(long long rows, int C) { return rows <= 0 || C < 8 || (C & 7) || (256 % (C >> 3)) != 0; }

int bn_grid(long long rows, int C) {
  long long blocks = (rows * (C >> 3) + 256 * 8 - 1) / (256 * 8);
  const long long cap = (long long)bb_num_sms() * 4;
  if (blocks > cap) blocks = cap;
  return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace

extern "C" long long bb_bn_workspace_bytes(long long rows, int C) {
  if (bad_bn(rows, C)) return -1;
  // partial rows of the reduction plus the two per-channel sums the backward pass keeps
  return ((long long)bn_grid(rows, C) * 2 * C + 2 * C) * (long long)sizeof(float);
}

extern "C" int bb_bn_stats(const void* y, long long rows, int C, float eps, float* mean, float* rstd, void* workspace,
                           long long workspace_bytes, void* stream) {
  if (!y || !mean || !rstd || !workspace || bad_bn(rows, C) || workspace_bytes < bb_bn_workspace_bytes(rows, C) ||
      ((uintptr_t)y & 15)) {
    bb_set_last_error_msg("bb_bn_stats: null/unaligned pointer, workspace too small, or channels not 8 x a power of two <= 2048");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = bn_grid(rows, C);
  float* ws = static_cast<float*>(workspace);
  bn_reduce_kernel<RED_STATS><<<grid, 256, 0, s>>>((const uint4*)y, nullptr, nullptr, nullptr, nullptr, 0, rows, C, ws);
  bn_finish_stats_kernel<<<(C + 127) / 128, 128, 0, s>>>(ws, grid, C, 1.0f / (float)rows, eps, mean, rstd);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_bn_apply(const void* y, const float* mean, const float* rstd, const void* gamma, const void* beta,
                           const void* residual, void* z, long long rows, int C, int relu, void* stream) {
  if (!y || !mean || !rstd || !gamma || !beta || !z || bad_bn(rows, C) || ((uintptr_t)y & 15) || ((uintptr_t)z & 15) ||
      ((uintptr_t)residual & 15)) {
    bb_set_last_error_msg("bb_bn_apply: null/unaligned pointer or channels not 8 x a power of two <= 2048");
    return BB_ERR_INVALID_ARG;
  }
  bn_apply_kernel<<<bn_grid(rows, C), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)y, mean, rstd, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, (const uint4*)residual, (uint4*)z,
      rows, C, relu);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_bn_bwd(const void* dz, const void* z, const void* y, const float* mean, const float* rstd, const void* gamma,
                         void* dy, void* dres, float* dgamma, float* dbeta, long long rows, int C, int relu, void* workspace,
                         long long workspace_bytes, void* stream) {
  if (!dz || !y || !mean || !rstd || !gamma || !dy || !dgamma || !dbeta || !workspace || (relu && !z) || bad_bn(rows, C) ||
      workspace_bytes < bb_bn_workspace_bytes(rows, C) ||
      (((uintptr_t)dz | (uintptr_t)z | (uintptr_t)y | (uintptr_t)dy | (uintptr_t)dres) & 15)) {
    bb_set_last_error_msg("bb_bn_bwd: null/unaligned pointer, workspace too small, or channels not 8 x a power of two <= 2048");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = bn_grid(rows, C);
  float* ws = static_cast<float*>(workspace);
  float* sums = ws + (long long)grid * 2 * C;
  bn_reduce_kernel<RED_BWD><<<grid, 256, 0, s>>>((const uint4*)dz, (const uint4*)z, (const uint4*)y, mean, rstd, relu, rows, C, ws);
  bn_finish_bwd_kernel<<<(C + 127) / 128, 128, 0, s>>>(ws, grid, C, sums, dgamma, dbeta);
  bn_bwd_apply_kernel<<<grid, 256, 0, s>>>((const uint4*)dz, (const uint4*)z, (const uint4*)y, mean, rstd,
                                           (const __nv_bfloat16*)gamma, sums, (uint4*)dy, (uint4*)dres, rows, C, relu,
                                           1.0f / (float)rows);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

// ---------------------------------------------------------------------------------- pooling
namespace {

// 3 x 3 window, stride 2, padding 1.  The position of the maximum inside the window (0..8, first
// one in row-major window order wins a tie, like the framework's scan) is kept per output
// element, so the backward pass routes the gradient to exactly that input.
__global__ void __launch_bounds__(256)
maxpool_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, uint2* __restrict__ argmax, int N, int H, int W, int C,
                   int Ho, int Wo) {
  const int chunks = C >> 3;
  const long long total = (long long)N * Ho * Wo * chunks;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int cc = (int)(e % chunks);
    const long long p = e / chunks;
    const int wo = (int)(p % Wo);
    const long long t = p / Wo;
    const int ho = (int)(t % Ho), n = (int)(t / Ho);
    float best[8];
    unsigned int where[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { best[i] = -INFINITY; where[i] = 0; }
    for (int r = 0; r < 3; ++r) {
      const int h = 2 * ho - 1 + r;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < 3; ++s) {
        const int w = 2 * wo - 1 + s;
        if (w < 0 || w >= W) continue;
        float v[8];
        unpack8(__ldg(x + (((long long)n * H + h) * W + w) * chunks + cc), v);
#pragma unroll
        for (int i = 0; i < 8; ++i) if (v[i] > best[i] || best[i] == -INFINITY) { best[i] = v[i]; where[i] = r * 3 + s; }
      }
    }
    y[e] = pack8(best);
    uint2 a;
    a.x = where[0] | (where[1] << 8) | (where[2] << 16) | (where[3] << 24);
    a.y = where[4] | (where[5] << 8) | (where[6] << 16) | (where[7] << 24);
    argmax[e] = a;
  }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_kernel(const uint4* __restrict__ dy, const uint2* __restrict__ argmax, uint4* __restrict__ dx, int N, int H, int W,
                   int C, int Ho, int Wo) {
  const int chunks = C >> 3;
  const long long total = (long long)N * H * W * chunks;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int cc = (int)(e % chunks);
    const long long pix = e / chunks;
    const int w = (int)(pix % W);
    const long long t = pix / W;
    const int h = (int)(t % H), n = (int)(t / H);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < 3; ++r) {
      const int hs = h + 1 - r;
      if (hs < 0 || (hs & 1)) continue;
      const int ho = hs >> 1;
      if (ho >= Ho) continue;
      for (int s = 0; s < 3; ++s) {
        const int ws = w + 1 - s;
        if (ws < 0 || (ws & 1)) continue;
        const int wo = ws >> 1;
        if (wo >= Wo) continue;
        const long long o = (((long long)n * Ho + ho) * Wo + wo) * chunks + cc;
        const uint2 a = __ldg(argmax + o);
        float g[8];
        unpack8(__ldg(dy + o), g);
        const unsigned int tap = r * 3 + s;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const unsigned int wi = ((i < 4 ? a.x : a.y) >> (8 * (i & 3))) & 0xFFu;
          if (wi == tap) acc[i] += g[i];
        }
      }
    }
    dx[e] = pack8(acc);
  }
}

// y[n, c] = mean over the hw pixels of x[n, :, c]
__global__ void __launch_bounds__(256)
avgpool_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int N, int HW, int C) {
  const int chunks = C >> 3;
  const long long total = (long long)N * chunks;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int cc = (int)(e % chunks), n = (int)(e / chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < HW; ++p) {
      float v[8];
      unpack8(__ldg(x + ((long long)n * HW + p) * chunks + cc), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += v[i];
    }
    const float inv = 1.0f / (float)HW;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= inv;
    y[e] = pack8(acc);
  }
}

__global__ void __launch_bounds__(256)
avgpool_bwd_kernel(const uint4* __restrict__ dy, uint4* __restrict__ dx, int N, int HW, int C) {
  const int chunks = C >> 3;
  const long long total = (long long)N * HW * chunks;
  const float inv = 1.0f / (float)HW;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
    const int cc = (int)(e % chunks);
    const int n = (int)(e / ((long long)HW * chunks));
    float v[8];
    unpack8(__ldg(dy + (long long)n * chunks + cc), v);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] *= inv;
    dx[e] = pack8(v);
  }
}

}  // namespace

extern "C" int bb_maxpool3x3s2_fwd(const void* x, void* y, void* argmax, int N, int H, int W, int C, void* stream) {
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  if (!x || !y || !argmax || N <= 0 || H <= 0 || W <= 0 || C <= 0 || (C & 7) ||
      (((uintptr_t)x | (uintptr_t)y) & 15) || ((uintptr_t)argmax & 7)) {
    bb_set_last_error_msg("bb_maxpool3x3s2_fwd: null/unaligned pointer or channels not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  maxpool_fwd_kernel<<<flat_grid((long long)N * Ho * Wo * (C >> 3)), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)x, (uint4*)y, (uint2*)argmax, N, H, W, C, Ho, Wo);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_maxpool3x3s2_bwd(const void* dy, const void* argmax, void* dx, int N, int H, int W, int C, void* stream) {
  const int Ho = (H + 2 - 3) / 2 + 1, Wo = (W + 2 - 3) / 2 + 1;
  if (!dy || !dx || !argmax || N <= 0 || H <= 0 || W <= 0 || C <= 0 || (C & 7) ||
      (((uintptr_t)dx | (uintptr_t)dy) & 15) || ((uintptr_t)argmax & 7)) {
    bb_set_last_error_msg("bb_maxpool3x3s2_bwd: null/unaligned pointer or channels not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  maxpool_bwd_kernel<<<flat_grid((long long)N * H * W * (C >> 3)), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)dy, (const uint2*)argmax, (uint4*)dx, N, H, W, C, Ho, Wo);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream) {
  if (!x || !y || N <= 0 || HW <= 0 || C <= 0 || (C & 7) || (((uintptr_t)x | (uintptr_t)y) & 15)) {
    bb_set_last_error_msg("bb_avgpool_fwd: null/unaligned pointer or channels not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  avgpool_fwd_kernel<<<flat_grid((long long)N * (C >> 3)), 256, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)y, N, HW, C);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream) {
  if (!dy || !dx || N <= 0 || HW <= 0 || C <= 0 || (C & 7) || (((uintptr_t)dx | (uintptr_t)dy) & 15)) {
    bb_set_last_error_msg("bb_avgpool_bwd: null/unaligned pointer or channels not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  avgpool_bwd_kernel<<<flat_grid((long long)N * HW * (C >> 3)), 256, 0, (cudaStream_t)stream>>>((const uint4*)dy, (uint4*)dx, N, HW, C);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

// ---------------------------------------------------------------------------------- one call per layer
// Convolution + batch norm (+ residual, + ReLU) forward and backward with every kernel issued from
// one foreign call: a ResNet-152 step has ~2500 such layers-times-micro-batches, and a Python host
// that pays per kernel becomes the bottleneck.  Same kernels and order as calling the entry points
// above one by one.
namespace {

inline long long up256(long long n) { return (n + 255) & ~255LL; }

struct ConvSizes {
  int Ho, Wo;
  long long P, K;
  bool direct;                       // 1 x 1 / stride 1: the activation tensor is the patch matrix
  long long col_bytes, dy_bytes, dcol_bytes, bn_bytes;
};

bool conv_sizes(const bb_conv_desc* d, ConvSizes* s) {
  if (!d || d->N <= 0 || d->H <= 0 || d->W <= 0 || d->Cin <= 0 || (d->Cin & 7) || d->Cout <= 0 || d->k <= 0 || d->stride <= 0 ||
      d->pad < 0 || !d->w || !d->gamma || !d->beta)
    return false;
  s->Ho = (d->H + 2 * d->pad - d->k) / d->stride + 1;
  s->Wo = (d->W + 2 * d->pad - d->k) / d->stride + 1;
  if (s->Ho <= 0 || s->Wo <= 0) return false;
  s->P = (long long)d->N * s->Ho * s->Wo;
  s->K = (long long)d->k * d->k * d->Cin;
  s->direct = d->k == 1 && d->stride == 1;
  s->bn_bytes = bb_bn_workspace_bytes(s->P, d->Cout);
  if (s->bn_bytes < 0) return false;
  s->col_bytes = s->direct ? 0 : up256(s->P * s->K * 2);
  s->dy_bytes = up256(s->P * d->Cout * 2);
  s->dcol_bytes = s->direct ? 0 : up256(s->P * s->K * 2);
  s->bn_bytes = up256(s->bn_bytes);
  return true;
}

int conv_gemm(const bb_conv_desc* d, int M, int N, int K, const void* A, long long lda, int a_mn, const void* B, long long ldb,
              int b_mn, void* D, long long ldd, int epi, void* stream) {
  bb_gemm_desc g = {};
  g.M = M; g.N = N; g.K = K; g.A = A; g.lda = lda; g.a_mn_major = a_mn; g.B = B; g.ldb = ldb; g.b_mn_major = b_mn;
  g.D = D; g.ldd = ldd; g.epilogue = epi; g.max_ctas = d->max_ctas;
  return bb_gemm_bf16(&g, stream);
}

#define BB_TRY(expr) do { int _rc = (expr); if (_rc != BB_OK) return _rc; } while (0)

}  // namespace

extern "C" long long bb_conv_bn_scratch_bytes(const bb_conv_desc* d, int backward, int need_dx) {
  ConvSizes s;
  if (!conv_sizes(d, &s)) return -1;
  if (!backward) return s.col_bytes + s.bn_bytes;
  return s.dy_bytes + s.col_bytes + (need_dx ? s.dcol_bytes : 0) + s.bn_bytes;
}

extern "C" int bb_conv_bn_fwd(const bb_conv_desc* d, const void* x, const void* residual, void* y, void* z, float* mean,
                              float* rstd, void* scratch, long long scratch_bytes, void* stream) {
  ConvSizes s;
  if (!conv_sizes(d, &s) || !x || !y || !z || !mean || !rstd || !scratch || scratch_bytes < s.col_bytes + s.bn_bytes) {
    bb_set_last_error_msg("bb_conv_bn_fwd: bad descriptor, null buffer or scratch smaller than bb_conv_bn_scratch_bytes");
    return BB_ERR_INVALID_ARG;
  }
  uint8_t* sc = static_cast<uint8_t*>(scratch);
  const void* col = x;
  if (!s.direct) {
    BB_TRY(bb_im2col_nhwc(x, sc, d->N, d->H, d->W, d->Cin, d->k, d->stride, d->pad, s.Ho, s.Wo, s.K, stream));
    col = sc;
  }
  BB_TRY(conv_gemm(d, (int)s.P, d->Cout, (int)s.K, col, s.K, 0, d->w, s.K, 0, y, d->Cout, BB_EPI_STORE, stream));
  BB_TRY(bb_bn_stats(y, s.P, d->Cout, d->eps, mean, rstd, sc + s.col_bytes, s.bn_bytes, stream));
  BB_TRY(bb_bn_apply(y, mean, rstd, d->gamma, d->beta, residual, z, s.P, d->Cout, d->relu, stream));
  return BB_OK;
}

extern "C" int bb_conv_bn_bwd(const bb_conv_desc* d, const void* x, const void* y, const void* z, const float* mean,
                              const float* rstd, const void* dz, void* dx, void* dres, void* scratch, long long scratch_bytes,
                              void* stream) {
  ConvSizes s;
  if (!conv_sizes(d, &s) || !x || !y || !z || !mean || !rstd || !dz || !scratch || !d->g_w || !d->g_gamma || !d->g_beta ||
      scratch_bytes < bb_conv_bn_scratch_bytes(d, 1, dx != nullptr)) {
    bb_set_last_error_msg("bb_conv_bn_bwd: bad descriptor, null buffer, missing gradient pointer or scratch too small");
    return BB_ERR_INVALID_ARG;
  }
  uint8_t* sc = static_cast<uint8_t*>(scratch);
  void* dy = sc;
  uint8_t* colbuf = sc + s.dy_bytes;
  uint8_t* dcolbuf = colbuf + s.col_bytes;
  uint8_t* bnws = dcolbuf + (dx ? s.dcol_bytes : 0);
  BB_TRY(bb_bn_bwd(dz, z, y, mean, rstd, d->gamma, dy, dres, d->g_gamma, d->g_beta, s.P, d->Cout, d->relu, bnws, s.bn_bytes, stream));
  const void* col = x;
  if (!s.direct) {
    BB_TRY(bb_im2col_nhwc(x, colbuf, d->N, d->H, d->W, d->Cin, d->k, d->stride, d->pad, s.Ho, s.Wo, s.K, stream));
    col = colbuf;
  }
  // dW[Cout, K] += dy^T patches
  BB_TRY(conv_gemm(d, d->Cout, (int)s.K, (int)s.P, dy, d->Cout, 1, col, s.K, 1, d->g_w, s.K, BB_EPI_ACCUM_F32, stream));
  if (dx) {
    void* dcol = s.direct ? dx : (void*)dcolbuf;
    BB_TRY(conv_gemm(d, (int)s.P, (int)s.K, d->Cout, dy, d->Cout, 0, d->w, s.K, 1, dcol, s.K, BB_EPI_STORE, stream));
    if (!s.direct)
      BB_TRY(bb_col2im_nhwc(dcol, dx, d->N, d->H, d->W, d->Cin, d->k, d->stride, d->pad, s.Ho, s.Wo, s.K, stream));
  }
  return BB_OK;
}
