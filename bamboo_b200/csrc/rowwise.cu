// HBM-bound row-wise kernels of a transformer stage: LayerNorm forward/backward (with the
// residual gradient folded in), bias-gradient column sums, token+position embedding
// gather and its gradient scatter.  All loads/stores are 16-byte vectors; one warp owns a
// row so no block-level synchronisation is needed on the hot loops; grids are sized as a
// multiple of the SM count and stride over rows.
#include "common.cuh"
#include <stdio.h>
#include <stdlib.h>

namespace {

constexpr int WARPS = 8;              // warps per CTA for warp-per-row kernels
constexpr int CTAS_PER_SM = 4;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

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

// ------------------------------------------------------------------ LayerNorm forward
// y = (x - mean) * rstd * gamma + beta ; statistics in fp32 (biased variance, eps inside sqrt)
__global__ void __launch_bounds__(WARPS * 32)
layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gamma,
                     const __nv_bfloat16* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int h, float eps) {
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * WARPS + (threadIdx.x >> 5);
  const int warp_stride = gridDim.x * WARPS;
  const int nch = h >> 3;
  for (int row = warp_global; row < rows; row += warp_stride) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    float s = 0.f;
    for (int c = lane; c < nch; c += 32) {
      float f[8]; unpack8(xr[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += f[i];
    }
    const float mean = warp_sum(s) / (float)h;
    float v = 0.f;
    for (int c = lane; c < nch; c += 32) {   // second pass hits L1
      float f[8]; unpack8(xr[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { float d = f[i] - mean; v += d * d; }
    }
    const float rstd = rsqrtf(warp_sum(v) / (float)h + eps);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * h);
    for (int c = lane; c < nch; c += 32) {
      float f[8], g[8], b[8];
      unpack8(xr[c], f);
      unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + c), g);
      unpack8(__ldg(reinterpret_cast<const uint4*>(beta) + c), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = (f[i] - mean) * rstd * g[i] + b[i];
      yr[c] = pack8(f);
    }
    if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
  }
}

// ------------------------------------------------------------------ LayerNorm backward
// dx = rstd * (dy*gamma - mean(dy*gamma) - xhat * mean(dy*gamma*xhat)) [+ dres]
// Per-CTA partial sums of dgamma = sum dy*xhat and dbeta = sum dy go to `partials`
// ([gridDim.x][2][h] fp32); reduce_partials_kernel folds them into the fp32 gradients.
__global__ void __launch_bounds__(WARPS * 32)
layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                     const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                     const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                     __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int rows, int h) {
  extern __shared__ float acc[];  // [warps][2][h], each lane owns its own columns
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  const int nch = h >> 3;
  float* my_g = acc + (size_t)warp * 2 * h;
  float* my_b = my_g + h;
  for (int c = lane; c < nch; c += 32)
#pragma unroll
    for (int i = 0; i < 8; ++i) { my_g[c * 8 + i] = 0.f; my_b[c * 8 + i] = 0.f; }
  const int warp_global = blockIdx.x * nwarps + warp;
  const int warp_stride = gridDim.x * nwarps;
  for (int row = warp_global; row < rows; row += warp_stride) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * h);
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    const float mean = mean_in[row], rstd = rstd_in[row];
    float s1 = 0.f, s2 = 0.f;
    for (int c = lane; c < nch; c += 32) {
      float d[8], f[8], g[8];
      unpack8(dyr[c], d); unpack8(xr[c], f);
      unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + c), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) { float t = d[i] * g[i]; s1 += t; s2 += t * (f[i] - mean) * rstd; }
    }
    const float c1 = warp_sum(s1) / (float)h, c2 = warp_sum(s2) / (float)h;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * h);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * h) : nullptr;
    for (int c = lane; c < nch; c += 32) {
      float d[8], f[8], g[8], o[8];
      unpack8(dyr[c], d); unpack8(xr[c], f);
      unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + c), g);
      float r[8];
      if (rr) unpack8(rr[c], r);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (f[i] - mean) * rstd;
        o[i] = rstd * (d[i] * g[i] - c1 - xh * c2) + (rr ? r[i] : 0.f);
        my_g[c * 8 + i] += d[i] * xh;
        my_b[c * 8 + i] += d[i];
      }
      dxr[c] = pack8(o);
    }
  }
  __syncthreads();
  float* out = partials + (size_t)blockIdx.x * 2 * h;
  for (int j = threadIdx.x; j < 2 * h; j += blockDim.x) {
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += acc[(size_t)w * 2 * h + j];
    out[j] = s;
  }
}

// Same computation with the per-lane dgamma/dbeta partial sums and the row's data held in
// registers (hidden sizes that are a multiple of 256 up to 1024): shared memory is only touched
// once per CTA, when the warps' partials are combined.
template <int NCH>
__global__ void __launch_bounds__(WARPS * 32)
layernorm_bwd_reg_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                         const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                         const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                         __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int rows) {
  constexpr int h = NCH * 256;
  extern __shared__ float acc[];  // [warps][2][h]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = blockDim.x >> 5;
  float ag[NCH * 8], ab[NCH * 8], g[NCH * 8];
#pragma unroll
  for (int j = 0; j < NCH; ++j) {
    unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + lane + 32 * j), g + 8 * j);
#pragma unroll
    for (int i = 0; i < 8; ++i) { ag[8 * j + i] = 0.f; ab[8 * j + i] = 0.f; }
  }
  for (int row = blockIdx.x * nwarps + warp; row < rows; row += gridDim.x * nwarps) {
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + (size_t)row * h);
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * h);
    const float mean = mean_in[row], rstd = rstd_in[row];
    uint4 qd[NCH], qx[NCH];
#pragma unroll
    for (int j = 0; j < NCH; ++j) { qd[j] = dyr[lane + 32 * j]; qx[j] = xr[lane + 32 * j]; }
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float d[8], f[8];
      unpack8(qd[j], d); unpack8(qx[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float t = d[i] * g[8 * j + i]; s1 += t; s2 += t * (f[i] - mean) * rstd; }
    }
    const float c1 = warp_sum(s1) * (1.f / h), c2 = warp_sum(s2) * (1.f / h);
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * h);
    const uint4* rr = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * h) : nullptr;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float d[8], f[8], o[8], r[8];
      unpack8(qd[j], d); unpack8(qx[j], f);
      if (rr) unpack8(rr[lane + 32 * j], r);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (f[i] - mean) * rstd;
        o[i] = rstd * (d[i] * g[8 * j + i] - c1 - xh * c2) + (rr ? r[i] : 0.f);
        ag[8 * j + i] += d[i] * xh;
        ab[8 * j + i] += d[i];
      }
      dxr[lane + 32 * j] = pack8(o);
    }
  }
  float* my_g = acc + (size_t)warp * 2 * h;
  float* my_b = my_g + h;
#pragma unroll
  for (int j = 0; j < NCH; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) { my_g[(lane + 32 * j) * 8 + i] = ag[8 * j + i]; my_b[(lane + 32 * j) * 8 + i] = ab[8 * j + i]; }
  __syncthreads();
  float* out = partials + (size_t)blockIdx.x * 2 * h;
  for (int j = threadIdx.x; j < 2 * h; j += blockDim.x) {
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += acc[(size_t)w * 2 * h + j];
    out[j] = s;
  }
}

// Column-owner variant (hidden sizes that are a multiple of 256, up to 8192): a thread owns 8
// columns of one of `slots` row slots; its dgamma/dbeta partial sums are 16 registers, so several
// CTAs fit on an SM and every thread keeps 2 x LNB_R 16-byte loads in flight (the warp-per-row
// kernels hold a whole row's partial sums per warp, run one CTA per SM and are latency-bound at
// about a third of the HBM rate).  The two row sums of LNB_R rows per slot are combined across
// the slot's warps through double-buffered shared memory: one block barrier per 8 rows.
constexpr int LNB_R = 4;
template <int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT <= 256 ? 2 : 1)
layernorm_bwd_cols_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                          const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                          const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                          __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int rows, int h, int slots) {
  extern __shared__ float sm[];
  const int tpr = h >> 3;                          // threads per row
  const int wps = tpr >> 5;                        // warps per slot
  const int slot = threadIdx.x / tpr, tc = threadIdx.x - slot * tpr;   // my slot, my 8-column group
  const int lane = threadIdx.x & 31, wis = tc >> 5;
  float* red = sm;                                 // [2][slots][wps][2 * LNB_R]
  float* fin = sm + 2 * slots * wps * 2 * LNB_R;   // [slots][2][h] final combination
  float g[8], ag[8], ab[8];
  unpack8(__ldg(reinterpret_cast<const uint4*>(gamma) + tc), g);
#pragma unroll
  for (int i = 0; i < 8; ++i) { ag[i] = 0.f; ab[i] = 0.f; }
  const float inv_h = 1.f / h;
  int buf = 0;
  for (int base = blockIdx.x * slots * LNB_R; base < rows; base += gridDim.x * slots * LNB_R) {
    const int r0 = base + slot * LNB_R;
    uint4 qd[LNB_R], qx[LNB_R];
    float mean[LNB_R], rstd[LNB_R];
#pragma unroll
    for (int r = 0; r < LNB_R; ++r) {
      const int row = r0 + r;
      if (row < rows) {
        qd[r] = reinterpret_cast<const uint4*>(dy + (size_t)row * h)[tc];
        qx[r] = reinterpret_cast<const uint4*>(x + (size_t)row * h)[tc];
        mean[r] = mean_in[row]; rstd[r] = rstd_in[row];
      } else {
        qd[r] = make_uint4(0, 0, 0, 0); qx[r] = qd[r]; mean[r] = 0.f; rstd[r] = 0.f;
      }
    }
    float s[2 * LNB_R];
#pragma unroll
    for (int r = 0; r < LNB_R; ++r) {
      float d[8], f[8];
      unpack8(qd[r], d); unpack8(qx[r], f);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float t = d[i] * g[i]; s1 += t; s2 += t * (f[i] - mean[r]) * rstd[r]; }
      s[2 * r] = s1; s[2 * r + 1] = s2;
    }
#pragma unroll
    for (int k = 0; k < 2 * LNB_R; ++k) s[k] = warp_sum(s[k]);
    float* my = red + ((buf * slots + slot) * wps + wis) * 2 * LNB_R;
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < 2 * LNB_R; ++k) my[k] = s[k];
    }
    __syncthreads();
    const float* all = red + (buf * slots + slot) * wps * 2 * LNB_R;
#pragma unroll
    for (int k = 0; k < 2 * LNB_R; ++k) {
      float t = 0.f;
      for (int w = 0; w < wps; ++w) t += all[w * 2 * LNB_R + k];    // fixed order
      s[k] = t * inv_h;
    }
    buf ^= 1;
#pragma unroll
    for (int r = 0; r < LNB_R; ++r) {
      const int row = r0 + r;
      if (row >= rows) continue;
      float d[8], f[8], o[8], rr[8];
      unpack8(qd[r], d); unpack8(qx[r], f);
      if (dres) unpack8(reinterpret_cast<const uint4*>(dres + (size_t)row * h)[tc], rr);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (f[i] - mean[r]) * rstd[r];
        o[i] = rstd[r] * (d[i] * g[i] - s[2 * r] - xh * s[2 * r + 1]) + (dres ? rr[i] : 0.f);
        ag[i] += d[i] * xh;
        ab[i] += d[i];
      }
      reinterpret_cast<uint4*>(dx + (size_t)row * h)[tc] = pack8(o);
    }
  }
  // combine the slots' column sums (fixed order) and write this CTA's partial row
  float* mine = fin + (size_t)slot * 2 * h;
#pragma unroll
  for (int i = 0; i < 8; ++i) { mine[tc * 8 + i] = ag[i]; mine[h + tc * 8 + i] = ab[i]; }
  __syncthreads();
  float* out = partials + (size_t)blockIdx.x * 2 * h;
  for (int j = threadIdx.x; j < 2 * h; j += blockDim.x) {
    float t = 0.f;
    for (int q = 0; q < slots; ++q) t += fin[(size_t)q * 2 * h + j];
    out[j] = t;
  }
}

// out[j] += sum_p partials[p * stride + j].  A 32-column x 8-way block: eight threads share
// a column, each sums every eighth partial, shared memory combines them in a fixed order
// (deterministic).
// blockIdx.y selects one of two (partials, out) pairs, `pair_offset` floats apart in `partials`
// (LayerNorm: dgamma and dbeta in one launch).
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partials, float* __restrict__ out0, float* __restrict__ out1,
                       long long pair_offset, int nparts, int n, long long stride) {
  __shared__ float red[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float* out = blockIdx.y ? out1 : out0;
  partials += blockIdx.y * pair_offset;
  float s = 0.f;
  if (j < n)
    for (int p = ty; p < nparts; p += 8) s += partials[(size_t)p * stride + j];
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < n) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][tx];
    out[j] += t;
  }
}

// ------------------------------------------------------------------ bias gradient
// partials[split][n] = sum over this split's rows of dy[row][n]
__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ partials, int rows, int n, long long ld, int rows_per_split) {
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_split;
  const int r1 = min(rows, r0 + rows_per_split);
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col0 < n) {
    for (int r = r0 + warp; r < r1; r += 8) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(dy + (size_t)r * ld + col0), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s[i] += f[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = s[i];
  __syncthreads();
  const int j = threadIdx.x, col = blockIdx.x * 256 + j;
  if (col < n) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][j];
    partials[(size_t)blockIdx.y * n + col] = t;
  }
}

// ------------------------------------------------------------------ GeLU backward (stand-alone)
// dx = dy * gelu'(pre), tanh form; 8 bf16 per thread.  The transformer blocks get this fused into
// the input-gradient GEMM's epilogue; it stands alone where the activation is followed by a
// LayerNorm instead of a GEMM (masked-LM head transform).
__global__ void __launch_bounds__(256)
gelu_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ dx, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float d[8], x[8], o[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(dy) + i), d);
    unpack8(__ldg(reinterpret_cast<const uint4*>(pre) + i), x);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = d[k] * bb::gelu_tanh_grad(x[k]);
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

// ------------------------------------------------------------------ embedding
// out[t,:] = wte[tok[t],:] + wpe[t % seq,:]
__global__ void __launch_bounds__(WARPS * 32)
embedding_fwd_kernel(const long long* __restrict__ tok, const __nv_bfloat16* __restrict__ wte,
                     const __nv_bfloat16* __restrict__ wpe, __nv_bfloat16* __restrict__ out, int tokens, int seq, int h,
                     int vocab, int* status) {
  const int lane = threadIdx.x & 31;
  const int nch = h >> 3;
  for (int t = blockIdx.x * WARPS + (threadIdx.x >> 5); t < tokens; t += gridDim.x * WARPS) {
    long long id = tok[t];
    if (id < 0 || id >= vocab) { if (lane == 0) atomicCAS(status, 0, BB_ERR_INVALID_ARG); id = 0; }
    const uint4* e = reinterpret_cast<const uint4*>(wte + (size_t)id * h);
    const uint4* p = wpe ? reinterpret_cast<const uint4*>(wpe + (size_t)(t % seq) * h) : nullptr;
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)t * h);
    for (int c = lane; c < nch; c += 32) {
      float a[8], b[8];
      unpack8(__ldg(e + c), a);
      if (p) { unpack8(__ldg(p + c), b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] += b[i]; }
      o[c] = pack8(a);
    }
  }
}

// dwte[tok[t],:] += dout[t,:] ; dwpe[t % seq,:] += dout[t,:]   (fp32 gradients, vector atomics)
__global__ void __launch_bounds__(WARPS * 32)
embedding_bwd_kernel(const long long* __restrict__ tok, const __nv_bfloat16* __restrict__ dout, float* __restrict__ dwte,
                     float* __restrict__ dwpe, int tokens, int seq, int h, int vocab) {
  const int lane = threadIdx.x & 31;
  const int nch = h >> 3;
  for (int t = blockIdx.x * WARPS + (threadIdx.x >> 5); t < tokens; t += gridDim.x * WARPS) {
    long long id = tok[t];
    if (id < 0 || id >= vocab) continue;
    const uint4* d = reinterpret_cast<const uint4*>(dout + (size_t)t * h);
    float4* ge = reinterpret_cast<float4*>(dwte + (size_t)id * h);
    float4* gp = dwpe ? reinterpret_cast<float4*>(dwpe + (size_t)(t % seq) * h) : nullptr;
    for (int c = lane; c < nch; c += 32) {
      float f[8]; unpack8(d[c], f);
      const float4 lo = make_float4(f[0], f[1], f[2], f[3]), hi = make_float4(f[4], f[5], f[6], f[7]);
      atomicAdd(ge + 2 * c, lo); atomicAdd(ge + 2 * c + 1, hi);
      if (gp) { atomicAdd(gp + 2 * c, lo); atomicAdd(gp + 2 * c + 1, hi); }
    }
  }
}

int row_grid(int rows) {
  long long want = ((long long)rows + WARPS - 1) / WARPS;
  long long cap = (long long)bb_num_sms() * CTAS_PER_SM;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace

extern "C" int bb_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                                int rows, int h, float eps, void* stream) {
  if (!x || !gamma || !beta || !y || !mean || !rstd || rows <= 0 || h <= 0 || (h & 7)) {
    bb_set_last_error_msg("bb_layernorm_fwd: null pointer or hidden size not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  layernorm_fwd_kernel<<<row_grid(rows), WARPS * 32, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta, (__nv_bfloat16*)y, mean, rstd, rows, h, eps);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

namespace {
int ln_bwd_warps(int h) {
  int w = (int)((200 * 1024) / ((size_t)2 * h * sizeof(float)));
  return w > WARPS ? WARPS : w;
}
// column-owner kernel: hidden size a multiple of 256 and at most 8192 (1024 threads per row slot)
bool ln_bwd_cols_ok(int h) {
  static int off = -1;
  if (off < 0) { const char* e = getenv("BB_LN_BWD_ROWS"); off = (e && e[0] == '1') ? 1 : 0; }   // 1: warp-per-row kernels
  return !off && h % 256 == 0 && h <= 8192;
}
int ln_bwd_cols_slots(int h) { const int tpr = h / 8; return tpr >= 256 ? 1 : 256 / tpr; }
int ln_bwd_grid(int rows, int h) {
  if (ln_bwd_cols_ok(h)) {
    const int per = ln_bwd_cols_slots(h) * LNB_R;
    long long want = ((long long)rows + per - 1) / per, cap = 2LL * bb_num_sms();
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
  }
  const int w = ln_bwd_warps(h);
  long long want = ((long long)rows + w - 1) / w;
  long long cap = (long long)bb_num_sms() * (w * 2 * h * 4 > 100 * 1024 ? 1 : 2);
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}
}  // namespace

namespace {
// launches the backward main kernel (register variant when the hidden size allows it)
int ln_bwd_main(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                void* dx, float* ws, int rows, int h, int grid, int warps, cudaStream_t s) {
  if (ln_bwd_cols_ok(h)) {
    const int slots = ln_bwd_cols_slots(h), tpr = h / 8;
    const size_t sm_bytes = ((size_t)2 * slots * (tpr / 32) * 2 * LNB_R + (size_t)slots * 2 * h) * sizeof(float);
    BB_ONCE_PER_DEVICE({
      BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_cols_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
      BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_cols_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
      BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_cols_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024));
    });
    const int threads = slots * tpr;
#define BB_LNC_ARGS (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd, \
                    (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, ws, rows, h, slots
    if (threads <= 256) layernorm_bwd_cols_kernel<256><<<grid, threads, sm_bytes, s>>>(BB_LNC_ARGS);
    else if (threads <= 512) layernorm_bwd_cols_kernel<512><<<grid, threads, sm_bytes, s>>>(BB_LNC_ARGS);
    else layernorm_bwd_cols_kernel<1024><<<grid, threads, sm_bytes, s>>>(BB_LNC_ARGS);
#undef BB_LNC_ARGS
    BB_CUDA_CHECK(cudaGetLastError());
    return BB_OK;
  }
  const size_t smem = (size_t)warps * 2 * h * sizeof(float);
  BB_ONCE_PER_DEVICE({
    BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_reg_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_reg_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
  });
#define BB_LN_ARGS (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd, \
                   (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, ws, rows
  if (h == 256) layernorm_bwd_reg_kernel<1><<<grid, warps * 32, smem, s>>>(BB_LN_ARGS);
  else if (h == 512) layernorm_bwd_reg_kernel<2><<<grid, warps * 32, smem, s>>>(BB_LN_ARGS);
  else if (h == 768) layernorm_bwd_reg_kernel<3><<<grid, warps * 32, smem, s>>>(BB_LN_ARGS);
  else if (h == 1024) layernorm_bwd_reg_kernel<4><<<grid, warps * 32, smem, s>>>(BB_LN_ARGS);
  else layernorm_bwd_kernel<<<grid, warps * 32, smem, s>>>(BB_LN_ARGS, h);
#undef BB_LN_ARGS
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
}  // namespace

extern "C" long long bb_layernorm_bwd_workspace_bytes(int rows, int h) {
  if (rows <= 0 || h <= 0 || ln_bwd_warps(h) < 1) return 0;
  return (long long)ln_bwd_grid(rows, h) * 2 * h * (long long)sizeof(float);
}

extern "C" int bb_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                                const void* dres, void* dx, float* dgamma, float* dbeta, void* workspace,
                                long long workspace_bytes, int rows, int h, void* stream) {
  if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || !workspace || rows <= 0 || h <= 0 || (h & 7)) {
    bb_set_last_error_msg("bb_layernorm_bwd: null pointer or hidden size not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  const int warps = ln_bwd_warps(h);
  if (warps < 1) { bb_set_last_error_msg("bb_layernorm_bwd: hidden size too large (max 25600)"); return BB_ERR_TOO_LARGE; }
  if (workspace_bytes < bb_layernorm_bwd_workspace_bytes(rows, h)) {
    bb_set_last_error_msg("bb_layernorm_bwd: workspace smaller than bb_layernorm_bwd_workspace_bytes()");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = ln_bwd_grid(rows, h);
  float* ws = (float*)workspace;
  if (int rc = ln_bwd_main(dy, x, gamma, mean, rstd, dres, dx, ws, rows, h, grid, warps, s)) return rc;
  reduce_partials_kernel<<<dim3((h + 31) / 32, 2), 256, 0, s>>>(ws, dgamma, dbeta, (long long)h, grid, h, 2LL * h);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

// ------------------------------------------------------------------ LayerNorm backward without caller scratch
namespace {
// Scratch of the allocation-free entry point: lives in the library image, one copy per GPU
// that loads it, until the process exits.
constexpr long long LN_STATIC_SCRATCH_FLOATS = 2LL * 1024 * 1024;   // 8 MiB
static __device__ __align__(256) float g_ln_static_scratch[LN_STATIC_SCRATCH_FLOATS];

// Device address of the scratch array on the current device.  The symbol's name in host code
// is only a handle, so the address is looked up (once per device, with that device current).
float* ln_static_scratch_ptr() {
  static float* ptr[64] = {nullptr};
  const int dev = bb_current_device();
  if (dev < 0) {
    bb_set_last_error_msg("bb_layernorm_bwd_static: the current device cannot be read or its index is 64 or more "
                          "(the per-device address table holds 64 entries)");
    return nullptr;
  }
  if (!ptr[dev]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_ln_static_scratch);
    if (e != cudaSuccess) { bb_set_last_error("cudaGetSymbolAddress(g_ln_static_scratch)", e); return nullptr; }
    ptr[dev] = static_cast<float*>(p);
  }
  return ptr[dev];
}
}  // namespace

extern "C" long long bb_layernorm_bwd_static_capacity_bytes(void) {
  return LN_STATIC_SCRATCH_FLOATS * (long long)sizeof(float);
}

extern "C" int bb_layernorm_bwd_static(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                                       const void* dres, void* dx, float* dgamma, float* dbeta, int rows, int h, void* stream) {
  if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || rows <= 0 || h <= 0 || (h & 7)) {
    bb_set_last_error_msg("bb_layernorm_bwd_static: null pointer or hidden size not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  const int warps = ln_bwd_warps(h);
  const long long need = bb_layernorm_bwd_workspace_bytes(rows, h);
  if (warps < 1 || need <= 0 || need > bb_layernorm_bwd_static_capacity_bytes()) {
    char msg[200];
    snprintf(msg, sizeof(msg), "bb_layernorm_bwd_static: rows=%d h=%d needs %lld bytes of scratch, the built-in scratch holds %lld; "
             "use bb_layernorm_bwd with a caller workspace", rows, h, need, bb_layernorm_bwd_static_capacity_bytes());
    bb_set_last_error_msg(msg);
    return BB_ERR_TOO_LARGE;
  }
  float* ws = ln_static_scratch_ptr();
  if (!ws) return BB_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = ln_bwd_grid(rows, h);
  // every partial row that the reduction reads is rewritten by this launch, so the scratch
  // needs no clearing although it still holds the previous call's sums
  if (int rc = ln_bwd_main(dy, x, gamma, mean, rstd, dres, dx, ws, rows, h, grid, warps, s)) return rc;
  reduce_partials_kernel<<<dim3((h + 31) / 32, 2), 256, 0, s>>>(ws, dgamma, dbeta, (long long)h, grid, h, 2LL * h);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

namespace {
int colsum_splits(int rows) {
  int s = (rows + 255) / 256;
  return s < 1 ? 1 : (s > 64 ? 64 : s);
}
}  // namespace

extern "C" int bb_gelu_bwd(const void* dy, const void* pre, void* dx, long long n, void* stream) {
  if (!dy || !pre || !dx || n <= 0 || (n & 7) || ((uintptr_t)dy & 15) || ((uintptr_t)pre & 15) || ((uintptr_t)dx & 15)) {
    bb_set_last_error_msg("bb_gelu_bwd: null/unaligned pointer or n not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  const long long n8 = n >> 3;
  long long grid = (n8 + 255) / 256, cap = (long long)bb_num_sms() * 8;
  gelu_bwd_kernel<<<(int)(grid < cap ? grid : cap), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)pre, (__nv_bfloat16*)dx, n8);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" long long bb_colsum_workspace_bytes(int rows, int n) {
  if (rows <= 0 || n <= 0) return 0;
  return (long long)colsum_splits(rows) * n * (long long)sizeof(float);
}

extern "C" int bb_colsum_accum(const void* dy, long long ld, float* out, void* workspace, long long workspace_bytes,
                               int rows, int n, void* stream) {
  if (!dy || !out || !workspace || rows <= 0 || n <= 0 || (n & 7) || (ld & 7)) {
    bb_set_last_error_msg("bb_colsum_accum: null pointer, or n / ld not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  if (workspace_bytes < bb_colsum_workspace_bytes(rows, n)) {
    bb_set_last_error_msg("bb_colsum_accum: workspace smaller than bb_colsum_workspace_bytes()");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int splits = colsum_splits(rows);
  const int rps = (rows + splits - 1) / splits;
  dim3 grid((n + 255) / 256, splits);
  colsum_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (float*)workspace, rows, n, ld, rps);
  reduce_partials_kernel<<<dim3((n + 31) / 32, 1), 256, 0, s>>>((const float*)workspace, out, nullptr, 0LL, splits, n, (long long)n);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_embedding_fwd(const long long* tokens, const void* wte, const void* wpe, void* out, int n_tokens,
                                int seq, int h, int vocab, void* stream) {
  if (!tokens || !wte || !out || n_tokens <= 0 || seq <= 0 || h <= 0 || (h & 7) || vocab <= 0) {
    bb_set_last_error_msg("bb_embedding_fwd: null pointer or hidden size not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  embedding_fwd_kernel<<<row_grid(n_tokens), WARPS * 32, 0, (cudaStream_t)stream>>>(
      tokens, (const __nv_bfloat16*)wte, (const __nv_bfloat16*)wpe, (__nv_bfloat16*)out, n_tokens, seq, h, vocab,
      bb_device_status_word());
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_embedding_bwd(const long long* tokens, const void* dout, float* dwte, float* dwpe, int n_tokens, int seq,
                                int h, int vocab, void* stream) {
  if (!tokens || !dout || !dwte || n_tokens <= 0 || seq <= 0 || h <= 0 || (h & 7) || vocab <= 0) {
    bb_set_last_error_msg("bb_embedding_bwd: null pointer or hidden size not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  embedding_bwd_kernel<<<row_grid(n_tokens), WARPS * 32, 0, (cudaStream_t)stream>>>(
      tokens, (const __nv_bfloat16*)dout, dwte, dwpe, n_tokens, seq, h, vocab);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
