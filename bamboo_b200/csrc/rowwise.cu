// HBM-bound row-wise kernels of a transformer stage: LayerNorm forward/backward (with the
// residual gradient folded in, and optionally its column sums), bias-gradient column sums, token+position
// embedding gather and its gradient scatter.  All loads/stores are 8- or 16-byte vectors.  Forward and
// embedding kernels: one warp owns a row, no block-level synchronisation.  LayerNorm backward for hidden
// sizes that are multiples of 256: a thread owns a few columns of a row slot and keeps their column sums in
// registers (one block barrier per iteration combines the row sums); other sizes: one warp per row.  Grids are
// sized as a multiple of the SM count and stride over rows.
#include "common.cuh"
#include <stdio.h>
#include <stdlib.h>
#include <atomic>

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
// CTAs fit on an SM (the warp-per-row kernels hold a whole row's partial sums per warp, run one
// CTA per SM and are latency-bound at about a third of the HBM rate).  Every operand of the R rows
// a thread handles per iteration - dy, x and the residual gradient - is requested before the first
// use, so a thread keeps 3 x R 16-byte loads in flight and an iteration pays one memory latency.
// The two row sums of R rows per slot are combined across the slot's warps through
// double-buffered shared memory: one block barrier per iteration.
// SUMRES: the thread also keeps the column sums of the residual gradient (a third partial row).
template <int CW> struct ColVec;
template <> struct ColVec<8> {
  using T = uint4;
  static __device__ __forceinline__ T zero() { return make_uint4(0, 0, 0, 0); }
  static __device__ __forceinline__ void unpack(const T& q, float* f) { unpack8(q, f); }
  static __device__ __forceinline__ T pack(const float* f) { return pack8(f); }
  static __device__ __forceinline__ void opaque(T& q) { asm volatile("" : "+r"(q.x), "+r"(q.y), "+r"(q.z), "+r"(q.w)); }
};
template <> struct ColVec<4> {
  using T = uint2;
  static __device__ __forceinline__ T zero() { return make_uint2(0, 0); }
  static __device__ __forceinline__ void unpack(const T& q, float* f) {
    f[0] = bb::bf16_lo(q.x); f[1] = bb::bf16_hi(q.x); f[2] = bb::bf16_lo(q.y); f[3] = bb::bf16_hi(q.y);
  }
  static __device__ __forceinline__ T pack(const float* f) { return make_uint2(bb::pack_bf16x2(f[0], f[1]), bb::pack_bf16x2(f[2], f[3])); }
  static __device__ __forceinline__ void opaque(T& q) { asm volatile("" : "+r"(q.x), "+r"(q.y)); }
};

// CW: columns per thread (8: 16-byte accesses; 4: 8-byte accesses and half the registers, for
// hidden sizes up to 1024 where more resident warps matter more than the access width).
// PF: the operands of the next iteration are requested before the current one is processed
// (twice the operand registers, memory requests in flight all the time).
template <int MAXT, int CW, int R, int MINB, bool PF, bool SUMRES>
__global__ void __launch_bounds__(MAXT, MINB)
layernorm_bwd_cols_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                          const __nv_bfloat16* __restrict__ gamma, const float* __restrict__ mean_in,
                          const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                          __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int rows, int h, int slots) {
  extern __shared__ float sm[];
  using V = ColVec<CW>;
  using VT = typename V::T;
  constexpr int NS = SUMRES ? 3 : 2;               // partial rows per CTA: dgamma, dbeta (, residual sums)
  const int tpr = h / CW;                          // threads per row
  const int wps = tpr >> 5;                        // warps per slot
  const int slot = threadIdx.x / tpr, tc = threadIdx.x - slot * tpr;   // my slot, my column group
  const int lane = threadIdx.x & 31, wis = tc >> 5;
  float* red = sm;                                 // [2][slots][wps][2 * R]
  float* fin = sm + 2 * slots * wps * 2 * R;       // [slots][NS][h] final combination
  float g[CW], ag[CW], ab[CW], ar[CW];
  V::unpack(__ldg(reinterpret_cast<const VT*>(gamma) + tc), g);
#pragma unroll
  for (int i = 0; i < CW; ++i) { ag[i] = 0.f; ab[i] = 0.f; ar[i] = 0.f; }
  const float inv_h = 1.f / h;
  int buf = 0;
  // operands of R rows starting at `first` (zeros past the last row)
  auto load_rows = [&](int first, VT* ld, VT* lx, VT* lr, float* lm, float* ls) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = first + r;
      ld[r] = V::zero(); lx[r] = ld[r]; lr[r] = ld[r]; lm[r] = 0.f; ls[r] = 0.f;
      if (row < rows) {
        ld[r] = reinterpret_cast<const VT*>(dy + (size_t)row * h)[tc];
        lx[r] = reinterpret_cast<const VT*>(x + (size_t)row * h)[tc];
        if (dres) lr[r] = reinterpret_cast<const VT*>(dres + (size_t)row * h)[tc];
        lm[r] = mean_in[row]; ls[r] = rstd_in[row];
      }
    }
  };
  const int step = gridDim.x * slots * R;
  VT qd[R], qx[R], qr[R];
  float mean[R], rstd[R];
  if ((int)blockIdx.x * slots * R < rows) load_rows(blockIdx.x * slots * R + slot * R, qd, qx, qr, mean, rstd);
  for (int base = blockIdx.x * slots * R; base < rows; base += step) {
    const int r0 = base + slot * R;
    VT nd[R], nx[R], nr[R];
    float nm[R], ns[R];
    if (PF && base + step < rows) load_rows(r0 + step, nd, nx, nr, nm, ns);
    float s[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float d[CW], f[CW];
      V::unpack(qd[r], d); V::unpack(qx[r], f);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < CW; ++i) { const float t = d[i] * g[i]; s1 += t; s2 += t * (f[i] - mean[r]) * rstd[r]; }
      s[2 * r] = s1; s[2 * r + 1] = s2;
    }
#pragma unroll
    for (int k = 0; k < 2 * R; ++k) s[k] = warp_sum(s[k]);
    float* my = red + ((buf * slots + slot) * wps + wis) * 2 * R;
    if (lane == 0) {
#pragma unroll
      for (int k = 0; k < 2 * R; ++k) my[k] = s[k];
    }
    __syncthreads();
    // the operands stay packed across the barrier (the compiler would otherwise keep the unpacked
    // floats of the first pass alive: twice the registers)
#pragma unroll
    for (int r = 0; r < R; ++r) { V::opaque(qd[r]); V::opaque(qx[r]); }
    const float* all = red + (buf * slots + slot) * wps * 2 * R;
#pragma unroll
    for (int k = 0; k < 2 * R; ++k) {
      float t = 0.f;
      for (int w = 0; w < wps; ++w) t += all[w * 2 * R + k];    // fixed order
      s[k] = t * inv_h;
    }
    buf ^= 1;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int row = r0 + r;
      if (row >= rows) continue;
      float d[CW], f[CW], o[CW], rr[CW];
      V::unpack(qd[r], d); V::unpack(qx[r], f); V::unpack(qr[r], rr);
#pragma unroll
      for (int i = 0; i < CW; ++i) {
        const float xh = (f[i] - mean[r]) * rstd[r];
        o[i] = rstd[r] * (d[i] * g[i] - s[2 * r] - xh * s[2 * r + 1]) + rr[i];
        ag[i] += d[i] * xh;
        ab[i] += d[i];
        if (SUMRES) ar[i] += rr[i];
      }
      reinterpret_cast<VT*>(dx + (size_t)row * h)[tc] = V::pack(o);
    }
    if (base + step < rows) {
      if (PF) {
#pragma unroll
        for (int r = 0; r < R; ++r) { qd[r] = nd[r]; qx[r] = nx[r]; qr[r] = nr[r]; mean[r] = nm[r]; rstd[r] = ns[r]; }
      } else {
        load_rows(r0 + step, qd, qx, qr, mean, rstd);
      }
    }
  }
  // combine the slots' column sums (fixed order) and write this CTA's partial rows
  float* mine = fin + (size_t)slot * NS * h;
#pragma unroll
  for (int i = 0; i < CW; ++i) {
    mine[tc * CW + i] = ag[i]; mine[h + tc * CW + i] = ab[i];
    if (SUMRES) mine[2 * h + tc * CW + i] = ar[i];
  }
  __syncthreads();
  float* out = partials + (size_t)blockIdx.x * NS * h;
  for (int j = threadIdx.x; j < NS * h; j += blockDim.x) {
    float t = 0.f;
    for (int q = 0; q < slots; ++q) t += fin[(size_t)q * NS * h + j];
    out[j] = t;
  }
}

// out[j] += sum_p partials[p * stride + j].  A 32-column x 32-way block: 32 threads share a
// column, each sums every 32nd partial (eight loads in flight), shared memory combines them in a
// fixed order (deterministic).
// blockIdx.y selects one of up to three (partials, out) pairs, `pair_offset` floats apart in
// `partials` (LayerNorm: dgamma, dbeta and the residual gradient's column sums in one launch).
__global__ void __launch_bounds__(1024)
reduce_partials_kernel(const float* __restrict__ partials, float* __restrict__ out0, float* __restrict__ out1,
                       float* __restrict__ out2, long long pair_offset, int nparts, int n, long long stride) {
  __shared__ float red[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float* out = blockIdx.y == 0 ? out0 : (blockIdx.y == 1 ? out1 : out2);
  partials += blockIdx.y * pair_offset;
  float s = 0.f;
  if (j < n) {
    for (int p = ty; p < nparts; p += 32 * 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = (p + 32 * u < nparts) ? __ldcg(partials + (size_t)(p + 32 * u) * stride + j) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
  }
  red[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < n) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) t += red[w][tx];
    out[j] += t;
  }
}

// ------------------------------------------------------------------ bias gradient
// out[n] += sum over rows of dy[row][n], one launch.  CTA (bx, by) sums the rows of split `by`
// over 256 columns (a warp reads 512 contiguous bytes of a row, four rows in flight per warp)
// and writes one partial row; the CTA that finishes last for its 256 columns (a ticket counter
// per column block) adds the partial rows in split order, so the result does not depend on the
// order in which CTAs ran.  The counter returns to zero for its next user.
constexpr int COLSUM_TICKET_SLOTS = 1 << 16;
__device__ unsigned int g_colsum_tickets[COLSUM_TICKET_SLOTS];

__global__ void __launch_bounds__(256)
colsum_kernel(const __nv_bfloat16* __restrict__ dy, float* __restrict__ partials, float* __restrict__ out, int rows, int n,
              long long ld, int rows_per_split, unsigned int* __restrict__ tickets) {
  __shared__ float red[8][256];
  __shared__ int s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int col0 = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_split;
  const int r1 = min(rows, r0 + rows_per_split);
  const int splits = gridDim.y;
  float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (col0 < n) {
    const __nv_bfloat16* src = dy + col0;
    // eight rows in flight per warp; rows past the split's end load nothing and add zeros
    for (int r = r0 + warp; r < r1; r += 64) {
      uint4 q[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        q[u] = (r + 8 * u < r1) ? *reinterpret_cast<const uint4*>(src + (size_t)(r + 8 * u) * ld) : make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float f[8];
        unpack8(q[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s[i] += f[i];
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = s[i];
  __syncthreads();
  const int j = threadIdx.x, col = blockIdx.x * 256 + j;
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w][j];
  if (splits == 1) {
    if (col < n) out[col] += t;
    return;
  }
  if (col < n) partials[(size_t)blockIdx.y * n + col] = t;
  __threadfence();                                   // my partial is visible before my ticket
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(&tickets[blockIdx.x], 1u) == (unsigned)(splits - 1));
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (col < n) {
    float acc = 0.f;
    for (int p = 0; p < splits; p += 16) {
      float v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) v[u] = (p + u < splits) ? __ldcg(partials + (size_t)(p + u) * n + col) : 0.f;
#pragma unroll
      for (int u = 0; u < 16; ++u) acc += v[u];
    }
    out[col] += acc;
  }
  if (threadIdx.x == 0) tickets[blockIdx.x] = 0u;
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
// Shape of the column-owner kernel for a hidden size: columns per thread, rows per slot per
// iteration, resident CTAs per SM (what the register count of that instantiation allows) and
// the CTA size bound.  Every instantiation below compiles without register spills.
struct LnColsCfg { int cw, r, ctas, maxt, pf; };
LnColsCfg ln_cols_cfg(int h) {
  if (h <= 1024) {
    // BB_LN_BWD_VARIANT=1|2 in the environment picks another instantiation (A/B measurements):
    // measured on 8192 x 1024, both launches, less the fixed cost of two launches:
    // 0: 16.2 us, 1: 21.1 us, 2: 14.8 us (but 20.2 us with the residual sums: it spills there)
    static int v = -1;
    if (v < 0) { const char* e = getenv("BB_LN_BWD_VARIANT"); v = (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 0; }
    switch (v) {
      case 1: return {4, 4, 3, 256, 0};
      case 2: return {8, 1, 3, 256, 1};
      default: return {8, 3, 2, 256, 0};
    }
  }
  if (h <= 2048) return {8, 2, 3, 256, 0};
  if (h <= 4096) return {8, 4, 1, 512, 0};
  return {8, 1, 1, 1024, 0};
}
int ln_bwd_cols_slots(int h) { const int tpr = h / ln_cols_cfg(h).cw; return tpr >= 256 ? 1 : 256 / tpr; }
int ln_bwd_grid(int rows, int h) {
  if (ln_bwd_cols_ok(h)) {
    const LnColsCfg c = ln_cols_cfg(h);
    const int per = ln_bwd_cols_slots(h) * c.r;
    long long want = ((long long)rows + per - 1) / per, cap = (long long)c.ctas * bb_num_sms();
    return (int)(want < cap ? (want > 0 ? want : 1) : cap);
  }
  const int w = ln_bwd_warps(h);
  long long want = ((long long)rows + w - 1) / w;
  long long cap = (long long)bb_num_sms() * (w * 2 * h * 4 > 100 * 1024 ? 1 : 2);
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}
}  // namespace

namespace {
template <int MAXT, int CW, int R, int MINB, bool PF>
int ln_bwd_cols_launch(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                       void* dx, float* ws, bool sum_res, int rows, int h, int grid, cudaStream_t s) {
  const int slots = ln_bwd_cols_slots(h), tpr = h / CW, threads = slots * tpr;
  const size_t sm_bytes = ((size_t)2 * slots * (tpr / 32) * 2 * R + (size_t)slots * (sum_res ? 3 : 2) * h) * sizeof(float);
  BB_ONCE_PER_DEVICE({
    BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_cols_kernel<MAXT, CW, R, MINB, PF, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
    BB_CUDA_CHECK(cudaFuncSetAttribute(layernorm_bwd_cols_kernel<MAXT, CW, R, MINB, PF, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
  });
#define BB_LNC_ARGS (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)gamma, mean, rstd, \
                    (const __nv_bfloat16*)dres, (__nv_bfloat16*)dx, ws, rows, h, slots
  if (sum_res) layernorm_bwd_cols_kernel<MAXT, CW, R, MINB, PF, true><<<grid, threads, sm_bytes, s>>>(BB_LNC_ARGS);
  else layernorm_bwd_cols_kernel<MAXT, CW, R, MINB, PF, false><<<grid, threads, sm_bytes, s>>>(BB_LNC_ARGS);
#undef BB_LNC_ARGS
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

// launches the backward main kernel (column-owner variant when the hidden size allows it); with
// `sum_res` (column-owner variant only) every CTA writes a third partial row: the residual
// gradient's column sums
int ln_bwd_main(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dres,
                void* dx, float* ws, bool sum_res, int rows, int h, int grid, int warps, cudaStream_t s) {
  if (ln_bwd_cols_ok(h)) {
    const LnColsCfg c = ln_cols_cfg(h);
#define BB_LNC_CASE(MAXT, CW, R, MINB, PF) \
    if (c.maxt == MAXT && c.cw == CW && c.r == R && c.ctas == MINB && c.pf == PF) \
      return ln_bwd_cols_launch<MAXT, CW, R, MINB, PF != 0>(dy, x, gamma, mean, rstd, dres, dx, ws, sum_res, rows, h, grid, s);
    BB_LNC_CASE(256, 8, 3, 2, 0) BB_LNC_CASE(256, 4, 4, 3, 0) BB_LNC_CASE(256, 8, 1, 3, 1)
    BB_LNC_CASE(256, 8, 2, 3, 0) BB_LNC_CASE(512, 8, 4, 1, 0) BB_LNC_CASE(1024, 8, 1, 1, 0)
#undef BB_LNC_CASE
    bb_set_last_error_msg("layernorm backward: no column-owner instantiation for this shape");
    return BB_ERR_INVALID_ARG;
  }
  if (sum_res) { bb_set_last_error_msg("layernorm backward: residual sums need the column-owner kernel"); return BB_ERR_INVALID_ARG; }
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

namespace {
int ln_bwd_check(const char* who, const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                 const void* dx, const float* dgamma, const float* dbeta, const void* workspace, int rows, int h) {
  char msg[160];
  if (!dy || !x || !gamma || !mean || !rstd || !dx || !dgamma || !dbeta || !workspace || rows <= 0 || h <= 0 || (h & 7)) {
    snprintf(msg, sizeof(msg), "%s: null pointer or hidden size not a multiple of 8", who);
    bb_set_last_error_msg(msg);
    return BB_ERR_INVALID_ARG;
  }
  if (ln_bwd_warps(h) < 1) {
    snprintf(msg, sizeof(msg), "%s: hidden size too large (max 25600)", who);
    bb_set_last_error_msg(msg);
    return BB_ERR_TOO_LARGE;
  }
  return BB_OK;
}
}  // namespace

extern "C" int bb_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                                const void* dres, void* dx, float* dgamma, float* dbeta, void* workspace,
                                long long workspace_bytes, int rows, int h, void* stream) {
  if (int rc = ln_bwd_check("bb_layernorm_bwd", dy, x, gamma, mean, rstd, dx, dgamma, dbeta, workspace, rows, h)) return rc;
  if (workspace_bytes < bb_layernorm_bwd_workspace_bytes(rows, h)) {
    bb_set_last_error_msg("bb_layernorm_bwd: workspace smaller than bb_layernorm_bwd_workspace_bytes()");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = ln_bwd_grid(rows, h);
  float* ws = (float*)workspace;
  if (int rc = ln_bwd_main(dy, x, gamma, mean, rstd, dres, dx, ws, false, rows, h, grid, ln_bwd_warps(h), s)) return rc;
  reduce_partials_kernel<<<dim3((h + 31) / 32, 2), 1024, 0, s>>>(ws, dgamma, dbeta, nullptr, (long long)h, grid, h, 2LL * h);
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
  if (int rc = ln_bwd_main(dy, x, gamma, mean, rstd, dres, dx, ws, false, rows, h, grid, warps, s)) return rc;
  reduce_partials_kernel<<<dim3((h + 31) / 32, 2), 1024, 0, s>>>(ws, dgamma, dbeta, nullptr, (long long)h, grid, h, 2LL * h);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

namespace {
// enough splits for about four CTAs per SM, at least 64 rows each (eight per warp: one batch of
// loads), at most 64 (the last CTA of a column block adds the partial rows)
int colsum_splits(int rows, int n) {
  const int col_blocks = (n + 255) / 256;
  int s = (4 * bb_num_sms() + col_blocks - 1) / col_blocks;
  const int by_rows = (rows + 63) / 64;
  if (s > by_rows) s = by_rows;
  return s < 1 ? 1 : (s > 64 ? 64 : s);
}

// ticket counters of one launch: `col_blocks` consecutive entries of the device table, handed out
// round-robin so that launches in flight on different streams never share an entry
unsigned int* colsum_tickets(int col_blocks) {
  static unsigned int* table[64] = {nullptr};
  static std::atomic<unsigned long long> next{0};
  const int dev = bb_current_device();
  if (dev < 0 || col_blocks > COLSUM_TICKET_SLOTS) return nullptr;
  if (!table[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_colsum_tickets) != cudaSuccess) return nullptr;
    table[dev] = static_cast<unsigned int*>(ptr);
  }
  for (;;) {
    const unsigned long long at = next.fetch_add((unsigned long long)col_blocks);
    const unsigned first = (unsigned)(at % COLSUM_TICKET_SLOTS);
    if (first + (unsigned)col_blocks <= (unsigned)COLSUM_TICKET_SLOTS) return table[dev] + first;   // else the range wraps: take the next one
  }
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
  return (long long)colsum_splits(rows, n) * n * (long long)sizeof(float);
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
  const int splits = colsum_splits(rows, n);
  const int rps = (rows + splits - 1) / splits;
  dim3 grid((n + 255) / 256, splits);
  unsigned int* tickets = colsum_tickets((int)grid.x);
  if (!tickets) { bb_set_last_error_msg("bb_colsum_accum: ticket counters unavailable on this device"); return BB_ERR_CUDA; }
  colsum_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)dy, (float*)workspace, out, rows, n, ld, rps, tickets);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

// ------------------------------------------------------------------ LayerNorm backward + residual column sums
extern "C" long long bb_layernorm_bwd_res_workspace_bytes(int rows, int h) {
  if (rows <= 0 || h <= 0 || ln_bwd_warps(h) < 1) return 0;
  if (ln_bwd_cols_ok(h)) return (long long)ln_bwd_grid(rows, h) * 3 * h * (long long)sizeof(float);
  // other hidden sizes: the plain backward, then a column-sum pass over the residual gradient
  const long long a = (bb_layernorm_bwd_workspace_bytes(rows, h) + 255) & ~255LL;
  return a + bb_colsum_workspace_bytes(rows, h);
}

extern "C" int bb_layernorm_bwd_res(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                                    const void* dres, void* dx, float* dgamma, float* dbeta, float* dres_sum, void* workspace,
                                    long long workspace_bytes, int rows, int h, void* stream) {
  if (int rc = ln_bwd_check("bb_layernorm_bwd_res", dy, x, gamma, mean, rstd, dx, dgamma, dbeta, workspace, rows, h)) return rc;
  if (!dres || !dres_sum) { bb_set_last_error_msg("bb_layernorm_bwd_res: dres and dres_sum are required"); return BB_ERR_INVALID_ARG; }
  if (workspace_bytes < bb_layernorm_bwd_res_workspace_bytes(rows, h)) {
    bb_set_last_error_msg("bb_layernorm_bwd_res: workspace smaller than bb_layernorm_bwd_res_workspace_bytes()");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  float* ws = (float*)workspace;
  if (!ln_bwd_cols_ok(h)) {
    const long long a = (bb_layernorm_bwd_workspace_bytes(rows, h) + 255) & ~255LL;
    // the column sums first: dx may alias dres
    if (int rc = bb_colsum_accum(dres, h, dres_sum, (char*)workspace + a, workspace_bytes - a, rows, h, stream)) return rc;
    return bb_layernorm_bwd(dy, x, gamma, mean, rstd, dres, dx, dgamma, dbeta, workspace, a, rows, h, stream);
  }
  const int grid = ln_bwd_grid(rows, h);
  if (int rc = ln_bwd_main(dy, x, gamma, mean, rstd, dres, dx, ws, true, rows, h, grid, ln_bwd_warps(h), s)) return rc;
  reduce_partials_kernel<<<dim3((h + 31) / 32, 3), 1024, 0, s>>>(ws, dgamma, dbeta, dres_sum, (long long)h, grid, h, 3LL * h);
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
