// Cross-entropy over vocabulary rows (online log-sum-exp, one pass over the logits) with
// its gradient written in place, and the fused Adam step over a stage's flat parameter
// arena (fp32 master weights / moments, bf16 working copy, gradient cleared in the same
// pass).  Both are HBM-bound: 16-byte vector accesses, grid a multiple of the SM count.
#include "common.cuh"
#include <math.h>

namespace {

constexpr int CE_THREADS = 256;

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  f[0] = bb::bf16_lo(q.x); f[1] = bb::bf16_hi(q.x); f[2] = bb::bf16_lo(q.y); f[3] = bb::bf16_hi(q.y);
  f[4] = bb::bf16_lo(q.z); f[5] = bb::bf16_hi(q.z); f[6] = bb::bf16_lo(q.w); f[7] = bb::bf16_hi(q.w);
}

// (m, s) pair of an online softmax: running max and sum of exp(x - m)
__device__ __forceinline__ void lse_merge(float& m, float& s, float m2, float s2) {
  const float mm = fmaxf(m, m2);
  if (mm == -INFINITY) { s = 0.f; return; }  // both sides empty
  s = s * __expf(m - mm) + s2 * __expf(m2 - mm);
  m = mm;
}

// One CTA per token row.  row_loss[row] = logsumexp(logits[row, :V]) - logits[row, target]
// (0 for ignored targets); lse[row] saved for the backward pass.
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
              float* __restrict__ lse_out, float* __restrict__ row_loss, int rows, int V, long long ignore_index, int* status) {
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + (size_t)row * ld;
  const int nfull = V >> 3;
  float m = -INFINITY, s = 0.f;
  for (int c = threadIdx.x; c < nfull; c += CE_THREADS) {
    float f[8]; unpack8(*reinterpret_cast<const uint4*>(lr + c * 8), f);
    float cm = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) cm = fmaxf(cm, f[i]);
    float cs = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) cs += __expf(f[i] - cm);
    lse_merge(m, s, cm, cs);
  }
  for (int j = nfull * 8 + threadIdx.x; j < V; j += CE_THREADS) lse_merge(m, s, __bfloat162float(lr[j]), 1.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    lse_merge(m, s, m2, s2);
  }
  if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = m; ss[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < CE_THREADS / 32; ++w) lse_merge(m, s, sm[w], ss[w]);
    const float lse = m + __logf(s);
    lse_out[row] = lse;
    const long long t = targets[row];
    float loss = 0.f;
    if (t != ignore_index) {
      if (t < 0 || t >= V) atomicCAS(status, 0, BB_ERR_INVALID_ARG);
      else loss = lse - __bfloat162float(lr[t]);
    }
    row_loss[row] = loss;
  }
}

// loss_out[0] = sum(row_loss) / max(1, #valid) ; loss_out[1] = #valid.  Single CTA, fixed order.
__global__ void __launch_bounds__(1024)
ce_finalize_kernel(const float* __restrict__ row_loss, const long long* __restrict__ targets, float* __restrict__ loss_out,
                   int rows, long long ignore_index) {
  __shared__ float s_sum[32], s_cnt[32];
  float s = 0.f, n = 0.f;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    s += row_loss[r];
    n += (targets[r] != ignore_index) ? 1.f : 0.f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); n += __shfl_xor_sync(0xffffffffu, n, o); }
  if ((threadIdx.x & 31) == 0) { s_sum[threadIdx.x >> 5] = s; s_cnt[threadIdx.x >> 5] = n; }
  __syncthreads();
  if (threadIdx.x == 0) {
    s = 0.f; n = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { s += s_sum[w]; n += s_cnt[w]; }
    loss_out[0] = s / fmaxf(n, 1.f);
    loss_out[1] = n;
  }
}

// dlogits[row, j] = (softmax_j - [j == target]) * gscale / #valid for j < V, 0 for the padded
// columns V..ld_cols; rows with an ignored target get 0.  May run in place.
__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(const __nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
              const float* __restrict__ lse_in, const float* __restrict__ loss_out, const float* __restrict__ gscale_ptr,
              float gscale, __nv_bfloat16* __restrict__ dlogits, long long ldd, int V, int cols, long long ignore_index) {
  const int row = blockIdx.x;
  const long long t = targets[row];
  const float nvalid = fmaxf(loss_out[1], 1.f);
  const float g = (t == ignore_index) ? 0.f : (gscale_ptr ? gscale_ptr[0] : 1.f) * gscale / nvalid;
  const float lse = lse_in[row];
  const __nv_bfloat16* lr = logits + (size_t)row * ld;
  __nv_bfloat16* dr = dlogits + (size_t)row * ldd;
  const int nch = cols >> 3;
  for (int c = threadIdx.x; c < nch; c += CE_THREADS) {
    float f[8]; unpack8(*reinterpret_cast<const uint4*>(lr + c * 8), f);
    const int j0 = c * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int j = j0 + i;
      float p = (j < V) ? __expf(f[i] - lse) : 0.f;
      if (j == t) p -= 1.f;
      f[i] = p * g;
    }
    uint4 q;
    q.x = bb::pack_bf16x2(f[0], f[1]); q.y = bb::pack_bf16x2(f[2], f[3]);
    q.z = bb::pack_bf16x2(f[4], f[5]); q.w = bb::pack_bf16x2(f[6], f[7]);
    *reinterpret_cast<uint4*>(dr + j0) = q;
  }
}

// ------------------------------------------------------------------ Adam
// Follows Bamboo's FusedAdam functor (csrc/adam/multi_tensor_adam.cu:72-108):
//   mode 0 (L2):     g += decay*p
//   m = b1*m + (1-b1)*g ; v = b2*v + (1-b2)*g*g
//   update = (m/bc1) / (sqrt(v/bc2) + eps)  [+ decay*p in mode 1, decoupled]
//   p -= lr*update
// plus what the reference does in separate passes: the low-precision working copy of the
// weights is refreshed and the gradient is cleared.
__global__ void __launch_bounds__(256)
adam_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
            __nv_bfloat16* __restrict__ p_lp, long long n, float lr, float b1, float b2, float eps, float bc1, float bc2,
            float decay, int mode, float gscale, int zero_grad) {
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 P = reinterpret_cast<float4*>(p)[i], G = reinterpret_cast<float4*>(g)[i];
    float4 M = reinterpret_cast<float4*>(m)[i], Vv = reinterpret_cast<float4*>(v)[i];
    float pp[4] = {P.x, P.y, P.z, P.w}, gg[4] = {G.x, G.y, G.z, G.w};
    float mm[4] = {M.x, M.y, M.z, M.w}, vv[4] = {Vv.x, Vv.y, Vv.z, Vv.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float gk = gg[k] * gscale;
      if (mode == 0) gk += decay * pp[k];
      mm[k] = b1 * mm[k] + (1.f - b1) * gk;
      vv[k] = b2 * vv[k] + (1.f - b2) * gk * gk;
      const float denom = sqrtf(vv[k] / bc2) + eps;
      float upd = (mm[k] / bc1) / denom;
      if (mode != 0) upd += decay * pp[k];
      pp[k] -= lr * upd;
    }
    reinterpret_cast<float4*>(p)[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p_lp) {
      uint2 q; q.x = bb::pack_bf16x2(pp[0], pp[1]); q.y = bb::pack_bf16x2(pp[2], pp[3]);
      reinterpret_cast<uint2*>(p_lp)[i] = q;
    }
  }
}

// dst(bf16) = src(fp32), used when a shadow copy of a stage is promoted or refreshed
__global__ void __launch_bounds__(256)
cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long n4 = n >> 2;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 a = reinterpret_cast<const float4*>(src)[i];
    uint2 q; q.x = bb::pack_bf16x2(a.x, a.y); q.y = bb::pack_bf16x2(a.z, a.w);
    reinterpret_cast<uint2*>(dst)[i] = q;
  }
}

int flat_grid(long long n4) {
  long long want = (n4 + 255) / 256;
  long long cap = (long long)bb_num_sms() * 8;
  return (int)(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace

extern "C" int bb_cross_entropy_fwd(const void* logits, long long ld, const long long* targets, float* lse, float* row_loss,
                                    float* loss_out, int rows, int vocab, long long ignore_index, void* stream) {
  if (!logits || !targets || !lse || !row_loss || !loss_out || rows <= 0 || vocab <= 0 || (ld & 7) || ld < vocab) {
    bb_set_last_error_msg("bb_cross_entropy_fwd: null pointer, ld < vocab, or ld not a multiple of 8");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  ce_fwd_kernel<<<rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, ld, targets, lse, row_loss, rows, vocab,
                                            ignore_index, bb_device_status_word());
  ce_finalize_kernel<<<1, 1024, 0, s>>>(row_loss, targets, loss_out, rows, ignore_index);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_cross_entropy_bwd(const void* logits, long long ld, const long long* targets, const float* lse,
                                    const float* loss_out, const float* grad_scale_dev, float grad_scale, void* dlogits,
                                    long long ldd, int rows, int vocab, int cols, long long ignore_index, void* stream) {
  if (!logits || !targets || !lse || !loss_out || !dlogits || rows <= 0 || vocab <= 0 || cols < vocab || (cols & 7) ||
      (ld & 7) || (ldd & 7) || ld < cols || ldd < cols) {
    bb_set_last_error_msg("bb_cross_entropy_bwd: null pointer or cols/ld/ldd not multiples of 8 covering vocab");
    return BB_ERR_INVALID_ARG;
  }
  ce_bwd_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, ld, targets, lse, loss_out,
                                                               grad_scale_dev, grad_scale, (__nv_bfloat16*)dlogits, ldd,
                                                               vocab, cols, ignore_index);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_adam_step(float* master, float* grad, float* exp_avg, float* exp_avg_sq, void* param_bf16, long long n,
                            float lr, float beta1, float beta2, float eps, int step, int adam_w_mode, int bias_correction,
                            float weight_decay, float grad_scale, int zero_grad, void* stream) {
  if (!master || !grad || !exp_avg || !exp_avg_sq || n <= 0 || (n & 3) || step < 1 ||
      (((uintptr_t)master | (uintptr_t)grad | (uintptr_t)exp_avg | (uintptr_t)exp_avg_sq) & 15) || ((uintptr_t)param_bf16 & 7)) {
    bb_set_last_error_msg("bb_adam_step: null/unaligned pointer, n not a multiple of 4, or step < 1");
    return BB_ERR_INVALID_ARG;
  }
  float bc1 = 1.f, bc2 = 1.f;
  if (bias_correction) {
    bc1 = 1.f - powf(beta1, (float)step);
    bc2 = 1.f - powf(beta2, (float)step);
  }
  adam_kernel<<<flat_grid(n >> 2), 256, 0, (cudaStream_t)stream>>>(master, grad, exp_avg, exp_avg_sq,
                                                                  (__nv_bfloat16*)param_bf16, n, lr, beta1, beta2, eps, bc1,
                                                                  bc2, weight_decay, adam_w_mode ? 1 : 0, grad_scale, zero_grad);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream) {
  if (!src || !dst || n <= 0 || (n & 3) || ((uintptr_t)src & 15) || ((uintptr_t)dst & 7)) {
    bb_set_last_error_msg("bb_cast_f32_to_bf16: null/unaligned pointer or n not a multiple of 4");
    return BB_ERR_INVALID_ARG;
  }
  cast_f32_bf16_kernel<<<flat_grid(n >> 2), 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, n);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
