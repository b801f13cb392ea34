// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = op(A)[M,K] * op(B)[N,K]^T with a
// fused epilogue.  One persistent CTA per SM; warp 0 feeds shared memory with TMA
// (128-byte swizzle, no cluster multicast), warp 1 issues tcgen05.mma into two TMEM
// accumulators, warps 2-5 drain TMEM (tcgen05.ld) and run the epilogue while the next
// tile's main loop is already running.
//
// Operand storage (all row-major, bf16):
//   a_mn = 0 : A is [M, K] (K contiguous)     a_mn = 1 : A is stored [K, M] (M contiguous)
//   b_mn = 0 : B is [N, K] (K contiguous)     b_mn = 1 : B is stored [K, N] (N contiguous)
// which covers a linear layer's forward (0,0), input gradient (0,1) and weight gradient
// (1,1) without a transpose pass.
#include "common.cuh"
#include "bamboo_b200.h"
#include <cuda.h>

namespace {

constexpr int BM = 128;
constexpr int BK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB

template <int BN> struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int epi;
  void* D; void* D2; const void* bias; const void* aux;
  long long ldd, ld_aux;
  int* status;
};

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float* v) {
  uint4 q;
  q.x = bb::pack_bf16x2(v[0], v[1]); q.y = bb::pack_bf16x2(v[2], v[3]);
  q.z = bb::pack_bf16x2(v[4], v[5]); q.w = bb::pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = q;
}

// Epilogue for 32 consecutive columns of one output row held in registers.
__device__ __forceinline__ void epilogue_row32(const GemmParams& p, int m, int n0, uint32_t* r) {
  if (m >= p.M || n0 >= p.N) return;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
  const bool full = (n0 + 32 <= p.N);
  const int epi = p.epi;
  if (epi == BB_EPI_BIAS || epi == BB_EPI_BIAS_GELU || epi == BB_EPI_BIAS_RESIDUAL) {
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 q = __ldg(reinterpret_cast<const uint4*>(b + i));
        v[i + 0] += bb::bf16_lo(q.x); v[i + 1] += bb::bf16_hi(q.x);
        v[i + 2] += bb::bf16_lo(q.y); v[i + 3] += bb::bf16_hi(q.y);
        v[i + 4] += bb::bf16_lo(q.z); v[i + 5] += bb::bf16_hi(q.z);
        v[i + 6] += bb::bf16_lo(q.w); v[i + 7] += bb::bf16_hi(q.w);
      }
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) v[i] += __bfloat162float(b[i]);
    }
  }
  if (epi == BB_EPI_ACCUM_F32 || epi == BB_EPI_STORE_F32) {
    float* d = reinterpret_cast<float*>(p.D) + (long long)m * p.ldd + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 4) {
        float4 o = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
        if (epi == BB_EPI_ACCUM_F32) {
          float4 c = *reinterpret_cast<const float4*>(d + i);
          o.x += c.x; o.y += c.y; o.z += c.z; o.w += c.w;
        }
        *reinterpret_cast<float4*>(d + i) = o;
      }
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) d[i] = (epi == BB_EPI_ACCUM_F32 ? d[i] : 0.f) + v[i];
    }
    return;
  }
  __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.D) + (long long)m * p.ldd + n0;
  if (epi == BB_EPI_BIAS_GELU) {
    __nv_bfloat16* d2 = reinterpret_cast<__nv_bfloat16*>(p.D2) + (long long)m * p.ldd + n0;
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) store8_bf16(d2 + i, v + i);
    } else {
      for (int i = 0; i < 32 && n0 + i < p.N; ++i) d2[i] = __float2bfloat16(v[i]);
    }
    // GeLU is evaluated on the bf16-rounded pre-activation so that forward and backward
    // (which re-reads the stored pre-activation) see the same argument.
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = bb::gelu_tanh(__bfloat162float(__float2bfloat16(v[i])));
  } else if (epi == BB_EPI_MUL_DGELU || epi == BB_EPI_BIAS_RESIDUAL) {
    const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)m * p.ld_aux + n0;
    float x[32];
    if (full) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 q = *reinterpret_cast<const uint4*>(a + i);
        x[i + 0] = bb::bf16_lo(q.x); x[i + 1] = bb::bf16_hi(q.x);
        x[i + 2] = bb::bf16_lo(q.y); x[i + 3] = bb::bf16_hi(q.y);
        x[i + 4] = bb::bf16_lo(q.z); x[i + 5] = bb::bf16_hi(q.z);
        x[i + 6] = bb::bf16_lo(q.w); x[i + 7] = bb::bf16_hi(q.w);
      }
    } else {
      for (int i = 0; i < 32; ++i) x[i] = (n0 + i < p.N) ? __bfloat162float(a[i]) : 0.f;
    }
    if (epi == BB_EPI_MUL_DGELU) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] *= bb::gelu_tanh_grad(x[i]);
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] += x[i];
    }
  }
  if (full) {
#pragma unroll
    for (int i = 0; i < 32; i += 8) store8_bf16(d + i, v + i);
  } else {
    for (int i = 0; i < 32 && n0 + i < p.N; ++i) d[i] = __float2bfloat16(v[i]);
  }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms need 1024-byte aligned stage buffers
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::STAGES * A_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES]
  uint64_t* empty_bar = bars + C::STAGES;         // [STAGES]
  uint64_t* tmem_full = bars + 2 * C::STAGES;     // [2]
  uint64_t* tmem_empty = bars + 2 * C::STAGES + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) { bb::mbar_init(&full_bar[s], 1); bb::mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { bb::mbar_init(&tmem_full[a], 1); bb::mbar_init(&tmem_empty[a], 4); }
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tmA);
    bb::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    bb::tmem_alloc(tmem_slot, C::TMEM_COLS);
    bb::tmem_relinquish();
  }
  bb::tc_fence_before_sync();
  __syncthreads();
  bb::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0; uint32_t phase = 0;
      bool alive = true;
      for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
        const int m0 = (tile % num_m) * BM, n0 = (tile / num_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!bb::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag, p.status)) { alive = false; break; }
          bb::mbar_arrive_expect_tx(&full_bar[s], C::STAGE_BYTES);
          uint8_t* a = sA + s * A_STAGE_BYTES;
          uint8_t* b = sB + s * C::B_STAGE_BYTES;
          const int k0 = kb * BK;
          if (!p.a_mn) {
            bb::tma_load_2d(a, &tmA, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) bb::tma_load_2d(a + j * 8192, &tmA, &full_bar[s], m0 + 64 * j, k0);
          }
          if (!p.b_mn) {
            bb::tma_load_2d(b, &tmB, &full_bar[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) bb::tma_load_2d(b + j * 8192, &tmB, &full_bar[s], n0 + 64 * j, k0);
          }
          if (++s == C::STAGES) { s = 0; phase ^= 1; }
        }
      }
      if (!alive) {
        // give copies that are still in flight time to land before the CTA's shared
        // memory is released (bounded)
        uint64_t t0 = bb::globaltimer_ns();
        while (bb::globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------ MMA issuer
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                           ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
    // K-major: 8-row groups 1024 B apart (LBO unused); MN-major: 64-wide column groups are
    // separate 8 KiB TMA boxes (LBO), 8 k-rows are 1024 B (SBO).
    const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
    const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;
    int s = 0; uint32_t phase = 0;
    int acc = 0; uint32_t acc_phase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      if (!bb::mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!bb::mbar_wait(&full_bar[s], phase, abort_flag, p.status)) { alive = false; break; }
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t a_addr = bb::smem_u32(sA + s * A_STAGE_BYTES);
          const uint32_t b_addr = bb::smem_u32(sB + s * C::B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t ad = bb::make_smem_desc_sw128(a_addr + k * a_kstep, a_lbo, 1024u);
            uint64_t bd = bb::make_smem_desc_sw128(b_addr + k * b_kstep, b_lbo, 1024u);
            bb::umma_f16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          bb::umma_commit(&empty_bar[s]);
          if (kb == num_kb - 1) bb::umma_commit(&tmem_full[acc]);
        }
        __syncwarp();
        if (++s == C::STAGES) { s = 0; phase ^= 1; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------ epilogue (4 warps, one TMEM lane quarter each)
    const int quarter = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      const int m0 = (tile % num_m) * BM, n0 = (tile / num_m) * BN;
      if (!bb::mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const int m = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        bb::tmem_ld_32x32b_x32(t_row + c * 32, r);
        bb::tmem_ld_wait();
        if (c == BN / 32 - 1) {
          // accumulator fully read: hand it back before the last stores
          bb::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) bb::mbar_arrive(&tmem_empty[acc]);
        }
        epilogue_row32(p, m, n0 + c * 32, r);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  bb::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) bb::tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with leading dimension ld (elements).
int encode_2d(CUtensorMap* tm, const void* base, long long rows, long long cols, long long ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { bb_set_last_error_msg("cuTensorMapEncodeTiled entry point not available"); return BB_ERR_CUDA; }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    bb_set_last_error_msg("cuTensorMapEncodeTiled failed (operands need 16-byte aligned base and row pitch)");
    return BB_ERR_INVALID_ARG;
  }
  return BB_OK;
}

template <int BN>
int launch(const bb_gemm_desc* g, cudaStream_t stream) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!g->a_mn_major) rc = encode_2d(&tmA, g->A, g->M, g->K, g->lda, BK, BM);
  else rc = encode_2d(&tmA, g->A, g->K, g->M, g->lda, 64, BK);
  if (rc) return rc;
  if (!g->b_mn_major) rc = encode_2d(&tmB, g->B, g->N, g->K, g->ldb, BK, BN);
  else rc = encode_2d(&tmB, g->B, g->K, g->N, g->ldb, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.M = g->M; p.N = g->N; p.K = g->K; p.a_mn = g->a_mn_major; p.b_mn = g->b_mn_major; p.epi = g->epilogue;
  p.D = g->D; p.D2 = g->D2; p.bias = g->bias; p.aux = g->aux; p.ldd = g->ldd; p.ld_aux = g->ld_aux ? g->ld_aux : g->ldd;
  p.status = bb_device_status_word();
  static bool attr_set = false;
  if (!attr_set) {
    BB_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr_set = true;
  }
  const int tiles = ((g->M + BM - 1) / BM) * ((g->N + BN - 1) / BN);
  int grid = bb_num_sms();
  if (g->max_ctas > 0 && g->max_ctas < grid) grid = g->max_ctas;
  if (tiles < grid) grid = tiles;
  gemm_bf16_tcgen05_kernel<BN><<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, p);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

}  // namespace

extern "C" int bb_gemm_bf16(const bb_gemm_desc* g, void* stream) {
  if (!g || !g->A || !g->B || !g->D || g->M <= 0 || g->N <= 0 || g->K <= 0) {
    bb_set_last_error_msg("bb_gemm_bf16: null operand or non-positive size");
    return BB_ERR_INVALID_ARG;
  }
  const int e = g->epilogue;
  if (e < BB_EPI_STORE || e > BB_EPI_BIAS_RESIDUAL) { bb_set_last_error_msg("bb_gemm_bf16: unknown epilogue"); return BB_ERR_INVALID_ARG; }
  if ((e == BB_EPI_BIAS || e == BB_EPI_BIAS_GELU || e == BB_EPI_BIAS_RESIDUAL) && !g->bias) {
    bb_set_last_error_msg("bb_gemm_bf16: epilogue needs bias"); return BB_ERR_INVALID_ARG; }
  if (e == BB_EPI_BIAS_GELU && !g->D2) { bb_set_last_error_msg("bb_gemm_bf16: GeLU epilogue needs D2"); return BB_ERR_INVALID_ARG; }
  if ((e == BB_EPI_MUL_DGELU || e == BB_EPI_BIAS_RESIDUAL) && !g->aux) {
    bb_set_last_error_msg("bb_gemm_bf16: epilogue needs aux"); return BB_ERR_INVALID_ARG; }
  const bool f32 = (e == BB_EPI_ACCUM_F32 || e == BB_EPI_STORE_F32);
  if (g->lda % 8 || g->ldb % 8 || g->ldd % (f32 ? 4 : 8) || (g->ld_aux % 8) ||
      ((uintptr_t)g->A & 15) || ((uintptr_t)g->B & 15) || ((uintptr_t)g->D & 15) || ((uintptr_t)g->D2 & 15) ||
      ((uintptr_t)g->aux & 15) || ((uintptr_t)g->bias & 15)) {
    bb_set_last_error_msg("bb_gemm_bf16: pointers must be 16-byte aligned and leading dimensions multiples of 8 elements");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int bn = g->tile_n;
  if (bn == 0) {
    // 256-wide tiles halve the A re-reads; use them when they still fill the machine
    const long long tiles256 = (long long)((g->M + BM - 1) / BM) * ((g->N + 255) / 256);
    bn = (g->N > 128 && tiles256 >= bb_num_sms()) ? 256 : 128;
  }
  if (bn == 256) return launch<256>(g, s);
  if (bn == 128) return launch<128>(g, s);
  bb_set_last_error_msg("bb_gemm_bf16: tile_n must be 0, 128 or 256");
  return BB_ERR_INVALID_ARG;
}
