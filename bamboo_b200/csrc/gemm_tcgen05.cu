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
#include "tma_host.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 320;   // TMA warp, MMA warp, two epilogue groups of four warps
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
// Epilogue staging: output panels of 128 rows x 128 bytes (64 bf16 or 32 fp32 columns) in the
// 128-byte-swizzled layout a TMA store expects.  Two panels: double-buffered for one output,
// one each for the two outputs of the GeLU epilogue (shared memory is better spent on
// main-loop stages: the kernel is bound by operand bytes in flight).
constexpr int PANEL_BYTES = BM * 128;
constexpr int NUM_PANELS = 2;

template <int BN> struct Cfg {
  static constexpr int B_STAGE_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + NUM_PANELS * PANEL_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int epi;
  int ksplit, kb_per_split;   // split-K work units (fp32 add-reduction epilogue only)
  void* D; void* D2; const void* bias; const void* aux;
  long long ldd, ld_aux;
  int* status;
};

__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  f[0] = bb::bf16_lo(q.x); f[1] = bb::bf16_hi(q.x); f[2] = bb::bf16_lo(q.y); f[3] = bb::bf16_hi(q.y);
  f[4] = bb::bf16_lo(q.z); f[5] = bb::bf16_hi(q.z); f[6] = bb::bf16_lo(q.w); f[7] = bb::bf16_hi(q.w);
}

// One output row's slice of a panel (128 bytes = 8 chunks of 16 bytes) into swizzled shared memory.
__device__ __forceinline__ void panel_store_row_bf16(uint8_t* panel, int row, const float* v /*64*/) {
  uint8_t* base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = bb::pack_bf16x2(v[8 * c + 0], v[8 * c + 1]); q.y = bb::pack_bf16x2(v[8 * c + 2], v[8 * c + 3]);
    q.z = bb::pack_bf16x2(v[8 * c + 4], v[8 * c + 5]); q.w = bb::pack_bf16x2(v[8 * c + 6], v[8 * c + 7]);
    *reinterpret_cast<uint4*>(base + ((c ^ (row & 7)) << 4)) = q;
  }
}
__device__ __forceinline__ void panel_load_row_bf16(const uint8_t* panel, int row, float* x /*64*/) {
  const uint8_t* base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) unpack8(*reinterpret_cast<const uint4*>(base + ((c ^ (row & 7)) << 4)), x + 8 * c);
}
__device__ __forceinline__ void panel_store_row_f32(uint8_t* panel, int row, const float* v /*32*/) {
  uint8_t* base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(base + ((c ^ (row & 7)) << 4)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

// bias[n0 .. n0+W) added to v; columns past N read as zero
template <int W>
__device__ __forceinline__ void add_bias(const GemmParams& p, int n0, float* v) {
  const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + n0;
  if (n0 + W <= p.N) {
#pragma unroll
    for (int i = 0; i < W; i += 8) {
      float f[8]; unpack8(__ldg(reinterpret_cast<const uint4*>(b + i)), f);
#pragma unroll
      for (int k = 0; k < 8; ++k) v[i + k] += f[k];
    }
  } else {
    for (int i = 0; i < W && n0 + i < p.N; ++i) v[i] += __bfloat162float(b[i]);
  }
}

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmD2,
                         const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms need 1024-byte aligned stage buffers
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::STAGES * A_STAGE_BYTES;
  uint8_t* panels = smem + C::STAGES * C::STAGE_BYTES;   // NUM_PANELS x 16 KiB, 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(panels + NUM_PANELS * PANEL_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES]
  uint64_t* empty_bar = bars + C::STAGES;         // [STAGES]
  uint64_t* tmem_full = bars + 2 * C::STAGES;     // [2]
  uint64_t* tmem_empty = bars + 2 * C::STAGES + 2;  // [2]
  uint64_t* aux_bar = bars + 2 * C::STAGES + 4;     // [2] one per epilogue group: aux panel landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_mn = num_m * num_n;
  const int num_tiles = num_mn * p.ksplit;        // work units: (m, n, k-split)
  const int total_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) { bb::mbar_init(&full_bar[s], 1); bb::mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { bb::mbar_init(&tmem_full[a], 1); bb::mbar_init(&tmem_empty[a], 8); bb::mbar_init(&aux_bar[a], 1); }
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tmA);
    bb::tma_prefetch_desc(&tmB);
    bb::tma_prefetch_desc(&tmD);
    if (p.epi == BB_EPI_BIAS_GELU || p.epi == BB_EPI_MUL_DGELU || p.epi == BB_EPI_BIAS_RESIDUAL) bb::tma_prefetch_desc(&tmD2);
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
        const int mn = tile % num_mn, ks = tile / num_mn;
        const int m0 = (mn % num_m) * BM, n0 = (mn / num_m) * BN;
        const int kb0 = ks * p.kb_per_split, kb1 = min(total_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
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
      const int ks = tile / num_mn;
      const int num_kb = min(total_kb, (ks + 1) * p.kb_per_split) - ks * p.kb_per_split;
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
    // ------------------------------------------------ epilogue: two groups of 4 warps (one TMEM lane quarter per warp)
    // Per 128-byte-wide output panel: TMEM -> registers -> fused math -> swizzled shared
    // memory -> one TMA store (or fp32 add-reduction) issued by the group's first thread.
    // The groups take alternate panels.  GeLU (two outputs) sends the pre-activation and then the
    // activation through the same staging panel; the GeLU math overlaps the first store's read.
    const int eg = (warp - 2) >> 2;                // epilogue group 0 / 1
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // row inside the tile == TMEM lane
    const bool leader = (threadIdx.x == 64 + 128 * eg);
    const int epi = p.epi;
    const bool f32 = (epi == BB_EPI_ACCUM_F32 || epi == BB_EPI_STORE_F32);
    const bool dual = (epi == BB_EPI_BIAS_GELU);
    const bool has_aux = (epi == BB_EPI_MUL_DGELU || epi == BB_EPI_BIAS_RESIDUAL);
    uint32_t aux_uses = 0;                         // completed aux loads of this group (barrier phase)
    uint8_t* panel = panels + eg * PANEL_BYTES;    // this group's staging panel
    int acc = 0; uint32_t acc_phase = 0;
    bool alive = true;
    for (int tile = blockIdx.x; tile < num_tiles && alive; tile += gridDim.x) {
      const int mn = tile % num_mn;
      const int m0 = (mn % num_m) * BM, n0 = (mn / num_m) * BN;
      // the four warps of a group share named barriers below: all continue or all leave
      const bool got = bb::mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status);
      if (!bb::named_bar_all(3 + eg, 128, got)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      const int width = f32 ? 32 : 64;             // columns per panel
      const int npanels = BN / width;
      const int first = eg, step = 2;
#pragma unroll 1
      for (int pn = first; pn < npanels; pn += step) {
        const int nb = n0 + pn * width;
        float v[64];
        {
          uint32_t r[32];
          bb::tmem_ld_32x32b_x32(t_row + pn * width, r);
          bb::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (!f32) {
            bb::tmem_ld_32x32b_x32(t_row + pn * width + 32, r);
            bb::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[32 + i] = __uint_as_float(r[i]);
          }
        }
        if (pn + step >= npanels) {
          // this group has read its share of the accumulator: hand it back before the last stores
          bb::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) bb::mbar_arrive(&tmem_empty[acc]);
        }
        if (nb >= p.N) continue;                   // panel entirely outside the matrix (uniform)
        // the panel must have been read by its previous store before it is overwritten
        if (leader) bb::bulk_wait_group_read<0>();
        if (has_aux) {
          // the [128 x 64] aux tile (second operand of the epilogue) comes in by TMA into the
          // staging panel; each thread then reads and rewrites only its own row
          if (leader) {
            bb::mbar_arrive_expect_tx(&aux_bar[eg], PANEL_BYTES);
            bb::tma_load_2d(panel, &tmD2, &aux_bar[eg], nb, m0);
          }
          const bool landed = bb::mbar_wait(&aux_bar[eg], aux_uses & 1, abort_flag, p.status);
          if (!bb::named_bar_all(3 + eg, 128, landed)) { alive = false; break; }
          ++aux_uses;
        } else {
          bb::named_bar_sync(1 + eg, 128);
        }
        if (f32) {
          panel_store_row_f32(panel, row, v);
        } else {
          if (epi == BB_EPI_BIAS || dual || epi == BB_EPI_BIAS_RESIDUAL) add_bias<64>(p, nb, v);
          if (dual) {
            panel_store_row_bf16(panel, row, v);   // pre-activation first
            bb::fence_proxy_async();
            bb::named_bar_sync(1 + eg, 128);
            if (leader) { bb::tma_store_2d(&tmD2, panel, nb, m0); bb::bulk_commit_group(); }
            // GeLU of the bf16-rounded pre-activation: forward and backward (which re-reads the
            // stored pre-activation) see the same argument
#pragma unroll
            for (int i = 0; i < 64; ++i) v[i] = bb::gelu_tanh(__bfloat162float(__float2bfloat16(v[i])));
            if (leader) bb::bulk_wait_group_read<0>();
            bb::named_bar_sync(1 + eg, 128);
          } else if (has_aux) {
            float x[64];
            panel_load_row_bf16(panel, row, x);
            if (epi == BB_EPI_MUL_DGELU) {
#pragma unroll
              for (int i = 0; i < 64; ++i) v[i] *= bb::gelu_tanh_grad(x[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 64; ++i) v[i] += x[i];
            }
          }
          panel_store_row_bf16(panel, row, v);
        }
        bb::fence_proxy_async();                   // generic-proxy writes -> visible to the TMA engine
        bb::named_bar_sync(1 + eg, 128);
        if (leader) {
          if (epi == BB_EPI_ACCUM_F32) bb::tma_reduce_add_2d(&tmD, panel, nb, m0);
          else bb::tma_store_2d(&tmD, panel, nb, m0);
          bb::bulk_commit_group();
        }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (leader) bb::bulk_wait_group<0>();          // all stores landed before shared memory goes away
  }

  bb::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) bb::tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ---------------------------------------------------------------- host side
using bbhost::encode_2d;

template <int BN>
int launch(const bb_gemm_desc* g, cudaStream_t stream) {
  using C = Cfg<BN>;
  CUtensorMap tmA, tmB, tmD, tmD2;
  int rc;
  const int out_f32 = (g->epilogue == BB_EPI_ACCUM_F32 || g->epilogue == BB_EPI_STORE_F32);
  rc = encode_2d(&tmD, g->D, g->M, g->N, g->ldd, out_f32 ? 32 : 64, BM, out_f32);
  if (rc) return rc;
  tmD2 = tmD;
  if (g->epilogue == BB_EPI_BIAS_GELU) {
    rc = encode_2d(&tmD2, g->D2, g->M, g->N, g->ldd, 64, BM, 0);
    if (rc) return rc;
  } else if (g->epilogue == BB_EPI_MUL_DGELU || g->epilogue == BB_EPI_BIAS_RESIDUAL) {
    rc = encode_2d(&tmD2, g->aux, g->M, g->N, g->ld_aux ? g->ld_aux : g->ldd, 64, BM, 0);   // the aux operand
    if (rc) return rc;
  }
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
  const int total_kb = (g->K + BK - 1) / BK;
  const int mn_tiles = ((g->M + BM - 1) / BM) * ((g->N + BN - 1) / BN);
  int ksplit = 1;
  if (g->epilogue == BB_EPI_ACCUM_F32) {
    if (g->split_k > 0) {
      ksplit = g->split_k;
    } else {
      // too few output tiles to fill the machine: split the reduction; partial sums meet in
      // the fp32 add-reduction of the epilogue.  Cost model: waves x (k-blocks + fixed overhead).
      const int sms = bb_num_sms();
      long long best = -1;
      for (int s = 1; s <= 16; ++s) {
        const int kbs = (total_kb + s - 1) / s;
        if (s > 1 && kbs < 8) break;
        const long long waves = ((long long)mn_tiles * s + sms - 1) / sms;
        const long long cost = waves * (kbs + 8);
        if (best < 0 || cost < best) { best = cost; ksplit = s; }
      }
    }
  }
  if (ksplit > total_kb) ksplit = total_kb;
  if (ksplit < 1) ksplit = 1;
  p.kb_per_split = (total_kb + ksplit - 1) / ksplit;
  p.ksplit = (total_kb + p.kb_per_split - 1) / p.kb_per_split;   // no empty splits
  static bool attr_set = false;
  if (!attr_set) {
    BB_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr_set = true;
  }
  const int tiles = mn_tiles * p.ksplit;
  int grid = bb_num_sms();
  if (g->max_ctas > 0 && g->max_ctas < grid) grid = g->max_ctas;
  if (tiles < grid) grid = tiles;
  gemm_bf16_tcgen05_kernel<BN><<<grid, NUM_THREADS, C::SMEM_BYTES, stream>>>(tmA, tmB, tmD, tmD2, p);
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
  // cuTensorMapEncodeTiled is a driver call and needs a context bound to the calling thread;
  // a thread that has only ever set its device (autograd worker threads) has none yet.
  if (int rc = bbhost::bind_context()) return rc;
  int bn = g->tile_n;
  if (bn == 0) {
    // 256-wide tiles halve the A re-reads; use them when they still fill the machine
    const long long tiles256 = (long long)((g->M + BM - 1) / BM) * ((g->N + 255) / 256);
    // the add-reduction epilogue can split K to fill the machine, so it always takes wide tiles
    bn = (g->N > 128 && (tiles256 >= bb_num_sms() || e == BB_EPI_ACCUM_F32)) ? 256 : 128;
  }
  if (bn == 256) return launch<256>(g, s);
  if (bn == 128) return launch<128>(g, s);
  bb_set_last_error_msg("bb_gemm_bf16: tile_n must be 0, 128 or 256");
  return BB_ERR_INVALID_ARG;
}
