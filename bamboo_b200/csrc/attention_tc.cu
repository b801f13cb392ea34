// Fused attention on the 5th-generation tensor cores: head dimension 64 (forward and backward) and 128 (forward).
//
// Every contraction (Q.K^T, P.V, dO.V^T, dS.K, P^T.dO, dS^T.Q) is a tcgen05.mma with fp32
// accumulators in tensor memory; tiles arrive by TMA into 128-byte-swizzled shared memory;
// the same [128 x 64] tile serves as a K-major operand (reduction over the head dimension) and
// as an MN-major operand (reduction over its rows) just by changing the matrix descriptor, so
// nothing is transposed.  Probabilities are recomputed from the saved log-sum-exp in the
// backward pass; scores never reach HBM.
//
// In every kernel warp 0 issues TMA, one or two warps issue MMAs and the remaining warps (one TMEM
// lane quarter each) do the softmax / element-wise work and the final stores.  Kernels:
//   forward          : CTA owns 256 query rows as two tiles in ping-pong (one softmax group per tile),
//                      the output row accumulates in tensor memory; templated on the head dimension;
//   fused backward   : CTA owns 128 key rows, streams 64-row query / dO sub-tiles, computes the scores
//                      once and produces dK, dV (fixed summation order) and dQ (fp32 add-reductions
//                      into an accumulator that a small kernel scales and converts);
//   two-role backward: dK/dV CTAs and dQ CTAs in one launch, scores computed by both roles, every
//                      sum in a fixed order (no reductions) - selected by BB_ATTENTION_BWD=split.
#include "tma_host.cuh"
#include <math.h>
#include <stdlib.h>

namespace {

constexpr int TQ = 128;        // rows per tile (queries or keys)
constexpr int HD = 64;         // head dimension
constexpr int TILE_BYTES = TQ * HD * 2;          // 16 KiB: [128 x 64] bf16, 128-byte rows
constexpr float LOG2E = 1.4426950408889634f;

struct TcParams {
  const __nv_bfloat16* o;       // forward output (delta kernel)
  __nv_bfloat16 *out, *dq, *dk, *dv;
  float* lse;                   // [B, H, S]
  float* delta;                 // [B, H, S]
  float* dq_acc;                // [B, H, S, 64] fp32 sums of dQ (fused backward), or null
  long long stride_o, stride_dqkv;
  int B, H, S;
  int hidden;                   // H * 64: column offset between q, k and v in the packed projection
  int causal;
  float scale;
  int* status;
};

// instruction descriptor: bf16 x bf16 -> fp32, M = 128
__device__ __forceinline__ uint32_t idesc(int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(TQ >> 4) << 24);
}
// Matrix descriptors.  The MMA-issuing warp shares its scheduler with compute warps, so the
// instructions spent per MMA count: a tile's descriptor is built once (`desc_*0`) and every later
// k-step only adds a constant to its address field (16-byte units; no carry into the next field
// for any shared-memory address).
// [rows x 64] tile, reduction over the 64 columns: k-step = 16 columns = 32 bytes
__device__ __forceinline__ uint64_t desc_k0(uint32_t tile) { return bb::make_smem_desc_sw128(tile, 16, 1024); }
__device__ __forceinline__ uint64_t desc_kmajor(uint64_t d0, int kstep) { return d0 + (uint64_t)(kstep * (32 >> 4)); }
// [rows x 64] tile, reduction over its rows (N or M = the 64 columns): k-step = 16 rows = 2 KiB
__device__ __forceinline__ uint64_t desc_mn0(uint32_t tile) { return bb::make_smem_desc_sw128(tile, 8192, 1024); }
__device__ __forceinline__ uint64_t desc_mnmajor64(uint64_t d0, int kstep) { return d0 + (uint64_t)(kstep * (2048 >> 4)); }
__device__ __forceinline__ void pack32(const float* v, uint32_t* out16) {
#pragma unroll
  for (int i = 0; i < 16; ++i) out16[i] = bb::pack_bf16x2(v[2 * i], v[2 * i + 1]);
}
// half a row (64 bytes: chunks 4*half .. 4*half+3) of a [128 x 64] bf16 atom from 16 packed registers
__device__ __forceinline__ void atom_store_half_row(uint8_t* atom, int row, int half, const uint32_t* pk) {
  uint8_t* base = atom + row * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(base + (((4 * half + c) ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// two 32-column TMEM reads in flight, one wait
__device__ __forceinline__ void ld32x2(uint32_t ta, uint32_t tb, float* a, float* b) {
  uint32_t ra[32], rb[32];
  bb::tmem_ld_32x32b_x32(ta, ra);
  bb::tmem_ld_32x32b_x32(tb, rb);
  bb::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) { a[i] = __uint_as_float(ra[i]); b[i] = __uint_as_float(rb[i]); }
}
__device__ __forceinline__ void ld32(uint32_t taddr, float* v) {
  uint32_t r[32];
  bb::tmem_ld_32x32b_x32(taddr, r);
  bb::tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// one row of 64 fp32 values -> bf16 in global memory (128 contiguous bytes)
__device__ __forceinline__ void store_row64(__nv_bfloat16* dst, const float* v, float mul) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 q;
    q.x = bb::pack_bf16x2(v[8 * c + 0] * mul, v[8 * c + 1] * mul); q.y = bb::pack_bf16x2(v[8 * c + 2] * mul, v[8 * c + 3] * mul);
    q.z = bb::pack_bf16x2(v[8 * c + 4] * mul, v[8 * c + 5] * mul); q.w = bb::pack_bf16x2(v[8 * c + 6] * mul, v[8 * c + 7] * mul);
    reinterpret_cast<uint4*>(dst)[c] = q;
  }
}

// 32 fp32 values of one row -> bf16 in global memory (64 contiguous bytes)
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const float* v, float mul) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = bb::pack_bf16x2(v[8 * c + 0] * mul, v[8 * c + 1] * mul); q.y = bb::pack_bf16x2(v[8 * c + 2] * mul, v[8 * c + 3] * mul);
    q.z = bb::pack_bf16x2(v[8 * c + 4] * mul, v[8 * c + 5] * mul); q.w = bb::pack_bf16x2(v[8 * c + 6] * mul, v[8 * c + 7] * mul);
    reinterpret_cast<uint4*>(dst)[c] = q;
  }
}

// shared-memory bookkeeping common to the three kernels
struct Ctl {
  uint64_t bars[32];
  uint32_t tmem_slot;
  int abort_flag;
};


// delta[b, h, s] = sum_d dO * O.  Eight lanes per (token, head): each loads 16 bytes of O and dO
// (a warp reads four consecutive heads of a token: 512 contiguous bytes per operand), two
// independent units per thread for memory-level parallelism.  The same pass clears the fp32
// accumulator of the fused backward kernel, when there is one.
__global__ void __launch_bounds__(256)
attn_tc_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o, const TcParams p) {
  const int per_tok = p.H * 8;                                 // 16-byte chunks per token row
  const long long total = (long long)p.B * p.S * per_tok;
  const long long stride = (long long)gridDim.x * blockDim.x;
  if (p.dq_acc) {
    float4* z = reinterpret_cast<float4*>(p.dq_acc);
    const long long n4 = (long long)p.B * p.H * p.S * (HD / 4);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) z[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // the trip count is uniform within a warp (the shuffles below need every lane)
  for (long long w = (long long)blockIdx.x * blockDim.x + (threadIdx.x & ~31); w < total; w += 2 * stride) {
    const long long c = w + (threadIdx.x & 31);
    float s[2];
    long long cc[2] = {c, c + stride};
    uint4 a[2], b[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      a[u] = make_uint4(0, 0, 0, 0); b[u] = a[u];
      if (cc[u] < total) {
        const long long tok = cc[u] / per_tok; const int within = (int)(cc[u] % per_tok);
        a[u] = __ldg(reinterpret_cast<const uint4*>(o + tok * p.stride_o + within * 8));
        b[u] = __ldg(reinterpret_cast<const uint4*>(d_o + tok * p.stride_o + within * 8));
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const uint32_t x[4] = {a[u].x, a[u].y, a[u].z, a[u].w}, y[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
      float t = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) t += bb::bf16_lo(x[i]) * bb::bf16_lo(y[i]) + bb::bf16_hi(x[i]) * bb::bf16_hi(y[i]);
      t += __shfl_xor_sync(0xffffffffu, t, 1);
      t += __shfl_xor_sync(0xffffffffu, t, 2);
      t += __shfl_xor_sync(0xffffffffu, t, 4);
      s[u] = t;
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (cc[u] < total && (threadIdx.x & 7) == 0) {
        const long long tok = cc[u] / per_tok; const int head = (int)(cc[u] % per_tok) >> 3;
        p.delta[((tok / p.S) * p.H + head) * p.S + (tok % p.S)] = s[u];
      }
    }
  }
}

// =====================================================================================
// Pipelined backward kernels: 64-wide sub-blocks, every hand-off double-buffered, two compute
// groups (warps 2-5 and 6-9) that take alternate sub-blocks, so the tensor core always has the
// next S / dP and the previous dK / dV / dQ update queued while a group does its elementwise work.
// =====================================================================================
constexpr int SUB = 64;                          // streamed rows per sub-block
constexpr int SUB_BYTES = SUB * HD * 2;          // 8 KiB: [64 x 64] bf16
// Two compute groups of 8 warps.  A row's 64 scores are split between two threads (warps w and
// w + 4 of a group reach the same TMEM lane quarter): the element-wise work has no row
// reductions here, and four compute warps per scheduler hide the TMEM-load and ALU latencies that
// two could not (issue slots were 35 % busy with 4-warp groups).
constexpr int GROUP_THREADS = 256;
constexpr int NT2 = 64 + 2 * GROUP_THREADS;
constexpr int NST = 6;                           // streamed sub-tile ring depth
constexpr int NSB = 3;                           // score buffers in tensor memory

// ------------------------------------------------------------------ dQ (pipelined)
// smem: Q, dO [128 x 64] | K, V sub-tiles [64 x 64] x 3 stages | dS [128 q x 64 kv] x 2
// TMEM: S 2 x 64 | dP 2 x 64 | dQ 64
__device__ __forceinline__ void
attn_tc_dq2_body(const CUtensorMap& tm_q, const CUtensorMap& tm_kv, const CUtensorMap& tm_do, const TcParams& p,
                 const int bx, const int nbx) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + TILE_BYTES;
  uint8_t* sK = sDO + TILE_BYTES;              // NST stages x 8 KiB
  uint8_t* sV = sK + NST * SUB_BYTES;          // NST stages x 8 KiB
  uint8_t* sDS = sV + NST * SUB_BYTES;         // 2 x 16 KiB
  Ctl* ctl = reinterpret_cast<Ctl*>(sDS + 2 * TILE_BYTES);
  uint64_t* q_full = &ctl->bars[0];
  uint64_t* kv_full = &ctl->bars[1];           // [NST]
  uint64_t* kv_empty = &ctl->bars[1 + NST];    // [NST]
  uint64_t* s_full = &ctl->bars[1 + 2 * NST];  // [NSB]
  uint64_t* s_empty = s_full + NSB;            // [NSB]
  uint64_t* ds_full = s_empty + NSB;           // [2]
  uint64_t* ds_empty = ds_full + 2;            // [2]
  uint64_t* acc_full = ds_empty + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = nbx - 1 - bx, head = blockIdx.y, batch = blockIdx.z;
  const int q0 = qb * TQ;
  const int row_base = batch * p.S;
  const int colq = head * HD, colk = p.hidden + head * HD, colv = 2 * p.hidden + head * HD;
  int nblk = (p.S + SUB - 1) / SUB;
  if (p.causal) nblk = min(nblk, (q0 + TQ) / SUB);

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    bb::mbar_init(q_full, 1);
    for (int i = 0; i < NST; ++i) { bb::mbar_init(&kv_full[i], 1); bb::mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < NSB; ++i) { bb::mbar_init(&s_full[i], 1); bb::mbar_init(&s_empty[i], GROUP_THREADS / 32); }
    for (int i = 0; i < 2; ++i) { bb::mbar_init(&ds_full[i], GROUP_THREADS / 32); bb::mbar_init(&ds_empty[i], 1); }
    bb::mbar_init(acc_full, 1);
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tm_q); bb::tma_prefetch_desc(&tm_kv); bb::tma_prefetch_desc(&tm_do);
  }
  if (warp == 1) { bb::tmem_alloc(&ctl->tmem_slot, 512); bb::tmem_relinquish(); }
  bb::tc_fence_before_sync();
  __syncthreads();
  bb::tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t tDQ = tmem + 384;             // S[b] at tmem + 64 b, dP[b] at tmem + 192 + 64 b (b < 3)

  if (warp == 0) {
    if (lane == 0) {
      bb::mbar_arrive_expect_tx(q_full, 2 * TILE_BYTES);
      bb::tma_load_2d(sQ, &tm_q, q_full, colq, row_base + q0);
      bb::tma_load_2d(sDO, &tm_do, q_full, colq, row_base + q0);
      for (int j = 0; j < nblk; ++j) {
        const int s = j % NST;
        if (!bb::mbar_wait(&kv_empty[s], ((j / NST) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::mbar_arrive_expect_tx(&kv_full[s], 2 * SUB_BYTES);
        bb::tma_load_2d(sK + s * SUB_BYTES, &tm_kv, &kv_full[s], colk, row_base + j * SUB);
        bb::tma_load_2d(sV + s * SUB_BYTES, &tm_kv, &kv_full[s], colv, row_base + j * SUB);
      }
    }
  } else if (warp == 1) {
    const uint64_t dQ0 = desc_k0(bb::smem_u32(sQ)), dDO0 = desc_k0(bb::smem_u32(sDO));
    const uint64_t dK0 = desc_k0(bb::smem_u32(sK)), dV0 = desc_k0(bb::smem_u32(sV));     // stage 0; stage s: + s * SUB_BYTES / 16
    const uint64_t dKm0 = desc_mn0(bb::smem_u32(sK)), dDS0 = desc_k0(bb::smem_u32(sDS));
    const uint32_t i_s = idesc(64, 0, 0), i_dq = idesc(64, 0, 1);
    bool alive = bb::mbar_wait(q_full, 0, &ctl->abort_flag, p.status);
    // software pipeline: the scores run two sub-blocks ahead of the dQ updates
    for (int j = 0; j < nblk + 2 && alive; ++j) {
      if (j < nblk) {
        const int s = j % NST, b = j % NSB;
        if (!bb::mbar_wait(&kv_full[s], (j / NST) & 1, &ctl->abort_flag, p.status)) break;
        if (!bb::mbar_wait(&s_empty[b], ((j / NSB) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint64_t dK = dK0 + (uint64_t)(s * (SUB_BYTES >> 4)), dV = dV0 + (uint64_t)(s * (SUB_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            bb::umma_f16(tmem + 64 * b, desc_kmajor(dQ0, k), desc_kmajor(dK, k), i_s, k > 0);
            bb::umma_f16(tmem + 192 + 64 * b, desc_kmajor(dDO0, k), desc_kmajor(dV, k), i_s, k > 0);
          }
          bb::umma_commit(&s_full[b]);
        }
        __syncwarp();
      }
      if (j >= 2) {
        const int jj = j - 2, s2 = jj % NST, b2 = jj & 1;
        if (!bb::mbar_wait(&ds_full[b2], (jj >> 1) & 1, &ctl->abort_flag, p.status)) break;
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint64_t dK2 = dKm0 + (uint64_t)(s2 * (SUB_BYTES >> 4)), dDS = dDS0 + (uint64_t)(b2 * (TILE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k) bb::umma_f16(tDQ, desc_kmajor(dDS, k), desc_mnmajor64(dK2, k), i_dq, (jj > 0 || k > 0));
          bb::umma_commit(&ds_empty[b2]);
          bb::umma_commit(&kv_empty[s2]);
          if (jj == nblk - 1) bb::umma_commit(acc_full);
        }
        __syncwarp();
      }
    }
  } else {
    const int g = (warp - 2) >> 3;                           // compute group = buffer index
    const int hf = ((warp - 2) >> 2) & 1;                    // which 32 of the sub-block's 64 columns
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qrow = q0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float* lse_g = p.lse + ((long long)batch * p.H + head) * p.S;
    const float* delta_g = p.delta + ((long long)batch * p.H + head) * p.S;
    const float lse = (qrow < p.S) ? lse_g[qrow] * LOG2E : 0.f;
    const float dl = (qrow < p.S) ? delta_g[qrow] : 0.f;
    const float sl = p.scale * LOG2E;
    uint8_t* myDS = sDS + g * TILE_BYTES;
    bool alive = true;
    int n = 0;                                               // this group's iteration count
    for (int j = g; j < nblk && alive; j += 2, ++n) {
      const int sb = j % NSB;
      const uint32_t tS = tmem + 64 * sb, tDP = tmem + 192 + 64 * sb;
      const bool ok = bb::mbar_wait(&s_full[sb], (j / NSB) & 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const int c0 = j * SUB + hf * 32;
      // only sub-blocks that touch the sequence end or the causal diagonal need per-element masks
      const bool need_mask = (c0 + 32 > p.S) || (p.causal && c0 + 32 - 1 > q0);
      const float nlse = -lse;
      uint32_t pk[16];                                       // this thread's 32 dS values as bf16 pairs
      {
        float sv[32], dp[32];
        ld32x2(tS + lane_addr + hf * 32, tDP + lane_addr + hf * 32, sv, dp);
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) dp[i] = ex2(fmaf(sv[i], sl, nlse)) * (dp[i] - dl);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = c0 + i;
            float pv = ex2(fmaf(sv[i], sl, nlse));
            if (col >= p.S || (p.causal && col > qrow)) pv = 0.f;
            dp[i] = pv * (dp[i] - dl);
          }
        }
        pack32(dp, pk);
      }
      bb::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) bb::mbar_arrive(&s_empty[sb]);          // scores consumed: the MMA warp may refill
      // the staging buffer is free once the dQ update that read it two sub-blocks ago retired
      const bool ok2 = bb::mbar_wait(&ds_empty[g], (n & 1) ^ 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok2)) { alive = false; break; }
      atom_store_half_row(myDS, row, hf, pk);
      bb::fence_proxy_async();
      __syncwarp();
      if (lane == 0) bb::mbar_arrive(&ds_full[g]);
    }
    const bool fin = alive && bb::mbar_wait(acc_full, 0, &ctl->abort_flag, p.status);
    if (bb::named_bar_all(3 + g, GROUP_THREADS, fin) && g == 0) {
      bb::tc_fence_after_sync();
      float v[32];
      ld32(tDQ + lane_addr + hf * 32, v);
      if (qrow < p.S) store_row32(p.dq + (long long)(row_base + qrow) * p.stride_dqkv + colq + hf * 32, v, p.scale);
    }
  }
  bb::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) bb::tmem_dealloc(tmem, 512);
}

constexpr int DQ2_SMEM = 2 * TILE_BYTES + 2 * NST * SUB_BYTES + 2 * TILE_BYTES + (int)sizeof(Ctl) + 1024;

// ------------------------------------------------------------------ dK, dV (pipelined)
// smem: K, V [128 x 64] | Q, dO sub-tiles [64 x 64] x 3 stages | P^T, dS^T [128 kv x 64 q] x 2 each
//       | per-group lse / delta of the sub-block's 64 query columns
// TMEM: S^T 2 x 64 | dP^T 2 x 64 | dV 64 | dK 64
__device__ __forceinline__ void
attn_tc_dkv2_body(const CUtensorMap& tm128, const CUtensorMap& tm64, const CUtensorMap& tm_do64, const TcParams& p, const int bx) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;               // NST stages x 8 KiB
  uint8_t* sDO = sQ + NST * SUB_BYTES;         // NST stages x 8 KiB
  uint8_t* sP = sDO + NST * SUB_BYTES;         // 2 x 16 KiB
  uint8_t* sDS = sP + 2 * TILE_BYTES;          // 2 x 16 KiB
  float* s_lse = reinterpret_cast<float*>(sDS + 2 * TILE_BYTES);   // [2][64]
  float* s_delta = s_lse + 2 * SUB;                                // [2][64]
  Ctl* ctl = reinterpret_cast<Ctl*>(s_delta + 2 * SUB);
  uint64_t* kv_full = &ctl->bars[0];
  uint64_t* q_full = &ctl->bars[1];            // [NST]
  uint64_t* q_empty = &ctl->bars[1 + NST];     // [NST]
  uint64_t* s_full = &ctl->bars[1 + 2 * NST];  // [NSB]
  uint64_t* s_empty = s_full + NSB;            // [NSB]
  uint64_t* p_full = s_empty + NSB;            // [2]
  uint64_t* p_empty = p_full + 2;              // [2]
  uint64_t* acc_full = p_empty + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = bx, head = blockIdx.y, batch = blockIdx.z;
  const int k0 = kb * TQ;
  const int row_base = batch * p.S;
  const int colq = head * HD, colk = p.hidden + head * HD, colv = 2 * p.hidden + head * HD;
  const int nq = (p.S + SUB - 1) / SUB;
  const int qstart = p.causal ? (k0 / SUB) : 0;
  const int nblk = nq - qstart;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    bb::mbar_init(kv_full, 1);
    for (int i = 0; i < NST; ++i) { bb::mbar_init(&q_full[i], 1); bb::mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < NSB; ++i) { bb::mbar_init(&s_full[i], 1); bb::mbar_init(&s_empty[i], GROUP_THREADS / 32); }
    for (int i = 0; i < 2; ++i) { bb::mbar_init(&p_full[i], GROUP_THREADS / 32); bb::mbar_init(&p_empty[i], 1); }
    bb::mbar_init(acc_full, 1);
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tm128); bb::tma_prefetch_desc(&tm64); bb::tma_prefetch_desc(&tm_do64);
  }
  if (warp == 1) { bb::tmem_alloc(&ctl->tmem_slot, 512); bb::tmem_relinquish(); }
  bb::tc_fence_before_sync();
  __syncthreads();
  bb::tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  const uint32_t tDV = tmem + 384, tDK = tmem + 448;   // S^T[b] at tmem + 64 b, dP^T[b] at tmem + 192 + 64 b (b < 3)

  if (warp == 0) {
    if (lane == 0) {
      bb::mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      bb::tma_load_2d(sK, &tm128, kv_full, colk, row_base + k0);
      bb::tma_load_2d(sV, &tm128, kv_full, colv, row_base + k0);
      for (int i = 0; i < nblk; ++i) {
        const int s = i % NST;
        if (!bb::mbar_wait(&q_empty[s], ((i / NST) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::mbar_arrive_expect_tx(&q_full[s], 2 * SUB_BYTES);
        bb::tma_load_2d(sQ + s * SUB_BYTES, &tm64, &q_full[s], colq, row_base + (qstart + i) * SUB);
        bb::tma_load_2d(sDO + s * SUB_BYTES, &tm_do64, &q_full[s], colq, row_base + (qstart + i) * SUB);
      }
    }
  } else if (warp == 1) {
    const uint64_t dK0 = desc_k0(bb::smem_u32(sK)), dV0 = desc_k0(bb::smem_u32(sV));
    const uint64_t dQ0 = desc_k0(bb::smem_u32(sQ)), dDO0 = desc_k0(bb::smem_u32(sDO));   // stage 0; stage s: + s * SUB_BYTES / 16
    const uint64_t dQm0 = desc_mn0(bb::smem_u32(sQ)), dDOm0 = desc_mn0(bb::smem_u32(sDO));
    const uint64_t dP0 = desc_k0(bb::smem_u32(sP)), dDS0 = desc_k0(bb::smem_u32(sDS));
    const uint32_t i_s = idesc(64, 0, 0), i_acc = idesc(64, 0, 1);
    bool alive = bb::mbar_wait(kv_full, 0, &ctl->abort_flag, p.status);
    // the score products run two sub-blocks ahead of the dV / dK updates
    for (int i = 0; i < nblk + 2 && alive; ++i) {
      if (i < nblk) {
        const int s = i % NST, b = i % NSB;
        if (!bb::mbar_wait(&q_full[s], (i / NST) & 1, &ctl->abort_flag, p.status)) break;
        if (!bb::mbar_wait(&s_empty[b], ((i / NSB) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint64_t dQ = dQ0 + (uint64_t)(s * (SUB_BYTES >> 4)), dDO = dDO0 + (uint64_t)(s * (SUB_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            bb::umma_f16(tmem + 64 * b, desc_kmajor(dK0, k), desc_kmajor(dQ, k), i_s, k > 0);
            bb::umma_f16(tmem + 192 + 64 * b, desc_kmajor(dV0, k), desc_kmajor(dDO, k), i_s, k > 0);
          }
          bb::umma_commit(&s_full[b]);
        }
        __syncwarp();
      }
      if (i >= 2) {
        const int ii = i - 2, s2 = ii % NST, b2 = ii & 1;
        if (!bb::mbar_wait(&p_full[b2], (ii >> 1) & 1, &ctl->abort_flag, p.status)) break;
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint64_t dQ2 = dQm0 + (uint64_t)(s2 * (SUB_BYTES >> 4)), dDO2 = dDOm0 + (uint64_t)(s2 * (SUB_BYTES >> 4));
          const uint64_t dP = dP0 + (uint64_t)(b2 * (TILE_BYTES >> 4)), dDS = dDS0 + (uint64_t)(b2 * (TILE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            bb::umma_f16(tDV, desc_kmajor(dP, k), desc_mnmajor64(dDO2, k), i_acc, (ii > 0 || k > 0));
            bb::umma_f16(tDK, desc_kmajor(dDS, k), desc_mnmajor64(dQ2, k), i_acc, (ii > 0 || k > 0));
          }
          bb::umma_commit(&p_empty[b2]);
          bb::umma_commit(&q_empty[s2]);
          if (ii == nblk - 1) bb::umma_commit(acc_full);
        }
        __syncwarp();
      }
    }
  } else {
    const int g = (warp - 2) >> 3;
    const int hf = ((warp - 2) >> 2) & 1;                  // which 32 of the sub-block's 64 query columns
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                   // key row inside the tile
    const int gt = threadIdx.x - 64 - GROUP_THREADS * g;   // thread index inside the group
    const int krow = k0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float* lse_g = p.lse + ((long long)batch * p.H + head) * p.S;
    const float* delta_g = p.delta + ((long long)batch * p.H + head) * p.S;
    const float sl = p.scale * LOG2E;
    uint8_t* myP = sP + g * TILE_BYTES;
    uint8_t* myDS = sDS + g * TILE_BYTES;
    float* my_lse = s_lse + g * SUB;
    float* my_delta = s_delta + g * SUB;
    bool alive = true;
    int n = 0;
    // per-column statistics are fetched one sub-block ahead so their latency is off the critical path
    float nx_lse = 0.f, nx_delta = 0.f;
    if (gt < SUB && g < nblk) {
      const int q = (qstart + g) * SUB + gt;
      if (q < p.S) { nx_lse = lse_g[q] * LOG2E; nx_delta = delta_g[q]; }
    }
    for (int i = g; i < nblk && alive; i += 2, ++n) {
      const int qc0 = (qstart + i) * SUB;
      // (the group's previous readers are past their last use once everybody is through this barrier)
      bb::named_bar_sync(1 + g, GROUP_THREADS);
      if (gt < SUB) { my_lse[gt] = nx_lse; my_delta[gt] = nx_delta; }
      bb::named_bar_sync(1 + g, GROUP_THREADS);
      if (gt < SUB && i + 2 < nblk) {
        const int q = (qstart + i + 2) * SUB + gt;
        nx_lse = (q < p.S) ? lse_g[q] * LOG2E : 0.f;
        nx_delta = (q < p.S) ? delta_g[q] : 0.f;
      }
      const int sb = i % NSB;
      const uint32_t tS = tmem + 64 * sb, tDP = tmem + 192 + 64 * sb;
      const bool ok = bb::mbar_wait(&s_full[sb], (i / NSB) & 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const bool need_mask = (qc0 + SUB > p.S) || (p.causal && k0 + TQ - 1 > qc0);
      uint32_t pkP[16], pkDS[16];                            // this thread's 32 P^T and dS^T values as bf16 pairs
      {
        float sv[32], dp[32];
        ld32x2(tS + lane_addr + hf * 32, tDP + lane_addr + hf * 32, sv, dp);
#pragma unroll
        for (int e4 = 0; e4 < 32; e4 += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(my_lse + hf * 32 + e4);
          const float4 d4 = *reinterpret_cast<const float4*>(my_delta + hf * 32 + e4);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 + u;
            float pv = ex2(fmaf(sv[e], sl, -ls[u]));
            if (need_mask) {
              const int q = qc0 + hf * 32 + e;
              if (q >= p.S || (p.causal && krow > q)) pv = 0.f;
            }
            sv[e] = pv;
            dp[e] = pv * (dp[e] - ds[u]);
          }
        }
        pack32(sv, pkP);
        pack32(dp, pkDS);
      }
      bb::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) bb::mbar_arrive(&s_empty[sb]);
      // the staging buffers are free once the dV / dK update that read them retired
      const bool ok2 = bb::mbar_wait(&p_empty[g], (n & 1) ^ 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok2)) { alive = false; break; }
      atom_store_half_row(myP, row, hf, pkP);
      atom_store_half_row(myDS, row, hf, pkDS);
      bb::fence_proxy_async();
      __syncwarp();
      if (lane == 0) bb::mbar_arrive(&p_full[g]);
    }
    const bool fin = alive && nblk > 0 && bb::mbar_wait(acc_full, 0, &ctl->abort_flag, p.status);
    if (bb::named_bar_all(3 + g, GROUP_THREADS, fin)) {
      bb::tc_fence_after_sync();
      float v[32];
      // the two groups split the final stores: group 0 writes dV, group 1 writes dK
      const uint32_t src = (g == 0) ? tDV : tDK;
      ld32(src + lane_addr + hf * 32, v);
      __nv_bfloat16* dst = (g == 0) ? p.dv : p.dk;
      if (krow < p.S) store_row32(dst + (long long)(row_base + krow) * p.stride_dqkv + colq + hf * 32, v, g == 0 ? 1.f : p.scale);
    }
  }
  bb::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) bb::tmem_dealloc(tmem, 512);
}

constexpr int DKV2_SMEM = 2 * TILE_BYTES + 2 * NST * SUB_BYTES + 4 * TILE_BYTES + 4 * SUB * (int)sizeof(float) + (int)sizeof(Ctl) + 1024;

// Both backward roles in one launch: of the 2 * nbx CTAs of a (batch, head), the first nbx own a
// key tile (dK, dV) and the rest a query tile (dQ).  The two roles are independent, so the tail
// of one fills with CTAs of the other instead of leaving SMs idle between two launches.
constexpr int BWD2_SMEM = DKV2_SMEM > DQ2_SMEM ? DKV2_SMEM : DQ2_SMEM;
__global__ void __launch_bounds__(NT2, 1)
attn_tc_bwd2_kernel(const __grid_constant__ CUtensorMap tm128, const __grid_constant__ CUtensorMap tm64,
                    const __grid_constant__ CUtensorMap tm_do128, const __grid_constant__ CUtensorMap tm_do64, const TcParams p) {
  const int nbx = gridDim.x >> 1;
  if ((int)blockIdx.x < nbx) attn_tc_dkv2_body(tm128, tm64, tm_do64, p, blockIdx.x);
  else attn_tc_dq2_body(tm128, tm64, tm_do128, p, blockIdx.x - nbx, nbx);
}

// ------------------------------------------------------------------ fused backward: dK, dV and dQ from one pass
// A CTA owns 128 key rows and streams the 64-row query / dO sub-tiles like the dK/dV role above,
// but S^T and dP^T are computed once: the staged dS^T tiles of two consecutive sub-blocks
// ([128 keys x 64 queries] each, adjacent in shared memory) also serve, read with the queries as
// the M dimension, as the A operand of dQ[128 queries x 64] = dS . K for that pair of sub-blocks.
// The pair's dQ [128 x 64] fp32 leaves tensor memory through a shared-memory staging tile and two
// bulk tensor add-reductions (one per 32-column half) into a [B, H, S, 64] accumulator: each query
// row receives one contribution per key tile, in no fixed order; a small kernel scales and converts
// the sums once all CTAs are done.  Five contractions instead of seven, one
// exponential pass instead of two, half the CTAs.
// smem: K, V [128 x 64] | Q, dO sub-tiles x NST3 | P^T x 2 | dS^T x 2 pair slots x 2 groups | dQ staging 2 x 16 KiB | lse / delta
// TMEM: S^T 2 x 64 | dP^T 2 x 64 | dV 64 | dK 64 | dQ 2 x 64
constexpr int NST3 = 4;
// warps: 0 TMA, 1 score products (S^T, dP^T), 2 updates (dV, dK, dQ), 3 idle (compute warp w must sit at
// w % 4 == its tensor-memory lane quarter), 4..19 the two compute groups
constexpr int NT3 = 128 + 2 * GROUP_THREADS;
__global__ void __launch_bounds__(NT3, 1)
attn_tc_bwd3_kernel(const __grid_constant__ CUtensorMap tm128, const __grid_constant__ CUtensorMap tm64,
                    const __grid_constant__ CUtensorMap tm_do64, const __grid_constant__ CUtensorMap tm_acc, const TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + TILE_BYTES;
  uint8_t* sQ = sV + TILE_BYTES;               // NST3 stages x 8 KiB
  uint8_t* sDO = sQ + NST3 * SUB_BYTES;        // NST3 stages x 8 KiB
  uint8_t* sP = sDO + NST3 * SUB_BYTES;        // [group] x 16 KiB
  uint8_t* sDS = sP + 2 * TILE_BYTES;          // [pair slot][group] x 16 KiB
  uint8_t* sDQ = sDS + 4 * TILE_BYTES;         // [column half] x 16 KiB: [128 queries x 32] fp32, 128-byte rows
  float* s_lse = reinterpret_cast<float*>(sDQ + 2 * TILE_BYTES);   // [2][64]
  float* s_delta = s_lse + 2 * SUB;                                // [2][64]
  Ctl* ctl = reinterpret_cast<Ctl*>(s_delta + 2 * SUB);
  uint64_t* kv_full = &ctl->bars[0];
  uint64_t* q_full = &ctl->bars[1];            // [NST3]
  uint64_t* q_empty = q_full + NST3;           // [NST3]
  uint64_t* s_full = q_empty + NST3;           // [2]
  uint64_t* s_empty = s_full + 2;              // [2]
  uint64_t* p_full = s_empty + 2;              // [2]  P^T and dS^T of a sub-block staged
  uint64_t* p_empty = p_full + 2;              // [2]  P^T buffer of a group read by its dV update
  uint64_t* ds_empty = p_empty + 2;            // [2]  both dS^T buffers of a pair slot read by dK and dQ
  uint64_t* dq_full = ds_empty + 2;            // [2]  a pair's dQ complete in tensor memory
  uint64_t* dq_empty = dq_full + 2;            // [2]  ... and drained
  uint64_t* acc_full = dq_empty + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int k0 = kb * TQ;
  const int row_base = batch * p.S;
  const int colq = head * HD, colk = p.hidden + head * HD, colv = 2 * p.hidden + head * HD;
  const int nq = (p.S + SUB - 1) / SUB;
  const int qstart = p.causal ? (k0 / SUB) : 0;
  // an even number of sub-blocks (they pair up for dQ); a padding sub-block lies past the
  // sequence end and is masked to zero
  const int nblk = (nq - qstart + 1) & ~1;
  const int npairs = nblk >> 1;

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    bb::mbar_init(kv_full, 1);
    for (int i = 0; i < NST3; ++i) { bb::mbar_init(&q_full[i], 1); bb::mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      bb::mbar_init(&s_full[i], 1); bb::mbar_init(&s_empty[i], GROUP_THREADS / 32);
      bb::mbar_init(&p_full[i], GROUP_THREADS / 32); bb::mbar_init(&p_empty[i], 1);
      bb::mbar_init(&ds_empty[i], 1);
      bb::mbar_init(&dq_full[i], 1); bb::mbar_init(&dq_empty[i], GROUP_THREADS / 32);
    }
    bb::mbar_init(acc_full, 1);
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tm128); bb::tma_prefetch_desc(&tm64); bb::tma_prefetch_desc(&tm_do64); bb::tma_prefetch_desc(&tm_acc);
  }
  if (warp == 1) { bb::tmem_alloc(&ctl->tmem_slot, 512); bb::tmem_relinquish(); }
  bb::tc_fence_before_sync();
  __syncthreads();
  bb::tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;
  // S^T[b] at tmem + 64 b, dP^T[b] at tmem + 128 + 64 b (b < 2)
  const uint32_t tDV = tmem + 256, tDK = tmem + 320, tDQ = tmem + 384;    // dQ[b] at tDQ + 64 b

  if (warp == 0) {
    if (lane == 0) {
      bb::mbar_arrive_expect_tx(kv_full, 2 * TILE_BYTES);
      bb::tma_load_2d(sK, &tm128, kv_full, colk, row_base + k0);
      bb::tma_load_2d(sV, &tm128, kv_full, colv, row_base + k0);
      for (int i = 0; i < nblk; ++i) {
        const int s = i % NST3;
        if (!bb::mbar_wait(&q_empty[s], ((i / NST3) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::mbar_arrive_expect_tx(&q_full[s], 2 * SUB_BYTES);
        bb::tma_load_2d(sQ + s * SUB_BYTES, &tm64, &q_full[s], colq, row_base + (qstart + i) * SUB);
        bb::tma_load_2d(sDO + s * SUB_BYTES, &tm_do64, &q_full[s], colq, row_base + (qstart + i) * SUB);
      }
    }
  } else if (warp == 1) {
    // score products: one thread issues S^T = K . Q^T and dP^T = V . dO^T for every sub-block, as soon as its
    // operands have landed and the group that owns the score buffer has read the previous contents
    const uint64_t dK0 = desc_k0(bb::smem_u32(sK)), dV0 = desc_k0(bb::smem_u32(sV));
    const uint64_t dQ0 = desc_k0(bb::smem_u32(sQ)), dDO0 = desc_k0(bb::smem_u32(sDO));   // stage 0; stage s: + s * SUB_BYTES / 16
    const uint32_t i_s = idesc(64, 0, 0);
    bool alive = bb::mbar_wait(kv_full, 0, &ctl->abort_flag, p.status);
    for (int i = 0; i < nblk && alive; ++i) {
      const int s = i % NST3, b = i & 1;
      if (!bb::mbar_wait(&q_full[s], (i / NST3) & 1, &ctl->abort_flag, p.status)) break;
      if (!bb::mbar_wait(&s_empty[b], ((i >> 1) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
      bb::tc_fence_after_sync();
      if (lane == 0) {
        const uint64_t dQ = dQ0 + (uint64_t)(s * (SUB_BYTES >> 4)), dDO = dDO0 + (uint64_t)(s * (SUB_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          bb::umma_f16(tmem + 64 * b, desc_kmajor(dK0, k), desc_kmajor(dQ, k), i_s, k > 0);
          bb::umma_f16(tmem + 128 + 64 * b, desc_kmajor(dV0, k), desc_kmajor(dDO, k), i_s, k > 0);
        }
        bb::umma_commit(&s_full[b]);
      }
      __syncwarp();
    }
  } else if (warp == 2) {
    // updates: a second issuing thread, so that the score products of the next sub-blocks never queue
    // behind a wait for staged operands (and the two instruction streams issue side by side)
    const uint64_t dQm0 = desc_mn0(bb::smem_u32(sQ)), dDOm0 = desc_mn0(bb::smem_u32(sDO));
    const uint64_t dP0 = desc_k0(bb::smem_u32(sP)), dDS0 = desc_k0(bb::smem_u32(sDS));
    // dS^T of a pair slot read with the queries as M: two 64-query blocks one tile apart, 8-key groups 1 KiB apart
    const uint64_t dDSm0 = bb::make_smem_desc_sw128(bb::smem_u32(sDS), TILE_BYTES, 1024);
    const uint64_t dKm0 = desc_mn0(bb::smem_u32(sK));
    const uint32_t i_acc = idesc(64, 0, 1), i_dq = idesc(64, 1, 1);
    bool alive = bb::mbar_wait(kv_full, 0, &ctl->abort_flag, p.status);
    for (int ii = 0; ii < nblk && alive; ++ii) {
      const int s2 = ii % NST3, g2 = ii & 1, pair = ii >> 1, ps = pair & 1;
      // (the sub-tiles landed long ago - the score products read them; the wait makes them visible to this thread)
      if (!bb::mbar_wait(&q_full[s2], (ii / NST3) & 1, &ctl->abort_flag, p.status)) break;
      if (!bb::mbar_wait(&p_full[g2], pair & 1, &ctl->abort_flag, p.status)) break;
      bb::tc_fence_after_sync();
      if (lane == 0) {
        const uint64_t dQ2 = dQm0 + (uint64_t)(s2 * (SUB_BYTES >> 4)), dDO2 = dDOm0 + (uint64_t)(s2 * (SUB_BYTES >> 4));
        const uint64_t dP = dP0 + (uint64_t)(g2 * (TILE_BYTES >> 4));
        const uint64_t dDS = dDS0 + (uint64_t)((ps * 2 + g2) * (TILE_BYTES >> 4));
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          bb::umma_f16(tDV, desc_kmajor(dP, k), desc_mnmajor64(dDO2, k), i_acc, (ii > 0 || k > 0));
          bb::umma_f16(tDK, desc_kmajor(dDS, k), desc_mnmajor64(dQ2, k), i_acc, (ii > 0 || k > 0));
        }
        bb::umma_commit(&p_empty[g2]);
        bb::umma_commit(&q_empty[s2]);
      }
      __syncwarp();
      if (g2 == 1) {
        // both halves of the pair are staged: dQ[pair] = dS . K over the tile's 128 keys
        if (!bb::mbar_wait(&dq_empty[pair & 1], ((pair >> 1) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint64_t dA = dDSm0 + (uint64_t)(ps * 2 * (TILE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < 8; ++k)
            bb::umma_f16(tDQ + 64 * (pair & 1), desc_mnmajor64(dA, k), desc_mnmajor64(dKm0, k), i_dq, k > 0);
          bb::umma_commit(&ds_empty[ps]);
          bb::umma_commit(&dq_full[pair & 1]);
          if (ii == nblk - 1) bb::umma_commit(acc_full);
        }
        __syncwarp();
      }
    }
  } else if (warp >= 4) {
    const int g = (warp - 4) >> 3;
    const int hf = ((warp - 4) >> 2) & 1;                  // which 32 of the sub-block's 64 query columns
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                   // key row inside the tile / query row inside a pair
    const int gt = threadIdx.x - 128 - GROUP_THREADS * g;  // thread index inside the group
    const int krow = k0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float* lse_g = p.lse + ((long long)batch * p.H + head) * p.S;
    const float* delta_g = p.delta + ((long long)batch * p.H + head) * p.S;
    const float sl = p.scale * LOG2E;
    uint8_t* myP = sP + g * TILE_BYTES;
    float* my_lse = s_lse + g * SUB;
    float* my_delta = s_delta + g * SUB;
    bool alive = true;
    int n = 0;
    int next_drain = 0;                                     // group 1 drains every pair
    const long long acc_row0 = ((long long)batch * p.H + head) * p.S;
    // one pair's dQ: tensor memory -> staging tile -> add-reduction into the accumulator rows of its 128
    // queries (rows past the sequence end carry exact zeros: their dS was masked)
    auto drain = [&](int pair) -> bool {
      const bool ok = bb::mbar_wait(&dq_full[pair & 1], (pair >> 1) & 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok)) return false;
      bb::tc_fence_after_sync();
      float v[32];
      ld32(tDQ + 64 * (pair & 1) + lane_addr + hf * 32, v);
      bb::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) bb::mbar_arrive(&dq_empty[pair & 1]);
      // the staging tile is free once the previous pair's reductions have read it
      if (gt == 0) bb::bulk_wait_group_read<0>();
      bb::named_bar_sync(3 + g, GROUP_THREADS);
      uint8_t* dst = sDQ + hf * TILE_BYTES + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<float4*>(dst + ((c ^ (row & 7)) << 4)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      bb::fence_proxy_async();
      bb::named_bar_sync(3 + g, GROUP_THREADS);
      if (gt == 0) {
        const int r0 = (int)(acc_row0 + (long long)(qstart + 2 * pair) * SUB);
        bb::tma_reduce_add_2d(&tm_acc, sDQ, 0, r0);
        bb::tma_reduce_add_2d(&tm_acc, sDQ + TILE_BYTES, 32, r0);
        bb::bulk_commit_group();
      }
      return true;
    };
    // per-column statistics are fetched one sub-block ahead so their latency is off the critical path
    float nx_lse = 0.f, nx_delta = 0.f;
    if (gt < SUB && g < nblk) {
      const int q = (qstart + g) * SUB + gt;
      if (q < p.S) { nx_lse = lse_g[q] * LOG2E; nx_delta = delta_g[q]; }
    }
    for (int i = g; i < nblk && alive; i += 2, ++n) {
      const int qc0 = (qstart + i) * SUB;
      const int ps = n & 1;                                  // sub-block i belongs to pair n
      // (the group's previous readers are past their last use once everybody is through this barrier)
      bb::named_bar_sync(1 + g, GROUP_THREADS);
      if (gt < SUB) { my_lse[gt] = nx_lse; my_delta[gt] = nx_delta; }
      bb::named_bar_sync(1 + g, GROUP_THREADS);
      if (gt < SUB && i + 2 < nblk) {
        const int q = (qstart + i + 2) * SUB + gt;
        nx_lse = (q < p.S) ? lse_g[q] * LOG2E : 0.f;
        nx_delta = (q < p.S) ? delta_g[q] : 0.f;
      }
      const uint32_t tS = tmem + 64 * g, tDP = tmem + 128 + 64 * g;
      const bool ok = bb::mbar_wait(&s_full[g], n & 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok)) { alive = false; break; }
      bb::tc_fence_after_sync();
      // (keys past the sequence end must not reach dQ: their rows of dK / dV are simply not stored)
      const bool need_mask = (qc0 + SUB > p.S) || (k0 + TQ > p.S) || (p.causal && k0 + TQ - 1 > qc0);
      uint32_t pkP[16], pkDS[16];                            // this thread's 32 P^T and dS^T values as bf16 pairs
      {
        float sv[32], dp[32];
        ld32x2(tS + lane_addr + hf * 32, tDP + lane_addr + hf * 32, sv, dp);
        // the scores are in registers: the buffer can take the sub-block after next while this one is worked on
        bb::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) bb::mbar_arrive(&s_empty[g]);
#pragma unroll
        for (int e4 = 0; e4 < 32; e4 += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(my_lse + hf * 32 + e4);
          const float4 d4 = *reinterpret_cast<const float4*>(my_delta + hf * 32 + e4);
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, ds[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int e = e4 + u;
            float pv = ex2(fmaf(sv[e], sl, -ls[u]));
            if (need_mask) {
              const int q = qc0 + hf * 32 + e;
              if (q >= p.S || krow >= p.S || (p.causal && krow > q)) pv = 0.f;
            }
            sv[e] = pv;
            dp[e] = pv * (dp[e] - ds[u]);
          }
        }
        pack32(sv, pkP);
        pack32(dp, pkDS);
      }
      // P^T's buffer is free once the dV update that read it retired; the pair slot's dS^T buffers once
      // the dK updates and the dQ product of the pair that used the slot before have
      const bool ok2 = bb::mbar_wait(&p_empty[g], (n & 1) ^ 1, &ctl->abort_flag, p.status) &&
                       bb::mbar_wait(&ds_empty[ps], ((n >> 1) & 1) ^ 1, &ctl->abort_flag, p.status);
      if (!bb::named_bar_all(3 + g, GROUP_THREADS, ok2)) { alive = false; break; }
      atom_store_half_row(myP, row, hf, pkP);
      atom_store_half_row(sDS + (ps * 2 + g) * TILE_BYTES, row, hf, pkDS);
      bb::fence_proxy_async();
      __syncwarp();
      if (lane == 0) bb::mbar_arrive(&p_full[g]);
      // group 1 drains the previous pair, whose second half it staged one iteration ago: certainly complete
      if (g == 1 && next_drain < n) {
        if (!drain(next_drain)) { alive = false; break; }
        ++next_drain;
      }
    }
    while (g == 1 && alive && next_drain < npairs) {
      if (!drain(next_drain)) { alive = false; break; }
      ++next_drain;
    }
    if (g == 1 && gt == 0) bb::bulk_wait_group<0>();       // the reductions read this CTA's shared memory
    const bool fin = alive && nblk > 0 && bb::mbar_wait(acc_full, 0, &ctl->abort_flag, p.status);
    if (bb::named_bar_all(3 + g, GROUP_THREADS, fin)) {
      bb::tc_fence_after_sync();
      float v[32];
      // the two groups split the final stores: group 0 writes dV, group 1 writes dK
      const uint32_t src = (g == 0) ? tDV : tDK;
      ld32(src + lane_addr + hf * 32, v);
      __nv_bfloat16* dst = (g == 0) ? p.dv : p.dk;
      if (krow < p.S) store_row32(dst + (long long)(row_base + krow) * p.stride_dqkv + colq + hf * 32, v, g == 0 ? 1.f : p.scale);
    }
  }
  bb::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) bb::tmem_dealloc(tmem, 512);
}

constexpr int BWD3_SMEM = 2 * TILE_BYTES + 2 * NST3 * SUB_BYTES + 2 * TILE_BYTES + 4 * TILE_BYTES + 2 * TILE_BYTES + 4 * SUB * (int)sizeof(float) +
                          (int)sizeof(Ctl) + 1024;

// dq (bf16, packed projection layout) = scale * accumulator; eight values per thread
__global__ void __launch_bounds__(256)
attn_tc_dq_convert_kernel(const TcParams p) {
  const int per_tok = p.H * 8;
  const long long total = (long long)p.B * p.S * per_tok;
  for (long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x; c < total; c += (long long)gridDim.x * blockDim.x) {
    const long long tok = c / per_tok;
    const int within = (int)(c % per_tok), head = within >> 3, part = within & 7;
    const float4* src = reinterpret_cast<const float4*>(p.dq_acc + (((tok / p.S) * p.H + head) * p.S + (tok % p.S)) * HD + part * 8);
    const float4 a = __ldcg(src), b = __ldcg(src + 1);
    uint4 o;
    o.x = bb::pack_bf16x2(a.x * p.scale, a.y * p.scale); o.y = bb::pack_bf16x2(a.z * p.scale, a.w * p.scale);
    o.z = bb::pack_bf16x2(b.x * p.scale, b.y * p.scale); o.w = bb::pack_bf16x2(b.z * p.scale, b.w * p.scale);
    *reinterpret_cast<uint4*>(p.dq + tok * p.stride_dqkv + head * HD + part * 8) = o;
  }
}

// ------------------------------------------------------------------ forward (two query tiles in ping-pong)
// A CTA owns 256 query rows of one (batch, head) as two 128-row tiles; compute group g (4 warps,
// one query row per thread) runs the online softmax of tile g.  Keys/values stream in 64-row
// sub-tiles that serve both query tiles.  Per sub-block jj and group g:
//   S_g(jj) = Q_g K_jj^T  ->  P_g = exp2(S_g * c - m_g)  ->  PV_g(jj) = P_g V_jj
// Scores are double-buffered in tensor memory and issued two sub-blocks ahead, so a group never
// waits for the tensor core between sub-blocks; P goes through shared memory (bf16, two buffers
// per group).  The output row accumulates in tensor memory over all sub-blocks (O_g += P_g V_jj);
// the exponent reference of a row only moves when the running maximum has grown by more than 2^8
// since it was set, and only then is the row's accumulator rescaled (tensor memory -> registers ->
// tensor memory, between two P V products): after the first few sub-blocks that is rare, and the
// per-sub-block work of a thread is the softmax alone.  P <= 2^8 and the row sums stay far inside
// fp32 / bf16 range; the final division by the row sum makes the choice of reference immaterial.
// smem: Q_0, Q_1 [128 x D] | K, V sub-tiles [64 x D] x NKV stages | P_g,b [128 x 64] x 4
// TMEM: S_g,b at 128 g + 64 b | O_g at 256 + 128 g (D columns)
// Head dimension D = 64 or 128.  A [rows x 128] operand lies in shared memory as two [rows x 64] atoms of
// 128-byte rows, one after the other (two TMA boxes): the score product walks its eight 16-column k-steps
// through both atoms; V as the B operand of P V (N = D, its columns) names the distance between the atoms in
// the descriptor's leading-dimension field.  The whole tensor memory is in use at D = 128 (2 x 2 score
// buffers of 64 columns, 2 outputs of 128), and the sub-tile ring is 3 deep instead of 6.
template <int D> struct Fwd2 {
  static constexpr int NA = D / 64;                            // 64-column atoms per row
  static constexpr int NKV = (D == 64) ? 6 : 3;                // sub-tile ring depth
  static constexpr int Q_BYTES = NA * TILE_BYTES;              // one query tile
  static constexpr int KV_BYTES = NA * SUB_BYTES;              // one key (or value) sub-tile
  static constexpr int SMEM = 2 * Q_BYTES + 2 * NKV * KV_BYTES + 4 * TILE_BYTES + (int)sizeof(Ctl) + 1024;
};
// warps: 0 TMA, 1 score products, 2 P V products (two issuing threads: the issue path of the small MMAs is the
// bound, and two instruction streams get about a third more through it than one), 3..10 the two softmax groups
constexpr int FWD2_THREADS = 96 + 256;

// one row (64 values) of a [128 x 64] bf16 atom
__device__ __forceinline__ void atom_store_row64(uint8_t* atom, int row, const float* a /*32*/, const float* b /*32*/) {
  uint8_t* base = atom + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float* v = (c < 4) ? a + 8 * c : b + 8 * (c - 4);
    uint4 q;
    q.x = bb::pack_bf16x2(v[0], v[1]); q.y = bb::pack_bf16x2(v[2], v[3]);
    q.z = bb::pack_bf16x2(v[4], v[5]); q.w = bb::pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(base + ((c ^ (row & 7)) << 4)) = q;
  }
}

template <int D>
__global__ void __launch_bounds__(FWD2_THREADS, 1)
attn_tc_fwd2_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_kv, const TcParams p) {
  using C = Fwd2<D>;
  constexpr int NA = C::NA, NKV = C::NKV, Q_BYTES = C::Q_BYTES, KV_BYTES = C::KV_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                          // 2 tiles
  uint8_t* sK = sQ + 2 * Q_BYTES;              // NKV sub-tiles
  uint8_t* sV = sK + NKV * KV_BYTES;           // NKV sub-tiles
  uint8_t* sP = sV + NKV * KV_BYTES;           // [group][buffer] x 16 KiB
  Ctl* ctl = reinterpret_cast<Ctl*>(sP + 4 * TILE_BYTES);
  uint64_t* q_full = &ctl->bars[0];
  uint64_t* kv_full = &ctl->bars[1];           // [NKV]
  uint64_t* kv_empty = &ctl->bars[1 + NKV];    // [NKV]
  uint64_t* s_full = &ctl->bars[1 + 2 * NKV];  // [group][buffer] scores ready
  uint64_t* p_full = s_full + 4;               // [group] probabilities in shared memory, scores read
  uint64_t* pv_full = p_full + 2;              // [group] P V product ready
  // [group][buffer] the group is done with the scores in this buffer.  Completes at the same moment as p_full, but
  // per buffer: its next phase needs the next score product into the buffer, which only the waiter issues, so
  // the waiter can never find it two phases on (p_full can be: the other issuing warp moves that one along)
  uint64_t* s_free = pv_full + 2;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cb = gridDim.x - 1 - blockIdx.x, head = blockIdx.y, batch = blockIdx.z;   // long CTAs first
  const int row_base = batch * p.S;
  const int colq = head * D, colk = p.hidden + head * D, colv = 2 * p.hidden + head * D;
  const int nsub = (p.S + SUB - 1) / SUB;
  // last key sub-block of each query tile (-1: the tile lies past the end of the sequence)
  const int qa = cb * 2 * TQ, qb = qa + TQ;
  const int last0 = (qa >= p.S) ? -1 : (p.causal ? min(nsub - 1, (qa + TQ - 1) / SUB) : nsub - 1);
  const int last1 = (qb >= p.S) ? -1 : (p.causal ? min(nsub - 1, (qb + TQ - 1) / SUB) : nsub - 1);
  const int jmax = max(last0, last1);
#define BB_LAST(g) ((g) ? last1 : last0)

  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    bb::mbar_init(q_full, 1);
    for (int i = 0; i < NKV; ++i) { bb::mbar_init(&kv_full[i], 1); bb::mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 4; ++i) { bb::mbar_init(&s_full[i], 1); bb::mbar_init(&s_free[i], 4); }
    for (int g = 0; g < 2; ++g) { bb::mbar_init(&p_full[g], 4); bb::mbar_init(&pv_full[g], 1); }
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tm_q); bb::tma_prefetch_desc(&tm_kv);
  }
  if (warp == 1) { bb::tmem_alloc(&ctl->tmem_slot, 512); bb::tmem_relinquish(); }
  bb::tc_fence_before_sync();
  __syncthreads();
  bb::tc_fence_after_sync();
  const uint32_t tmem = ctl->tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      bb::mbar_arrive_expect_tx(q_full, 2 * Q_BYTES);
#pragma unroll
      for (int a = 0; a < NA; ++a) {
        bb::tma_load_2d(sQ + a * TILE_BYTES, &tm_q, q_full, colq + 64 * a, row_base + qa);
        bb::tma_load_2d(sQ + Q_BYTES + a * TILE_BYTES, &tm_q, q_full, colq + 64 * a, row_base + qb);
      }
      for (int jj = 0; jj <= jmax; ++jj) {
        const int s = jj % NKV;
        if (!bb::mbar_wait(&kv_empty[s], ((jj / NKV) & 1) ^ 1, &ctl->abort_flag, p.status)) break;
        bb::mbar_arrive_expect_tx(&kv_full[s], 2 * KV_BYTES);
#pragma unroll
        for (int a = 0; a < NA; ++a) {
          bb::tma_load_2d(sK + s * KV_BYTES + a * SUB_BYTES, &tm_kv, &kv_full[s], colk + 64 * a, row_base + jj * SUB);
          bb::tma_load_2d(sV + s * KV_BYTES + a * SUB_BYTES, &tm_kv, &kv_full[s], colv + 64 * a, row_base + jj * SUB);
        }
      }
    }
  } else if (warp == 1) {
    const uint64_t dQ0 = desc_k0(bb::smem_u32(sQ));
    const uint64_t dK0 = desc_k0(bb::smem_u32(sK));   // stage 0; stage s: + s * KV_BYTES / 16
    const uint32_t i_s = idesc(64, 0, 0);
    bool alive = bb::mbar_wait(q_full, 0, &ctl->abort_flag, p.status);
    // scores of sub-block jj for group g into score buffer jj & 1
    auto issue_scores = [&](int g, int jj) {
      const uint64_t dK = dK0 + (uint64_t)((jj % NKV) * (KV_BYTES >> 4)), dQ = dQ0 + (uint64_t)(g * (Q_BYTES >> 4));
      const uint32_t tS = tmem + 128 * g + 64 * (jj & 1);
#pragma unroll
      for (int k = 0; k < D / 16; ++k)           // four k-steps per 64-column atom
        bb::umma_f16(tS, desc_kmajor(dQ + (uint64_t)((k >> 2) * (TILE_BYTES >> 4)), k & 3),
                     desc_kmajor(dK + (uint64_t)((k >> 2) * (SUB_BYTES >> 4)), k & 3), i_s, k > 0);
      bb::umma_commit(&s_full[2 * g + (jj & 1)]);
    };
    // prologue: the first two score products of each group
    for (int jj = 0; jj < 2 && jj <= jmax && alive; ++jj) {
      if (!bb::mbar_wait(&kv_full[jj % NKV], 0, &ctl->abort_flag, p.status)) { alive = false; break; }
      bb::tc_fence_after_sync();
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < 2; ++g) if (jj <= BB_LAST(g)) issue_scores(g, jj);
      }
      __syncwarp();
    }
    // steady state: the scores two sub-blocks ahead, as soon as the group has read the buffer they go to
    for (int jj = 0; jj + 2 <= jmax && alive; ++jj) {
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (jj + 2 > BB_LAST(g)) continue;
        // group g is done reading S_g(jj): its buffer is free
        if (!bb::mbar_wait(&s_free[2 * g + (jj & 1)], (jj >> 1) & 1, &ctl->abort_flag, p.status)) { alive = false; break; }
        if (!bb::mbar_wait(&kv_full[(jj + 2) % NKV], ((jj + 2) / NKV) & 1, &ctl->abort_flag, p.status)) { alive = false; break; }
        bb::tc_fence_after_sync();
        if (lane == 0) issue_scores(g, jj + 2);
        __syncwarp();
      }
    }
  } else if (warp == 2) {
    // V: [64 keys x D]; its atoms (64 columns each) lie SUB_BYTES apart, which is desc_mn0's leading-dimension field
    static_assert(SUB_BYTES == 8192, "desc_mn0 names the distance between the 64-column atoms of V");
    const uint64_t dP0 = desc_k0(bb::smem_u32(sP)), dVm0 = desc_mn0(bb::smem_u32(sV));   // stage 0; stage s: + s * KV_BYTES / 16
    const uint32_t i_pv = idesc(D, 0, 1);
    bool alive = true;
    for (int jj = 0; jj <= jmax && alive; ++jj) {
      const int s = jj % NKV;
      const uint64_t dV = dVm0 + (uint64_t)(s * (KV_BYTES >> 4));
      // (V_jj landed before the scores of this sub-block were issued; the wait makes it visible to this thread)
      if (!bb::mbar_wait(&kv_full[s], (jj / NKV) & 1, &ctl->abort_flag, p.status)) break;
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        if (jj > BB_LAST(g)) continue;
        if (!bb::mbar_wait(&p_full[g], jj & 1, &ctl->abort_flag, p.status)) { alive = false; break; }
        bb::tc_fence_after_sync();
        if (lane == 0) {
          const uint32_t tO = tmem + 256 + 128 * g;
          const uint64_t dPg = dP0 + (uint64_t)((2 * g + (jj & 1)) * (TILE_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < 4; ++k) bb::umma_f16(tO, desc_kmajor(dPg, k), desc_mnmajor64(dV, k), i_pv, (jj > 0 || k > 0));
          bb::umma_commit(&pv_full[g]);
        }
        __syncwarp();
      }
      // K_jj, V_jj: the score products that read K_jj retired before P(jj) existed, the P V products are issued
      if (alive && lane == 0) bb::umma_commit(&kv_empty[s]);
      __syncwarp();
    }
  } else if (warp >= 3) {
    const int g = (warp - 3) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int q0 = g ? qb : qa;
    const int qrow = q0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + 128 * g + lane_addr;
    const uint32_t tO = tmem + 256 + 128 * g + lane_addr;
    const float sl = p.scale * LOG2E;
    const int lastj = BB_LAST(g);
    constexpr float REF_SLACK = 8.f;                         // log2 units the maximum may grow past the reference
    float m_ref = -INFINITY, l_i = 0.f;                     // exponent reference of this row, row sum relative to it
    bool alive = true;
    for (int jj = 0; jj <= lastj; ++jj) {
      const int b = jj & 1;
      const bool got = bb::mbar_wait(&s_full[2 * g + b], (jj >> 1) & 1, &ctl->abort_flag, p.status);
      if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const int c0 = jj * SUB;
      // only sub-blocks that touch the causal diagonal or the end of the sequence need masks
      const bool need_mask = (c0 + SUB > p.S) || (p.causal && c0 + SUB - 1 > q0);
      float sa[32], sb[32];                                  // the row's 64 scores stay in registers
      ld32x2(tS + 64 * b, tS + 64 * b + 32, sa, sb);
      float mx = -INFINITY;
      if (!need_mask) {
#pragma unroll
        for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(sa[i], sb[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int ca = c0 + i, cc = ca + 32;
          if (ca >= p.S || (p.causal && ca > qrow)) sa[i] = -INFINITY;
          if (cc >= p.S || (p.causal && cc > qrow)) sb[i] = -INFINITY;
          mx = fmaxf(mx, fmaxf(sa[i], sb[i]));
        }
      }
      mx *= sl;                                              // scale > 0: the maximum commutes with it
      // move the reference only when the maximum outgrew it by more than the slack
      float alpha = 1.f;
      if (mx > m_ref + REF_SLACK || (m_ref == -INFINITY && mx > -INFINITY)) {
        alpha = ex2(m_ref - mx);                             // 0 for the first finite maximum
        m_ref = mx;
        l_i *= alpha;
      }
      const float nm = (m_ref == -INFINITY) ? 0.f : -m_ref;
      float rs = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {                         // exp2(-inf) = 0 covers the masked entries
        sa[i] = ex2(fmaf(sa[i], sl, nm)); sb[i] = ex2(fmaf(sb[i], sl, nm));
        rs += sa[i] + sb[i];
      }
      l_i += rs;
      if (jj > 0) {
        // the previous product has retired: its P buffer is free and the accumulator is at rest
        const bool ok = bb::mbar_wait(&pv_full[g], (jj - 1) & 1, &ctl->abort_flag, p.status);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
          // some row of this warp moved its reference: rescale the warp's accumulator rows in place
          bb::tc_fence_after_sync();
#pragma unroll
          for (int h = 0; h < D / 32; ++h) {
            uint32_t r[32];
            bb::tmem_ld_32x32b_x32(tO + 32 * h, r);
            bb::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            bb::tmem_st_32x32b_x32(tO + 32 * h, r);
          }
          bb::tmem_st_wait();
        }
      }
      atom_store_row64(sP + (2 * g + b) * TILE_BYTES, row, sa, sb);
      bb::tc_fence_before_sync();
      bb::fence_proxy_async();
      __syncwarp();
      if (lane == 0) { bb::mbar_arrive(&p_full[g]); bb::mbar_arrive(&s_free[2 * g + b]); }
    }
    if (lastj >= 0) {
      const bool fin = alive && bb::mbar_wait(&pv_full[g], lastj & 1, &ctl->abort_flag, p.status);
      if (__all_sync(0xffffffffu, fin)) {
        bb::tc_fence_after_sync();
        const float inv = l_i > 0.f ? 1.f / l_i : 0.f;
#pragma unroll
        for (int a = 0; a < NA; ++a) {
          float o[64];
          ld32x2(tO + 64 * a, tO + 64 * a + 32, o, o + 32);
          if (qrow < p.S) store_row64(p.out + (long long)(row_base + qrow) * p.stride_o + colq + 64 * a, o, inv);
        }
        if (qrow < p.S) {
          p.lse[((long long)batch * p.H + head) * p.S + qrow] = (l_i > 0.f) ? (m_ref + log2f(l_i)) / LOG2E : -INFINITY;
        }
      }
    }
  }
  bb::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) bb::tmem_dealloc(tmem, 512);
}
#undef BB_LAST


template <typename K> int set_smem(K kernel, int bytes) {
  BB_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  return BB_OK;
}

}  // namespace

// Entry points used by attention.cu's dispatch: forward for head dimensions 64 and 128, backward for 64.
namespace {
template <int D>
int launch_fwd2(const void* qkv_q, void* out, float* lse, int B, int H, int S, long long stride_qkv, long long stride_o,
                int causal, float scale, cudaStream_t stream) {
  CUtensorMap tm_q, tm_kv;
  const long long T = (long long)B * S;
  // the packed projection [T, 3*H*D]: q, k, v blocks of H*D columns each; boxes of 64 columns (one
  // 128-byte swizzle atom), 128 rows for the query tiles, 64 rows for the streamed key/value sub-tiles
  if (int rc = bbhost::encode_2d(&tm_q, qkv_q, T, 3LL * H * D, stride_qkv, 64, TQ)) return rc;
  if (int rc = bbhost::encode_2d(&tm_kv, qkv_q, T, 3LL * H * D, stride_qkv, 64, SUB)) return rc;
  TcParams p = {};
  p.out = (__nv_bfloat16*)out; p.lse = lse; p.stride_o = stride_o; p.B = B; p.H = H; p.S = S; p.hidden = H * D;
  p.causal = causal; p.scale = scale; p.status = bb_device_status_word();
  BB_ONCE_PER_DEVICE({ if (int rc = set_smem(attn_tc_fwd2_kernel<D>, Fwd2<D>::SMEM)) return rc; });
  dim3 grid((S + 2 * TQ - 1) / (2 * TQ), H, B);
  attn_tc_fwd2_kernel<D><<<grid, FWD2_THREADS, Fwd2<D>::SMEM, stream>>>(tm_q, tm_kv, p);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
}  // namespace

int bb_attention_tc_fwd(const void* qkv_q, void* out, float* lse, int B, int H, int S, int D, long long stride_qkv,
                        long long stride_o, int causal, float scale, cudaStream_t stream) {
  if (int rc = bbhost::bind_context()) return rc;
  if (D == 64) return launch_fwd2<64>(qkv_q, out, lse, B, H, S, stride_qkv, stride_o, causal, scale, stream);
  if (D == 128) return launch_fwd2<128>(qkv_q, out, lse, B, H, S, stride_qkv, stride_o, causal, scale, stream);
  return BB_ERR_UNSUPPORTED;
}

int bb_attention_tc_bwd(const void* qkv_q, const void* out, const void* d_out, const float* lse, void* dq, void* dk, void* dv,
                        float* delta, float* dq_acc, int B, int H, int S, long long stride_qkv, long long stride_o,
                        long long stride_dqkv, int causal, float scale, cudaStream_t stream) {
  if (int rc = bbhost::bind_context()) return rc;
  CUtensorMap tm_qkv, tm_do;
  const long long T = (long long)B * S;
  if (int rc = bbhost::encode_2d(&tm_qkv, qkv_q, T, 3LL * H * HD, stride_qkv, HD, TQ)) return rc;
  if (int rc = bbhost::encode_2d(&tm_do, d_out, T, (long long)H * HD, stride_o, HD, TQ)) return rc;
  TcParams p = {};
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.lse = const_cast<float*>(lse); p.delta = delta; p.stride_o = stride_o; p.stride_dqkv = stride_dqkv;
  p.B = B; p.H = H; p.S = S; p.hidden = H * HD; p.causal = causal; p.scale = scale; p.status = bb_device_status_word();
  CUtensorMap tm_qkv64, tm_do64;
  if (int rc = bbhost::encode_2d(&tm_qkv64, qkv_q, T, 3LL * H * HD, stride_qkv, HD, SUB)) return rc;
  if (int rc = bbhost::encode_2d(&tm_do64, d_out, T, (long long)H * HD, stride_o, HD, SUB)) return rc;
  // BB_ATTENTION_BWD=split in the environment selects the two-role kernel (dK/dV and dQ computed by
  // different CTAs, every sum in a fixed order); the default is the fused kernel
  static const bool split = [] { const char* e = getenv("BB_ATTENTION_BWD"); return e && e[0] == 's'; }();
  const long long chunks = T * H * 8;
  long long dgrid = (chunks + 511) / 512, cap = (long long)bb_num_sms() * 8;
  if (split) {
    BB_ONCE_PER_DEVICE({ if (int rc = set_smem(attn_tc_bwd2_kernel, BWD2_SMEM)) return rc; });
    attn_tc_delta_kernel<<<(int)(dgrid < cap ? dgrid : cap), 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, p);
    dim3 grid(2 * ((S + TQ - 1) / TQ), H, B);
    attn_tc_bwd2_kernel<<<grid, NT2, BWD2_SMEM, stream>>>(tm_qkv, tm_qkv64, tm_do, tm_do64, p);
    BB_CUDA_CHECK(cudaGetLastError());
    return BB_OK;
  }
  p.dq_acc = dq_acc;
  BB_ONCE_PER_DEVICE({ if (int rc = set_smem(attn_tc_bwd3_kernel, BWD3_SMEM)) return rc; });
  attn_tc_delta_kernel<<<(int)(dgrid < cap ? dgrid : cap), 256, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)d_out, p);
  dim3 grid((S + TQ - 1) / TQ, H, B);
  // the accumulator as [B * H * S rows, 64] fp32; a reduction moves [128 rows x 32 columns]
  CUtensorMap tm_acc;
  if (int rc = bbhost::encode_2d(&tm_acc, dq_acc, (long long)B * H * S, HD, HD, 32, TQ, 1)) return rc;
  attn_tc_bwd3_kernel<<<grid, NT3, BWD3_SMEM, stream>>>(tm_qkv, tm_qkv64, tm_do64, tm_acc, p);
  long long cgrid = (chunks + 255) / 256;
  attn_tc_dq_convert_kernel<<<(int)(cgrid < cap ? cgrid : cap), 256, 0, stream>>>(p);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
