// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = op(A)[M,K] * op(B)[N,K]^T with a
// fused epilogue.  One persistent CTA per SM; warp 0 feeds shared memory with TMA
// (128-byte swizzle, no cluster multicast), warp 1 issues tcgen05.mma into two TMEM
// accumulators, warps 2-9 drain TMEM (tcgen05.ld) and run the epilogue (coalesced global
// stores from warp-private staging slabs) while the next tile's main loop is already running.
//
// Work units are handed out dynamically: the first unit of a CTA is its own index, every further
// one comes from a per-launch ticket counter in global memory (one atomicAdd per unit, issued a
// whole unit ahead of its use), and the producer thread passes it to the MMA and epilogue warps
// (and to the second CTA of a pair) through a four-entry ring in shared memory.  A CTA that
// starts late - because a kernel of another stream still held its SM - therefore takes fewer
// units instead of stretching the launch by its fixed share.
//
// Large problems run as CTA pairs (cta_group::2, clusters of two): a pair owns a 256 x 256
// tile, each CTA loads its own 128 rows of A and only HALF of the B tile, rank 0 issues one
// 256-row MMA for both and each CTA drains its own 128 accumulator rows.  Per CTA that is a
// third less operand traffic from L2 and a third less shared memory per k-block than the
// single-CTA 128 x 256 tile, so six stages fit instead of four - the single-CTA kernel is
// bound by operand bytes in flight, not by the tensor pipe.
//
// Operand storage (all row-major, bf16):
//   a_mn = 0 : A is [M, K] (K contiguous)     a_mn = 1 : A is stored [K, M] (M contiguous)
//   b_mn = 0 : B is [N, K] (K contiguous)     b_mn = 1 : B is stored [K, N] (N contiguous)
// which covers a linear layer's forward (0,0), input gradient (0,1) and weight gradient
// (1,1) without a transpose pass.
#include "common.cuh"
#include "bamboo_b200.h"
#include "tma_host.cuh"
#include <atomic>
#include <mutex>
#include <stdlib.h>

namespace {

constexpr int BM = 128;
constexpr int BK = 64;        // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
// threads: TMA warp, MMA warp and EW epilogue warps per TMEM lane quarter (EW = 2: 320, EW = 4: 576)
constexpr int num_threads(int ew) { return 64 + 128 * ew; }
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
// Epilogue staging: one 4 KiB slab (32 rows x 128 bytes = 64 bf16 or 32 fp32 columns) per
// epilogue warp; shared memory is better spent on main-loop stages.
constexpr int SLAB_BYTES = 32 * 128;
constexpr int NUM_SLABS = 8;
constexpr int SCHED_RING = 4;  // work units announced ahead of their consumption (power of two)

template <int BN, bool PAIR> struct Cfg {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;      // B rows (output columns) this CTA loads
  static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int STAGES = (B_ROWS == 256) ? 4 : 6;
  static constexpr int TILE_M = PAIR ? 2 * BM : BM;      // rows of a work unit (both CTAs of a pair)
  static constexpr int TMEM_COLS = 2 * BN;  // two accumulators
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + NUM_SLABS * SLAB_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
};

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;
  int epi;
  int ksplit, kb_per_split;   // split-K work units (fp32 add-reduction epilogue only)
  int n_fast;                 // tile order: consecutive work units walk along N (else along M)
  int dynamic;                // 1: work units after a CTA's first come from the ticket counter
  unsigned int* ticket;       // this launch's ticket counter (global memory)
  unsigned int ticket_base;   // its value before this launch's first ticket
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
__device__ __forceinline__ void panel_store_row_f32(uint8_t* panel, int row, const float* v /*32*/) {
  uint8_t* base = panel + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<float4*>(base + ((c ^ (row & 7)) << 4)) = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
}

// ---- warp-private staging slab: 32 rows x 128 bytes, 16-byte chunks XOR-swizzled by the row.
// Row side: lane == row (panel_store_row_* / panel_load_row_bf16 with row = lane).
// Coalesced side: lane -> (row 4*i + lane/8, chunk lane%8), i = 0..7: one instruction moves four
// complete 128-byte row segments.
__device__ __forceinline__ uint32_t slab_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ void slab_put(uint8_t* slab, int lane, const uint4* ax) {
#pragma unroll
  for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(slab + slab_off(4 * i + (lane >> 3), lane & 7)) = ax[i];
}
// rows r0.., columns nb.. of a bf16 matrix -> ax (zero outside the matrix)
__device__ __forceinline__ void slab_fetch_bf16(const __nv_bfloat16* src, long long ld, int r0, int nb, int M, int N, int lane, uint4* ax) {
  const int c = nb + (lane & 7) * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = r0 + 4 * i + (lane >> 3);
    uint4 q = make_uint4(0, 0, 0, 0);
    if (r < M) {
      const __nv_bfloat16* g = src + (long long)r * ld + c;
      if (c + 8 <= N) {
        q = __ldg(reinterpret_cast<const uint4*>(g));
      } else {
        unsigned short e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = (c + k < N) ? __bfloat16_as_ushort(g[k]) : (unsigned short)0;
        q.x = e[0] | ((uint32_t)e[1] << 16); q.y = e[2] | ((uint32_t)e[3] << 16);
        q.z = e[4] | ((uint32_t)e[5] << 16); q.w = e[6] | ((uint32_t)e[7] << 16);
      }
    }
    ax[i] = q;
  }
}
__device__ __forceinline__ void slab_flush_bf16(const uint8_t* slab, __nv_bfloat16* dst, long long ld, int r0, int nb, int M, int N, int lane) {
  const int c = nb + (lane & 7) * 8;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = 4 * i + (lane >> 3);
    const int r = r0 + rl;
    const uint4 q = *reinterpret_cast<const uint4*>(slab + slab_off(rl, lane & 7));
    if (r < M) {
      __nv_bfloat16* g = dst + (long long)r * ld + c;
      if (c + 8 <= N) {
        *reinterpret_cast<uint4*>(g) = q;
      } else {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) if (c + k < N) g[k] = __ushort_as_bfloat16((unsigned short)(w[k >> 1] >> (16 * (k & 1))));
      }
    }
  }
}
template <bool ACCUM>
__device__ __forceinline__ void slab_flush_f32(const uint8_t* slab, float* dst, long long ld, int r0, int nb, int M, int N, int lane) {
  const int c = nb + (lane & 7) * 4;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = 4 * i + (lane >> 3);
    const int r = r0 + rl;
    const float4 q = *reinterpret_cast<const float4*>(slab + slab_off(rl, lane & 7));
    if (r < M) {
      float* g = dst + (long long)r * ld + c;
      if (c + 4 <= N) {
        if (ACCUM) asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(g), "f"(q.x), "f"(q.y), "f"(q.z), "f"(q.w) : "memory");
        else *reinterpret_cast<float4*>(g) = q;
      } else {
        const float w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (c + k < N) { if (ACCUM) atomicAdd(g + k, w[k]); else g[k] = w[k]; }
        }
      }
    }
  }
}

// ---- narrow variant (four epilogue warps per lane quarter): 32 rows x 64 bytes = 32 bf16
// columns per pass, 2 KiB per warp.  Chunk c of row r sits at c ^ ((r >> 1) & 3): eight
// consecutive rows cover all 32 banks once, on the row side (lane == row) and on the coalesced
// side (lane -> row 8*i + lane/4, chunk lane%4, i = 0..3).
__device__ __forceinline__ uint32_t slab64_off(int row, int chunk) { return row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4); }

__device__ __forceinline__ void slab64_store_row(uint8_t* slab, int row, const float* v /*32*/) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint4 q;
    q.x = bb::pack_bf16x2(v[8 * c + 0], v[8 * c + 1]); q.y = bb::pack_bf16x2(v[8 * c + 2], v[8 * c + 3]);
    q.z = bb::pack_bf16x2(v[8 * c + 4], v[8 * c + 5]); q.w = bb::pack_bf16x2(v[8 * c + 6], v[8 * c + 7]);
    *reinterpret_cast<uint4*>(slab + slab64_off(row, c)) = q;
  }
}
// rows r0.., columns nb..nb+31 of a bf16 matrix -> slab (zero outside the matrix), coalesced
__device__ __forceinline__ void slab64_fetch(uint8_t* slab, const __nv_bfloat16* src, long long ld, int r0, int nb, int M, int N, int lane) {
  const int c = nb + (lane & 3) * 8;
  uint4 q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 8 * i + (lane >> 2);
    q[i] = make_uint4(0, 0, 0, 0);
    if (r < M) {
      const __nv_bfloat16* g = src + (long long)r * ld + c;
      if (c + 8 <= N) {
        q[i] = __ldg(reinterpret_cast<const uint4*>(g));
      } else {
        unsigned short e[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) e[k] = (c + k < N) ? __bfloat16_as_ushort(g[k]) : (unsigned short)0;
        q[i].x = e[0] | ((uint32_t)e[1] << 16); q[i].y = e[2] | ((uint32_t)e[3] << 16);
        q[i].z = e[4] | ((uint32_t)e[5] << 16); q[i].w = e[6] | ((uint32_t)e[7] << 16);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(slab + slab64_off(8 * i + (lane >> 2), lane & 3)) = q[i];
}
__device__ __forceinline__ void slab64_flush(const uint8_t* slab, __nv_bfloat16* dst, long long ld, int r0, int nb, int M, int N, int lane) {
  const int c = nb + (lane & 3) * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rl = 8 * i + (lane >> 2);
    const int r = r0 + rl;
    const uint4 q = *reinterpret_cast<const uint4*>(slab + slab64_off(rl, lane & 3));
    if (r < M) {
      __nv_bfloat16* g = dst + (long long)r * ld + c;
      if (c + 8 <= N) {
        *reinterpret_cast<uint4*>(g) = q;
      } else {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) if (c + k < N) g[k] = __ushort_as_bfloat16((unsigned short)(w[k >> 1] >> (16 * (k & 1))));
      }
    }
  }
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
    // fully unrolled with predicates: a dynamically indexed v[] would live in local memory
#pragma unroll
    for (int i = 0; i < W; ++i) if (n0 + i < p.N) v[i] += __bfloat162float(b[i]);
  }
}

template <int BN, bool PAIR, int EW>
__global__ void __launch_bounds__(num_threads(EW), 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const GemmParams p) {
  using C = Cfg<BN, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle atoms need 1024-byte aligned stage buffers
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + C::STAGES * A_STAGE_BYTES;
  uint8_t* panels = smem + C::STAGES * C::STAGE_BYTES;   // NUM_SLABS x 4 KiB epilogue staging
  uint64_t* bars = reinterpret_cast<uint64_t*>(panels + NUM_SLABS * SLAB_BYTES);
  uint64_t* full_bar = bars;                      // [STAGES]
  uint64_t* empty_bar = bars + C::STAGES;         // [STAGES]
  uint64_t* tmem_full = bars + 2 * C::STAGES;     // [2]
  uint64_t* tmem_empty = bars + 2 * C::STAGES + 2;  // [2]
  uint64_t* sched_full = bars + 2 * C::STAGES + 4;  // [SCHED_RING]
  uint64_t* sched_empty = sched_full + SCHED_RING;  // [SCHED_RING] (pairs: rank 0's are used by both CTAs)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sched_empty + SCHED_RING);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* sched_tile = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [SCHED_RING]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // work units go to CTAs (pairs: to clusters; both CTAs of a pair walk the same units)
  const uint32_t rank = PAIR ? bb::cluster_ctarank() : 0u;
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int num_m = (p.M + C::TILE_M - 1) / C::TILE_M;
  const int num_n = (p.N + BN - 1) / BN;
  const int num_mn = num_m * num_n;
  const int num_tiles = num_mn * p.ksplit;        // work units: (m, n, k-split)
  const int total_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::STAGES; ++s) { bb::mbar_init(&full_bar[s], 1); bb::mbar_init(&empty_bar[s], 1); }
    // accumulator hand-back: one arrival per epilogue warp (of both CTAs for a pair, on rank 0's barrier)
    for (int a = 0; a < 2; ++a) { bb::mbar_init(&tmem_full[a], 1); bb::mbar_init(&tmem_empty[a], (PAIR ? 2 : 1) * 4 * EW); }
    // work-unit ring: one announcement per entry; read by the MMA warp and the epilogue warps of
    // this CTA and, for a pair, by the producer and the epilogue warps of the second CTA
    for (int r = 0; r < SCHED_RING; ++r) { bb::mbar_init(&sched_full[r], 1); bb::mbar_init(&sched_empty[r], (PAIR ? 2 : 1) * (1 + 4 * EW)); }
    bb::fence_barrier_init();
    bb::tma_prefetch_desc(&tmA);
    bb::tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    if (PAIR) { bb::tmem_alloc_pair(tmem_slot, C::TMEM_COLS); bb::tmem_relinquish_pair(); }
    else { bb::tmem_alloc(tmem_slot, C::TMEM_COLS); bb::tmem_relinquish(); }
  }
  bb::tc_fence_before_sync();
  if (PAIR) bb::cluster_sync();     // the peer's barriers are initialised before anything signals them
  else __syncthreads();
  bb::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  // Next work unit of this CTA as announced by the scheduling thread (-1: no more).  Called by a
  // whole warp (`warp_wide`) or by a single thread; the entry is handed back once it has been read.
  auto next_unit = [&](uint32_t it, int& tile, bool warp_wide) -> bool {
    const int r = (int)(it & (SCHED_RING - 1));
    const uint32_t ph = (it / SCHED_RING) & 1u;
    const bool got = PAIR ? bb::mbar_wait_cluster(&sched_full[r], ph, abort_flag, p.status)
                          : bb::mbar_wait(&sched_full[r], ph, abort_flag, p.status);
    if (warp_wide) { if (!__all_sync(0xffffffffu, got)) return false; }
    else if (!got) return false;
    tile = sched_tile[r];
    if (warp_wide) __syncwarp();
    if (!warp_wide || lane == 0) {
      if (PAIR) bb::mbar_arrive_cluster(bb::mapa_shared(bb::smem_u32(&sched_empty[r]), 0));
      else bb::mbar_arrive(&sched_empty[r]);
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------ TMA producer
    if (lane == 0) {
      int s = 0; uint32_t phase = 0;
      bool alive = true;
      // operand loads of one work unit
      auto load_unit = [&](int tile) {
        const int mn = tile % num_mn, ks = tile / num_mn;
        const int mi = p.n_fast ? mn / num_n : mn % num_m, ni = p.n_fast ? mn % num_n : mn / num_m;
        const int m0 = mi * C::TILE_M + (int)rank * BM;                    // this CTA's A rows
        const int n0 = ni * BN + (int)rank * C::B_ROWS;                    // this CTA's share of B (pairs: half)
        const int kb0 = ks * p.kb_per_split, kb1 = min(total_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!bb::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag, p.status)) { alive = false; break; }
          uint8_t* a = sA + s * A_STAGE_BYTES;
          uint8_t* b = sB + s * C::B_STAGE_BYTES;
          const int k0 = kb * BK;
          if constexpr (PAIR) {
            // both CTAs' copies complete on rank 0's barrier, where the MMA issuer waits
            if (rank == 0) bb::mbar_arrive_expect_tx(&full_bar[s], 2 * C::STAGE_BYTES);
            const uint32_t fb = bb::mapa_shared(bb::smem_u32(&full_bar[s]), 0);
            if (!p.a_mn) {
              bb::tma_load_2d_pair(a, &tmA, fb, k0, m0);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) bb::tma_load_2d_pair(a + j * 8192, &tmA, fb, m0 + 64 * j, k0);
            }
            if (!p.b_mn) {
              bb::tma_load_2d_pair(b, &tmB, fb, k0, n0);
            } else {
#pragma unroll
              for (int j = 0; j < C::B_ROWS / 64; ++j) bb::tma_load_2d_pair(b + j * 8192, &tmB, fb, n0 + 64 * j, k0);
            }
          } else {
            bb::mbar_arrive_expect_tx(&full_bar[s], C::STAGE_BYTES);
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
          }
          if (++s == C::STAGES) { s = 0; phase ^= 1; }
        }
      };
      if (rank == 0) {
        // ---- scheduling thread: announces every work unit of this CTA (pair) to its consumers
        auto announce = [&](uint32_t it, int tile) -> bool {
          const int r = (int)(it & (SCHED_RING - 1));
          const uint32_t ph = (it / SCHED_RING) & 1u;
          const bool free_ = PAIR ? bb::mbar_wait_cluster(&sched_empty[r], ph ^ 1, abort_flag, p.status)
                                  : bb::mbar_wait(&sched_empty[r], ph ^ 1, abort_flag, p.status);
          if (!free_) return false;
          sched_tile[r] = tile;
          if (PAIR) {
            bb::st_shared_cluster_u32(bb::mapa_shared(bb::smem_u32(const_cast<int*>(&sched_tile[r])), 1), (uint32_t)tile);
            bb::mbar_arrive_cluster(bb::mapa_shared(bb::smem_u32(&sched_full[r]), 1));
          }
          bb::mbar_arrive(&sched_full[r]);
          return true;
        };
        // ticket t of this launch stands for work unit num_workers + t (units below num_workers are
        // the CTAs' first ones); every scheduling thread draws until its first ticket past the
        // end, so a launch consumes exactly num_tiles tickets - the host relies on that count
        auto draw = [&]() -> int { return num_workers + (int)(atomicAdd(p.ticket, 1u) - p.ticket_base); };
        uint32_t it = 0;
        int cur = worker, nxt = worker;
        while (cur < num_tiles) {
          nxt = p.dynamic ? draw() : cur + num_workers;     // in flight while this unit's loads are issued
          if (!announce(it++, cur)) { alive = false; break; }
          load_unit(cur);
          if (!alive) break;
          cur = nxt;
        }
        if (alive) { if (!announce(it++, -1)) alive = false; }
        else if (p.dynamic) { while (nxt < num_tiles) nxt = draw(); }
      } else {
        // second CTA of a pair: follows rank 0's announcements
        for (uint32_t it = 0; alive; ++it) {
          int tile;
          if (!next_unit(it, tile, false)) { alive = false; break; }
          if (tile < 0) break;
          load_unit(tile);
        }
      }
      if constexpr (PAIR) {
        // rank 0's MMA commits arrive on this CTA's barriers too: wait until the last one of every
        // stage has landed, so that none is still on its way when the CTA leaves
        for (int i = 0; i < C::STAGES && alive; ++i) {
          if (!bb::mbar_wait(&empty_bar[s], phase ^ 1, abort_flag, p.status)) alive = false;
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
                           ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(C::TILE_M >> 4) << 24);
    // K-major: 8-row groups 1024 B apart (LBO unused); MN-major: 64-wide column groups are
    // separate 8 KiB TMA boxes (LBO), 8 k-rows are 1024 B (SBO).
    const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
    const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;
    int s = 0; uint32_t phase = 0;
    int acc = 0; uint32_t acc_phase = 0;
    bool alive = true;
    // pairs: rank 0 issues for both CTAs; the other CTA's MMA warp only allocates and frees TMEM
    for (uint32_t it = 0; alive && rank == 0; ++it) {
      int tile;
      if (!next_unit(it, tile, true)) { alive = false; break; }
      if (tile < 0) break;
      if (!bb::mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
      const int ks = tile / num_mn;
      const int num_kb = min(total_kb, (ks + 1) * p.kb_per_split) - ks * p.kb_per_split;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!bb::mbar_wait(&full_bar[s], phase, abort_flag, p.status)) { alive = false; break; }
        bb::tc_fence_after_sync();
        if (lane == 0) {
          // one descriptor per stage; a k-step only adds to its address field (16-byte units)
          const uint64_t ad0 = bb::make_smem_desc_sw128(bb::smem_u32(sA + s * A_STAGE_BYTES), a_lbo, 1024u);
          const uint64_t bd0 = bb::make_smem_desc_sw128(bb::smem_u32(sB + s * C::B_STAGE_BYTES), b_lbo, 1024u);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = ad0 + (uint64_t)(k * (a_kstep >> 4));
            const uint64_t bd = bd0 + (uint64_t)(k * (b_kstep >> 4));
            if (PAIR) bb::umma_f16_pair(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else bb::umma_f16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          if (PAIR) {
            bb::umma_commit_pair(&empty_bar[s], 3);            // frees the stage in both CTAs
            if (kb == num_kb - 1) bb::umma_commit_pair(&tmem_full[acc], 3);
          } else {
            bb::umma_commit(&empty_bar[s]);
            if (kb == num_kb - 1) bb::umma_commit(&tmem_full[acc]);
          }
        }
        __syncwarp();
        if (++s == C::STAGES) { s = 0; phase ^= 1; }
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------ epilogue: 8 independent warps
    // A warp owns one TMEM lane quarter (32 rows of the tile); the two warps of a quarter take
    // alternate 128-byte-wide column panels.  Per panel: TMEM -> registers (one row per lane) ->
    // fused math -> the warp's private 4 KiB staging slab in shared memory -> coalesced 16-byte
    // global stores (fp32 add-reduction: vector red) by the same warp.  Nothing here waits on
    // another warp or on the TMA queue, which the producer keeps full of operand loads.
    const int eg = (warp - 2) >> 2;                // which of the quarter's EW warps
    const int quarter = warp & 3;
    const int epi = p.epi;
    const bool f32 = (epi == BB_EPI_ACCUM_F32 || epi == BB_EPI_STORE_F32);
    const bool dual = (epi == BB_EPI_BIAS_GELU);
    const bool has_aux = (epi == BB_EPI_MUL_DGELU || epi == BB_EPI_BIAS_RESIDUAL);
    int acc = 0; uint32_t acc_phase = 0;
    bool alive = true;
    if constexpr (EW == 4) {
      // Narrow variant for the epilogues with the most arithmetic per element (GeLU and its
      // derivative) on short reductions, where eight warps cannot finish a tile's epilogue
      // within the next tile's main loop: sixteen warps, 32 bf16 columns per pass (bf16 outputs only).
      uint8_t* slab = panels + (warp - 2) * (SLAB_BYTES / 2);
      for (uint32_t it = 0; alive; ++it) {
        int tile;
        if (!next_unit(it, tile, true)) { alive = false; break; }
        if (tile < 0) break;
        const int mn = tile % num_mn;
        const int mi = p.n_fast ? mn / num_n : mn % num_m, ni = p.n_fast ? mn % num_n : mn / num_m;
        const int m0 = mi * C::TILE_M + (int)rank * BM, n0 = ni * BN;
        const int r0 = m0 + quarter * 32;
        const bool got = bb::mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status);
        if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
        bb::tc_fence_after_sync();
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
        constexpr int npanels = BN / 32;
#pragma unroll 1
        for (int pn = eg; pn < npanels; pn += 4) {
          const int nb = n0 + pn * 32;
          const bool inside = (nb < p.N) && (r0 < p.M);
          if (has_aux && inside) slab64_fetch(slab, reinterpret_cast<const __nv_bfloat16*>(p.aux), p.ld_aux, r0, nb, p.M, p.N, lane);
          float v[32];
          {
            uint32_t r[32];
            bb::tmem_ld_32x32b_x32(t_row + pn * 32, r);
            bb::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          }
          if (pn + 4 >= npanels) {
            bb::tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) {
              if (PAIR) bb::mbar_arrive_cluster(bb::mapa_shared(bb::smem_u32(&tmem_empty[acc]), 0));
              else bb::mbar_arrive(&tmem_empty[acc]);
            }
          }
          if (!inside) continue;
          if (epi == BB_EPI_BIAS || dual || epi == BB_EPI_BIAS_RESIDUAL) add_bias<32>(p, nb, v);
          if (dual) {
            slab64_store_row(slab, lane, v);           // pre-activation first
            __syncwarp();
            slab64_flush(slab, reinterpret_cast<__nv_bfloat16*>(p.D2), p.ldd, r0, nb, p.M, p.N, lane);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = bb::gelu_tanh(__bfloat162float(__float2bfloat16(v[i])));
            __syncwarp();
          } else if (has_aux) {
            __syncwarp();
            float x[32];
#pragma unroll
            for (int c = 0; c < 4; ++c) unpack8(*reinterpret_cast<const uint4*>(slab + slab64_off(lane, c)), x + 8 * c);
            if (epi == BB_EPI_MUL_DGELU) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] *= bb::gelu_tanh_grad(x[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += x[i];
            }
            __syncwarp();
          }
          slab64_store_row(slab, lane, v);
          __syncwarp();
          slab64_flush(slab, reinterpret_cast<__nv_bfloat16*>(p.D), p.ldd, r0, nb, p.M, p.N, lane);
          __syncwarp();
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    } else {
    uint8_t* slab = panels + (warp - 2) * SLAB_BYTES;
    for (uint32_t it = 0; alive; ++it) {
      int tile;
      if (!next_unit(it, tile, true)) { alive = false; break; }
      if (tile < 0) break;
      const int mn = tile % num_mn;
      const int mi = p.n_fast ? mn / num_n : mn % num_m, ni = p.n_fast ? mn % num_n : mn / num_m;
      const int m0 = mi * C::TILE_M + (int)rank * BM, n0 = ni * BN;
      const int r0 = m0 + quarter * 32;            // first output row of this warp
      const bool got = bb::mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status);
      if (!__all_sync(0xffffffffu, got)) { alive = false; break; }
      bb::tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      const int width = f32 ? 32 : 64;             // columns per panel
      const int npanels = BN / width;
#pragma unroll 1
      for (int pn = eg; pn < npanels; pn += 2) {
        const int nb = n0 + pn * width;
        const bool inside = (nb < p.N) && (r0 < p.M);   // warp-uniform
        if (has_aux && inside) {
          // the aux tile comes in coalesced (rows spread over lanes) and is turned through the
          // slab, so that every lane can pick up its own row after the accumulator arrived
          uint4 ax[8];
          slab_fetch_bf16(reinterpret_cast<const __nv_bfloat16*>(p.aux), p.ld_aux, r0, nb, p.M, p.N, lane, ax);
          slab_put(slab, lane, ax);
        }
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
        if (pn + 2 >= npanels) {
          // this warp has read its share of the accumulator: hand it back before the last stores
          bb::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            if (PAIR) bb::mbar_arrive_cluster(bb::mapa_shared(bb::smem_u32(&tmem_empty[acc]), 0));
            else bb::mbar_arrive(&tmem_empty[acc]);
          }
        }
        if (!inside) continue;                     // panel entirely outside the matrix
        if (f32) {
          panel_store_row_f32(slab, lane, v);
          __syncwarp();
          if (epi == BB_EPI_ACCUM_F32) slab_flush_f32<true>(slab, reinterpret_cast<float*>(p.D), p.ldd, r0, nb, p.M, p.N, lane);
          else slab_flush_f32<false>(slab, reinterpret_cast<float*>(p.D), p.ldd, r0, nb, p.M, p.N, lane);
          __syncwarp();
          continue;
        }
        if (epi == BB_EPI_BIAS || dual || epi == BB_EPI_BIAS_RESIDUAL) add_bias<64>(p, nb, v);
        if (dual) {
          panel_store_row_bf16(slab, lane, v);     // pre-activation first
          __syncwarp();
          slab_flush_bf16(slab, reinterpret_cast<__nv_bfloat16*>(p.D2), p.ldd, r0, nb, p.M, p.N, lane);
          // GeLU of the bf16-rounded pre-activation: forward and backward (which re-reads the
          // stored pre-activation) see the same argument
#pragma unroll
          for (int i = 0; i < 64; ++i) v[i] = bb::gelu_tanh(__bfloat162float(__float2bfloat16(v[i])));
          __syncwarp();
        } else if (has_aux) {
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float x[32];
#pragma unroll
            for (int c = 0; c < 4; ++c) unpack8(*reinterpret_cast<const uint4*>(slab + slab_off(lane, 4 * h + c)), x + 8 * c);
            if (epi == BB_EPI_MUL_DGELU) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[32 * h + i] *= bb::gelu_tanh_grad(x[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[32 * h + i] += x[i];
            }
          }
          __syncwarp();
        }
        panel_store_row_bf16(slab, lane, v);
        __syncwarp();
        slab_flush_bf16(slab, reinterpret_cast<__nv_bfloat16*>(p.D), p.ldd, r0, nb, p.M, p.N, lane);
        __syncwarp();
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    }   // EW == 2
  }

  bb::tc_fence_before_sync();
  if (PAIR) {
    // neither CTA leaves (or frees TMEM) while the other may still signal its barriers
    bb::cluster_sync();
    if (warp == 1) bb::tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
  } else {
    __syncthreads();
    if (warp == 1) bb::tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host side
using bbhost::encode_2d;

// Ticket counters of the dynamic work distribution: a launch takes the next slot of a ring of
// counters in device memory and draws exactly `units` tickets from it (see the scheduling
// thread), so the host knows every counter's value without reading it back and nothing is ever
// reset.  A slot is reused 65536 launches later, long after the launch that held it retired.
constexpr unsigned TICKET_SLOTS = 1u << 16;
__device__ unsigned int g_gemm_tickets[TICKET_SLOTS];

struct TicketTable {
  unsigned int* dev = nullptr;
  std::atomic<unsigned> next{0};
  unsigned base[TICKET_SLOTS] = {};
};

// BB_GEMM_STATIC_SCHEDULE=1 in the environment restores the fixed stride (unit i of a CTA =
// its index + i x CTAs), for A/B measurements of the two distributions.
const bool g_static_schedule = [] { const char* e = getenv("BB_GEMM_STATIC_SCHEDULE"); return e && e[0] == '1'; }();

TicketTable* ticket_table() {
  static TicketTable* tables[64] = {nullptr};
  static std::mutex mu;
  const int dev = bb_current_device();
  if (dev < 0) return nullptr;
  TicketTable* t = tables[dev];
  if (t) return t;
  std::lock_guard<std::mutex> lock(mu);
  if (tables[dev]) return tables[dev];
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_gemm_tickets) != cudaSuccess) return nullptr;
  t = new TicketTable();
  t->dev = static_cast<unsigned int*>(ptr);
  tables[dev] = t;
  return t;
}

template <int BN, bool PAIR, int EW>
int launch(const bb_gemm_desc* g, cudaStream_t stream) {
  using C = Cfg<BN, PAIR>;
  CUtensorMap tmA, tmB;
  int rc;
  if (!g->a_mn_major) rc = encode_2d(&tmA, g->A, g->M, g->K, g->lda, BK, BM);
  else rc = encode_2d(&tmA, g->A, g->K, g->M, g->lda, 64, BK);
  if (rc) return rc;
  if (!g->b_mn_major) rc = encode_2d(&tmB, g->B, g->N, g->K, g->ldb, BK, C::B_ROWS);
  else rc = encode_2d(&tmB, g->B, g->K, g->N, g->ldb, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.M = g->M; p.N = g->N; p.K = g->K; p.a_mn = g->a_mn_major; p.b_mn = g->b_mn_major; p.epi = g->epilogue;
  p.D = g->D; p.D2 = g->D2; p.bias = g->bias; p.aux = g->aux; p.ldd = g->ldd; p.ld_aux = g->ld_aux ? g->ld_aux : g->ldd;
  p.status = bb_device_status_word();
  // The CTAs that run at the same time share one operand and stream the other: walk along the
  // dimension of the SMALLER operand, so that the larger one passes through L2 once.
  p.n_fast = (long long)g->M > (long long)g->N ? 1 : 0;
  const int total_kb = (g->K + BK - 1) / BK;
  const int mn_tiles = ((g->M + C::TILE_M - 1) / C::TILE_M) * ((g->N + BN - 1) / BN);
  const int workers_max = PAIR ? bb_num_sms() / 2 : bb_num_sms();
  int ksplit = 1;
  if (g->epilogue == BB_EPI_ACCUM_F32) {
    if (g->split_k > 0) {
      ksplit = g->split_k;
    } else {
      // too few output tiles to fill the machine: split the reduction; partial sums meet in
      // the fp32 add-reduction of the epilogue.  Cost model: waves x (k-blocks + fixed overhead).
      const int sms = workers_max;
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
  BB_ONCE_PER_DEVICE(BB_CUDA_CHECK(cudaFuncSetAttribute(gemm_bf16_tcgen05_kernel<BN, PAIR, EW>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES)));
  const int tiles = mn_tiles * p.ksplit;
  int workers = workers_max;
  if (g->max_ctas > 0 && g->max_ctas / (PAIR ? 2 : 1) < workers) workers = g->max_ctas / (PAIR ? 2 : 1);
  if (workers < 1) workers = 1;
  if (tiles < workers) workers = tiles;
  // max_ctas < 0: one work unit per CTA (or pair).  Meant for work on a low-priority stream: a
  // persistent CTA that found a free SM keeps it for its whole tile loop, and a persistent kernel
  // of the main stream launched meanwhile waits for that SM with a fixed share of the tiles.
  if (g->max_ctas < 0) workers = tiles;
  // more units than CTAs: every unit after a CTA's first is drawn from this launch's ticket counter
  p.dynamic = 0; p.ticket = nullptr; p.ticket_base = 0;
  unsigned slot = 0;
  TicketTable* tt = nullptr;
  if (tiles > workers && !g_static_schedule) {
    tt = ticket_table();
    if (!tt) { bb_set_last_error_msg("bb_gemm_bf16: ticket counters unavailable on this device"); return BB_ERR_CUDA; }
    slot = tt->next.fetch_add(1u) & (TICKET_SLOTS - 1);
    p.dynamic = 1; p.ticket = tt->dev + slot; p.ticket_base = tt->base[slot];
    tt->base[slot] += (unsigned)tiles;
  }
  if constexpr (PAIR) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * workers); cfg.blockDim = dim3(num_threads(EW));
    cfg.dynamicSmemBytes = C::SMEM_BYTES; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t le = cudaLaunchKernelEx(&cfg, gemm_bf16_tcgen05_kernel<BN, true, EW>, tmA, tmB, p);
    if (le != cudaSuccess) {
      if (tt) tt->base[slot] -= (unsigned)tiles;     // nothing ran: the counter keeps its value
      bb_set_last_error("gemm_bf16_tcgen05_kernel (pair) launch", le);
      return BB_ERR_CUDA;
    }
  } else {
    gemm_bf16_tcgen05_kernel<BN, false, EW><<<workers, num_threads(EW), C::SMEM_BYTES, stream>>>(tmA, tmB, p);
  }
  {
    cudaError_t le = cudaGetLastError();
    if (le != cudaSuccess) {
      if (tt) tt->base[slot] -= (unsigned)tiles;     // nothing ran: the counter keeps its value
      bb_set_last_error("gemm_bf16_tcgen05_kernel launch", le);
      return BB_ERR_CUDA;
    }
  }
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
  if ((g->epi_warps != 0 && g->epi_warps != 2 && g->epi_warps != 4) || (g->epi_warps == 4 && f32)) {
    bb_set_last_error_msg("bb_gemm_bf16: epi_warps must be 0, 2 or 4 (4 only with bf16 outputs)");
    return BB_ERR_INVALID_ARG;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // cuTensorMapEncodeTiled is a driver call and needs a context bound to the calling thread;
  // a thread that has only ever set its device (autograd worker threads) has none yet.
  if (int rc = bbhost::bind_context()) return rc;
  // CTA pairs (256 x 256 per pair) pay off on long reductions and on long runs of tiles per
  // CTA; short problems are quicker to start and drain as single CTAs (measured on B200:
  // K >= 3072 or >= 40 tiles per CTA 2-6 % faster as pairs, K = 1024 with <= 7 tiles 4-8 % slower)
  const long long tiles_single = (long long)((g->M + BM - 1) / BM) * ((g->N + 255) / 256);
  const bool pair = g->cta_pair > 0 ||
                    (g->cta_pair == 0 && g->tile_n == 0 && g->M > BM && g->N > 128 &&
                     (g->K >= 2048 || tiles_single >= 16LL * bb_num_sms()));
  // sixteen epilogue warps for the GeLU epilogues on short reductions (see the narrow variant)
  const bool wide_epi = g->epi_warps == 4 || (g->epi_warps == 0 && (e == BB_EPI_BIAS_GELU || e == BB_EPI_MUL_DGELU) && g->K <= 2048);
  if (pair) return wide_epi ? launch<256, true, 4>(g, s) : launch<256, true, 2>(g, s);
  int bn = g->tile_n;
  if (bn == 0) {
    // 256-wide tiles halve the A re-reads; use them when they still fill the machine
    const long long tiles256 = (long long)((g->M + BM - 1) / BM) * ((g->N + 255) / 256);
    // the add-reduction epilogue can split K to fill the machine, so it always takes wide tiles
    bn = (g->N > 128 && (tiles256 >= bb_num_sms() || e == BB_EPI_ACCUM_F32)) ? 256 : 128;
  }
  if (bn == 256) return wide_epi ? launch<256, false, 4>(g, s) : launch<256, false, 2>(g, s);
  if (bn == 128) return wide_epi ? launch<128, false, 4>(g, s) : launch<128, false, 2>(g, s);
  bb_set_last_error_msg("bb_gemm_bf16: tile_n must be 0, 128 or 256");
  return BB_ERR_INVALID_ARG;
}
