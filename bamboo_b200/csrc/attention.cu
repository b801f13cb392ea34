// Fused multi-head attention, forward and backward, without ever writing the [S,S]
// score matrix: Q.K^T -> online softmax -> P.V per 64-column block (forward); the backward
// pass recomputes the probabilities from the saved log-sum-exp and runs as two kernels,
// one owning a key/value block (dK, dV) and one owning a query block (dQ), so no atomics
// and a fixed summation order.  Tiles come in through cp.async into XOR-swizzled shared
// memory; contractions use warp-level mma (m16n8k16 bf16, fp32 accumulate).
//
// Layout: q, k, v are addressed as base + token * stride + head * D (so a packed
// [tokens, 3, H, D] projection output is consumed in place), token = batch * S + position.
#include "common.cuh"
#include <math.h>
#include <stdlib.h>

namespace {

constexpr int BLK_M = 128;   // rows owned by a CTA (8 warps x 16)
constexpr int BLK_N = 64;    // rows of the streamed operand per iteration
constexpr int THREADS = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  const __nv_bfloat16 *q, *k, *v, *o, *d_o;
  __nv_bfloat16 *out, *dq, *dk, *dv;
  float* lse;          // [B, H, S] natural-log units
  float* delta;        // [B, H, S] rowsum(dO * O)
  long long stride_qkv, stride_o, stride_dqkv;
  int B, H, S;
  int causal;
  float scale;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t* r) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// byte offset of element (row, col) in a [rows x D] bf16 tile whose 16-byte chunks are
// XOR-swizzled with the row index (conflict-free ldmatrix)
template <int D> __device__ __forceinline__ uint32_t tile_off(int row, int col) {
  const int chunk = col >> 3;
  return (uint32_t)(row * (D * 2) + (((chunk ^ (row & 7))) << 4) + ((col & 7) << 1));
}

// cooperative load of a [ROWS x D] tile; rows >= rows_valid are zero-filled
template <int D, int ROWS>
__device__ __forceinline__ void load_tile(uint32_t smem_base, const __nv_bfloat16* g, long long stride, int row0, int rows_total) {
  constexpr int CH = D / 8;
  for (int idx = threadIdx.x; idx < ROWS * CH; idx += THREADS) {
    const int r = idx / CH, c = idx % CH;
    const bool ok = (row0 + r) < rows_total;
    const __nv_bfloat16* src = g + (long long)(ok ? (row0 + r) : 0) * stride + c * 8;
    cp_async16(smem_base + tile_off<D>(r, c * 8), src, ok);
  }
}

// A-operand fragments (16 rows x D) of a row-major tile: frag[kk] covers columns 16kk..16kk+15
template <int D> __device__ __forceinline__ void load_a_frags(uint32_t tile, int row0, uint32_t (*frag)[4]) {
  const int lane = threadIdx.x & 31;
  const int r = row0 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) ldsm_x4(tile + tile_off<D>(r, kk * 16 + (lane >> 4) * 8), frag[kk]);
}

// acc[nt] (16 x 8 each, NT tiles) += A(16 x D) * Y^T where Y is a row-major [8*NT x D] tile
template <int D, int NT>
__device__ __forceinline__ void mma_a_bt(float (*acc)[4], const uint32_t (*a)[4], uint32_t tileY) {
  const int lane = threadIdx.x & 31;
  const int rsel = (lane & 7) + (lane >> 4) * 8, csel = ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldsm_x4(tileY + tile_off<D>(np * 16 + rsel, kk * 16 + csel), b);
      mma_bf16(acc[2 * np], a[kk], b[0], b[1]);
      mma_bf16(acc[2 * np + 1], a[kk], b[2], b[3]);
    }
  }
}

// acc[nt] (16 x 8, D/8 tiles) += P(16 x 64, given as 4 A fragments) * Z where Z is a row-major [64 x D] tile
template <int D>
__device__ __forceinline__ void mma_p_z(float (*acc)[4], const uint32_t (*p)[4], uint32_t tileZ) {
  const int lane = threadIdx.x & 31;
  const int rsel = (lane & 7) + ((lane >> 3) & 1) * 8, csel = (lane >> 4) * 8;
#pragma unroll
  for (int kk = 0; kk < BLK_N / 16; ++kk) {
#pragma unroll
    for (int np = 0; np < D / 16; ++np) {
      uint32_t b[4];
      ldsm_x4_t(tileZ + tile_off<D>(kk * 16 + rsel, np * 16 + csel), b);
      mma_bf16(acc[2 * np], p[kk], b[0], b[1]);
      mma_bf16(acc[2 * np + 1], p[kk], b[2], b[3]);
    }
  }
}

// accumulator tiles (16 x 64 as 8 n-tiles) -> 4 bf16 A fragments
__device__ __forceinline__ void acc_to_a(const float (*s)[4], uint32_t (*p)[4]) {
#pragma unroll
  for (int kk = 0; kk < BLK_N / 16; ++kk) {
    p[kk][0] = bb::pack_bf16x2(s[2 * kk][0], s[2 * kk][1]);
    p[kk][1] = bb::pack_bf16x2(s[2 * kk][2], s[2 * kk][3]);
    p[kk][2] = bb::pack_bf16x2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    p[kk][3] = bb::pack_bf16x2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
  }
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// write a warp's 16 x D fp32 accumulator block as bf16 rows
template <int D>
__device__ __forceinline__ void store_rows(__nv_bfloat16* g, long long stride, int row0, int rows_total, const float (*acc)[4],
                                           float mul0, float mul1) {
  const int lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
  const int r0 = row0 + gq, r1 = r0 + 8;
#pragma unroll
  for (int nt = 0; nt < D / 8; ++nt) {
    const int col = nt * 8 + 2 * t;
    if (r0 < rows_total) *reinterpret_cast<uint32_t*>(g + (long long)r0 * stride + col) = bb::pack_bf16x2(acc[nt][0] * mul0, acc[nt][1] * mul0);
    if (r1 < rows_total) *reinterpret_cast<uint32_t*>(g + (long long)r1 * stride + col) = bb::pack_bf16x2(acc[nt][2] * mul1, acc[nt][3] * mul1);
  }
}

// ------------------------------------------------------------------ forward
template <int D>
__global__ void __launch_bounds__(THREADS, (D == 64) ? 2 : 1)
attn_fwd_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int QB = BLK_M * D * 2, KB = BLK_N * D * 2;
  const uint32_t sQ = bb::smem_u32(smem), sK = sQ + QB, sV = sK + 2 * KB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heaviest (last) causal blocks first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int q0 = qb * BLK_M;
  const long long tok0 = (long long)batch * p.S;
  const __nv_bfloat16* qg = p.q + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* kg = p.k + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* vg = p.v + tok0 * p.stride_qkv + head * D;
  int nkv = (p.S + BLK_N - 1) / BLK_N;
  if (p.causal) nkv = min(nkv, (q0 + BLK_M + BLK_N - 1) / BLK_N);

  load_tile<D, BLK_M>(sQ, qg, p.stride_qkv, q0, p.S);
  load_tile<D, BLK_N>(sK, kg, p.stride_qkv, 0, p.S);
  load_tile<D, BLK_N>(sV, vg, p.stride_qkv, 0, p.S);
  cp_async_commit();

  uint32_t qf[D / 16][4];
  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};
  const float sl = p.scale * LOG2E;
  const int row_a = q0 + warp * 16 + gq, row_b = row_a + 8;

  for (int j = 0; j < nkv; ++j) {
    const int buf = j & 1;
    if (j + 1 < nkv) {
      load_tile<D, BLK_N>(sK + (buf ^ 1) * KB, kg, p.stride_qkv, (j + 1) * BLK_N, p.S);
      load_tile<D, BLK_N>(sV + (buf ^ 1) * KB, vg, p.stride_qkv, (j + 1) * BLK_N, p.S);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (j == 0) load_a_frags<D>(sQ, warp * 16, qf);

    float s[BLK_N / 8][4];
#pragma unroll
    for (int i = 0; i < BLK_N / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    mma_a_bt<D, BLK_N / 8>(s, qf, sK + buf * KB);

    const int c0 = j * BLK_N;
    const bool need_mask = (c0 + BLK_N > p.S) || (p.causal && c0 + BLK_N - 1 > q0 + warp * 16);
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < BLK_N / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[nt][e] * sl;
        if (need_mask) {
          const int col = c0 + nt * 8 + 2 * t + (e & 1);
          const int row = (e < 2) ? row_a : row_b;
          if (col >= p.S || (p.causal && col > row)) x = -INFINITY;
        }
        s[nt][e] = x;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = quad_max(mx0); mx1 = quad_max(mx1);
    const float mn0 = fmaxf(m_i[0], mx0), mn1 = fmaxf(m_i[1], mx1);
    const float ms0 = (mn0 == -INFINITY) ? 0.f : mn0, ms1 = (mn1 == -INFINITY) ? 0.f : mn1;
    const float al0 = exp2f(m_i[0] - ms0), al1 = exp2f(m_i[1] - ms1);
    m_i[0] = mn0; m_i[1] = mn1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < BLK_N / 8; ++nt) {
      s[nt][0] = exp2f(s[nt][0] - ms0); s[nt][1] = exp2f(s[nt][1] - ms0);
      s[nt][2] = exp2f(s[nt][2] - ms1); s[nt][3] = exp2f(s[nt][3] - ms1);
      rs0 += s[nt][0] + s[nt][1]; rs1 += s[nt][2] + s[nt][3];
    }
    l_i[0] = l_i[0] * al0 + rs0; l_i[1] = l_i[1] * al1 + rs1;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
    uint32_t pf[BLK_N / 16][4];
    acc_to_a(s, pf);
    mma_p_z<D>(o, pf, sV + buf * KB);
    __syncthreads();
  }
  const float l0 = quad_sum(l_i[0]), l1 = quad_sum(l_i[1]);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  __nv_bfloat16* og = p.out + tok0 * p.stride_o + head * D;
  store_rows<D>(og, p.stride_o, q0 + warp * 16, p.S, o, inv0, inv1);
  if (t == 0) {
    float* lse = p.lse + ((long long)batch * p.H + head) * p.S;
    if (row_a < p.S) lse[row_a] = (l0 > 0.f) ? (m_i[0] + log2f(l0)) / LOG2E : -INFINITY;
    if (row_b < p.S) lse[row_b] = (l1 > 0.f) ? (m_i[1] + log2f(l1)) / LOG2E : -INFINITY;
  }
}

// ------------------------------------------------------------------ delta = rowsum(dO * O)
template <int D>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const AttnParams p) {
  // one warp per (token, head)
  const int lane = threadIdx.x & 31;
  const long long total = (long long)p.B * p.S * p.H;
  for (long long w = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); w < total; w += (long long)gridDim.x * 8) {
    const long long tok = w / p.H; const int head = (int)(w % p.H);
    const __nv_bfloat16* o = p.o + tok * p.stride_o + head * D;
    const __nv_bfloat16* d = p.d_o + tok * p.stride_o + head * D;
    float s = 0.f;
    for (int c = lane * 2; c < D; c += 64) {
      const uint32_t a = *reinterpret_cast<const uint32_t*>(o + c), b = *reinterpret_cast<const uint32_t*>(d + c);
      s += bb::bf16_lo(a) * bb::bf16_lo(b) + bb::bf16_hi(a) * bb::bf16_hi(b);
    }
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) s += __shfl_xor_sync(0xffffffffu, s, k);
    if (lane == 0) {
      const long long b = tok / p.S; const int pos = (int)(tok % p.S);
      p.delta[(b * p.H + head) * p.S + pos] = s;
    }
  }
}

// ------------------------------------------------------------------ backward: dK, dV (CTA owns 128 key rows)
template <int D>
__global__ void __launch_bounds__(THREADS)
attn_bwd_dkv_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int KB = BLK_M * D * 2, QB = BLK_N * D * 2;
  const uint32_t sK = bb::smem_u32(smem), sV = sK + KB, sQ = sV + KB, sDO = sQ + 2 * QB;
  float* s_lse = reinterpret_cast<float*>(smem + 2 * KB + 4 * QB);   // [2][BLK_N]
  float* s_delta = s_lse + 2 * BLK_N;                                // [2][BLK_N]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
  const int kb = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int k0 = kb * BLK_M;
  const long long tok0 = (long long)batch * p.S;
  const __nv_bfloat16* qg = p.q + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* kg = p.k + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* vg = p.v + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* dog = p.d_o + tok0 * p.stride_o + head * D;
  const float* lse_g = p.lse + ((long long)batch * p.H + head) * p.S;
  const float* delta_g = p.delta + ((long long)batch * p.H + head) * p.S;
  const int nq = (p.S + BLK_N - 1) / BLK_N;
  const int qstart = p.causal ? (k0 / BLK_N) : 0;

  auto load_q_block = [&](int i, int buf) {
    load_tile<D, BLK_N>(sQ + buf * QB, qg, p.stride_qkv, i * BLK_N, p.S);
    load_tile<D, BLK_N>(sDO + buf * QB, dog, p.stride_o, i * BLK_N, p.S);
    if (threadIdx.x < BLK_N) {
      const int r = i * BLK_N + threadIdx.x;
      s_lse[buf * BLK_N + threadIdx.x] = (r < p.S) ? lse_g[r] * LOG2E : 0.f;
      s_delta[buf * BLK_N + threadIdx.x] = (r < p.S) ? delta_g[r] : 0.f;
    }
  };
  load_tile<D, BLK_M>(sK, kg, p.stride_qkv, k0, p.S);
  load_tile<D, BLK_M>(sV, vg, p.stride_qkv, k0, p.S);
  if (qstart < nq) load_q_block(qstart, 0);
  cp_async_commit();

  uint32_t kf[D / 16][4], vf[D / 16][4];
  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f; dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f; }
  const float sl = p.scale * LOG2E;
  const int kr_a = k0 + warp * 16 + gq, kr_b = kr_a + 8;

  for (int i = qstart; i < nq; ++i) {
    const int buf = (i - qstart) & 1;
    if (i + 1 < nq) { load_q_block(i + 1, buf ^ 1); cp_async_commit(); cp_async_wait<1>(); }
    else cp_async_wait<0>();
    __syncthreads();
    if (i == qstart) { load_a_frags<D>(sK, warp * 16, kf); load_a_frags<D>(sV, warp * 16, vf); }

    // S^T = K Q^T  : rows = key, cols = query
    float st[BLK_N / 8][4];
#pragma unroll
    for (int n = 0; n < BLK_N / 8; ++n) st[n][0] = st[n][1] = st[n][2] = st[n][3] = 0.f;
    mma_a_bt<D, BLK_N / 8>(st, kf, sQ + buf * QB);
    // dP^T = V dO^T
    float dpt[BLK_N / 8][4];
#pragma unroll
    for (int n = 0; n < BLK_N / 8; ++n) dpt[n][0] = dpt[n][1] = dpt[n][2] = dpt[n][3] = 0.f;
    mma_a_bt<D, BLK_N / 8>(dpt, vf, sDO + buf * QB);

    const int qc0 = i * BLK_N;
#pragma unroll
    for (int n = 0; n < BLK_N / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qi = n * 8 + 2 * t + (e & 1);
        const int qrow = qc0 + qi;
        const int krow = (e < 2) ? kr_a : kr_b;
        float pv = exp2f(st[n][e] * sl - s_lse[buf * BLK_N + qi]);
        if (qrow >= p.S || krow >= p.S || (p.causal && krow > qrow)) pv = 0.f;
        st[n][e] = pv;
        dpt[n][e] = pv * (dpt[n][e] - s_delta[buf * BLK_N + qi]);
      }
    }
    uint32_t pf[BLK_N / 16][4], dsf[BLK_N / 16][4];
    acc_to_a(st, pf);
    acc_to_a(dpt, dsf);
    mma_p_z<D>(dv, pf, sDO + buf * QB);   // dV += P^T dO
    mma_p_z<D>(dk, dsf, sQ + buf * QB);   // dK += dS^T Q
    __syncthreads();
  }
  __nv_bfloat16* dkg = p.dk + tok0 * p.stride_dqkv + head * D;
  __nv_bfloat16* dvg = p.dv + tok0 * p.stride_dqkv + head * D;
  store_rows<D>(dkg, p.stride_dqkv, k0 + warp * 16, p.S, dk, p.scale, p.scale);
  store_rows<D>(dvg, p.stride_dqkv, k0 + warp * 16, p.S, dv, 1.f, 1.f);
}

// ------------------------------------------------------------------ backward: dQ (CTA owns 128 query rows)
template <int D>
__global__ void __launch_bounds__(THREADS)
attn_bwd_dq_kernel(const AttnParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int QB = BLK_M * D * 2, KB = BLK_N * D * 2;
  const uint32_t sQ = bb::smem_u32(smem), sDO = sQ + QB, sK = sDO + QB, sV = sK + 2 * KB;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gq = lane >> 2, t = lane & 3;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, batch = blockIdx.z;
  const int q0 = qb * BLK_M;
  const long long tok0 = (long long)batch * p.S;
  const __nv_bfloat16* qg = p.q + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* kg = p.k + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* vg = p.v + tok0 * p.stride_qkv + head * D;
  const __nv_bfloat16* dog = p.d_o + tok0 * p.stride_o + head * D;
  const float* lse_g = p.lse + ((long long)batch * p.H + head) * p.S;
  const float* delta_g = p.delta + ((long long)batch * p.H + head) * p.S;
  int nkv = (p.S + BLK_N - 1) / BLK_N;
  if (p.causal) nkv = min(nkv, (q0 + BLK_M + BLK_N - 1) / BLK_N);

  load_tile<D, BLK_M>(sQ, qg, p.stride_qkv, q0, p.S);
  load_tile<D, BLK_M>(sDO, dog, p.stride_o, q0, p.S);
  load_tile<D, BLK_N>(sK, kg, p.stride_qkv, 0, p.S);
  load_tile<D, BLK_N>(sV, vg, p.stride_qkv, 0, p.S);
  cp_async_commit();

  const int row_a = q0 + warp * 16 + gq, row_b = row_a + 8;
  const float lse_a = (row_a < p.S) ? lse_g[row_a] * LOG2E : 0.f, lse_b = (row_b < p.S) ? lse_g[row_b] * LOG2E : 0.f;
  const float dl_a = (row_a < p.S) ? delta_g[row_a] : 0.f, dl_b = (row_b < p.S) ? delta_g[row_b] : 0.f;
  uint32_t qf[D / 16][4], dof[D / 16][4];
  float dq[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) dq[i][0] = dq[i][1] = dq[i][2] = dq[i][3] = 0.f;
  const float sl = p.scale * LOG2E;

  for (int j = 0; j < nkv; ++j) {
    const int buf = j & 1;
    if (j + 1 < nkv) {
      load_tile<D, BLK_N>(sK + (buf ^ 1) * KB, kg, p.stride_qkv, (j + 1) * BLK_N, p.S);
      load_tile<D, BLK_N>(sV + (buf ^ 1) * KB, vg, p.stride_qkv, (j + 1) * BLK_N, p.S);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (j == 0) { load_a_frags<D>(sQ, warp * 16, qf); load_a_frags<D>(sDO, warp * 16, dof); }

    float s[BLK_N / 8][4], dp[BLK_N / 8][4];
#pragma unroll
    for (int n = 0; n < BLK_N / 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; dp[n][0] = dp[n][1] = dp[n][2] = dp[n][3] = 0.f; }
    mma_a_bt<D, BLK_N / 8>(s, qf, sK + buf * KB);     // S = Q K^T
    mma_a_bt<D, BLK_N / 8>(dp, dof, sV + buf * KB);   // dP = dO V^T
    const int c0 = j * BLK_N;
#pragma unroll
    for (int n = 0; n < BLK_N / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = c0 + n * 8 + 2 * t + (e & 1);
        const int row = (e < 2) ? row_a : row_b;
        float pv = exp2f(s[n][e] * sl - ((e < 2) ? lse_a : lse_b));
        if (col >= p.S || row >= p.S || (p.causal && col > row)) pv = 0.f;
        dp[n][e] = pv * (dp[n][e] - ((e < 2) ? dl_a : dl_b));
      }
    }
    uint32_t dsf[BLK_N / 16][4];
    acc_to_a(dp, dsf);
    mma_p_z<D>(dq, dsf, sK + buf * KB);   // dQ += dS K
    __syncthreads();
  }
  __nv_bfloat16* dqg = p.dq + tok0 * p.stride_dqkv + head * D;
  store_rows<D>(dqg, p.stride_dqkv, q0 + warp * 16, p.S, dq, p.scale, p.scale);
}

template <int D> int fwd_smem() { return BLK_M * D * 2 + 4 * BLK_N * D * 2; }
template <int D> int dkv_smem() { return 2 * BLK_M * D * 2 + 4 * BLK_N * D * 2 + 4 * BLK_N * (int)sizeof(float); }
template <int D> int dq_smem() { return 2 * BLK_M * D * 2 + 4 * BLK_N * D * 2; }

template <int D>
int launch_fwd(const AttnParams& p, cudaStream_t s) {
  BB_ONCE_PER_DEVICE(BB_CUDA_CHECK(cudaFuncSetAttribute(attn_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, fwd_smem<D>())));
  dim3 grid((p.S + BLK_M - 1) / BLK_M, p.H, p.B);
  attn_fwd_kernel<D><<<grid, THREADS, fwd_smem<D>(), s>>>(p);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

template <int D>
int launch_bwd(const AttnParams& p, cudaStream_t s) {
  BB_ONCE_PER_DEVICE({
    BB_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv_smem<D>()));
    BB_CUDA_CHECK(cudaFuncSetAttribute(attn_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, dq_smem<D>()));
  });
  const long long units = (long long)p.B * p.S * p.H;
  long long dgrid = (units + 7) / 8, cap = (long long)bb_num_sms() * 8;
  attn_delta_kernel<D><<<(int)(dgrid < cap ? dgrid : cap), 256, 0, s>>>(p);
  dim3 grid((p.S + BLK_M - 1) / BLK_M, p.H, p.B);
  attn_bwd_dkv_kernel<D><<<grid, THREADS, dkv_smem<D>(), s>>>(p);
  attn_bwd_dq_kernel<D><<<grid, THREADS, dq_smem<D>(), s>>>(p);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

bool bad_layout(long long stride, int D, const void* a, const void* b, const void* c) {
  return (stride & 7) || (D & 15) || (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15);
}

}  // namespace

// tcgen05 kernels (attention_tc.cu): forward for head dimensions 64 and 128, backward for 64
int bb_attention_tc_fwd(const void* qkv_q, void* out, float* lse, int B, int H, int S, int D, long long stride_qkv,
                        long long stride_o, int causal, float scale, cudaStream_t stream);
int bb_attention_tc_bwd(const void* qkv_q, const void* out, const void* d_out, const float* lse, void* dq, void* dk, void* dv,
                        float* delta, float* dq_acc, int B, int H, int S, long long stride_qkv, long long stride_o,
                        long long stride_dqkv, int causal, float scale, cudaStream_t stream);

namespace {
// The tcgen05 kernels (attention_tc.cu) read q, k, v through one tensor map over the packed
// projection [tokens, 3*H*D] and are the default for head dimension 64 (forward and backward) and
// for the forward pass at head dimension 128.  Measured on B200 (B8 H16 S1024 D64 causal): forward
// 70 us, backward 180 us, against 120 us and 593 us for the warp-level kernels above; B2 H32 S2048
// D128 causal: forward 121 us.  BB_ATTENTION_IMPL=mma in the environment forces the warp-level kernels.
bool use_tc_path(const void* q, const void* k, const void* v, int H, int D, long long stride_qkv, bool forward) {
  static int mode = -1;   // 0 = tcgen05 kernels where they apply (default), 2 = warp-level kernels only
  if (mode < 0) {
    const char* e = getenv("BB_ATTENTION_IMPL");
    mode = (e && e[0] == 'm') ? 2 : 0;
  }
  if (mode == 2 || !(D == 64 || (D == 128 && forward))) return false;
  // the tcgen05 kernels address q, k and v through one tensor map over the packed projection
  const long long hb = (long long)H * D * 2;
  return (const char*)k - (const char*)q == hb && (const char*)v - (const char*)q == 2 * hb && stride_qkv >= 3LL * H * D &&
         (long long)H * D * 3 < (1LL << 31);
}
}  // namespace

extern "C" int bb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int S, int D,
                                long long stride_qkv, long long stride_o, int causal, float scale, void* stream) {
  if (!q || !k || !v || !out || !lse || B <= 0 || H <= 0 || S <= 0 || bad_layout(stride_qkv, D, q, k, v) ||
      bad_layout(stride_o, D, out, nullptr, nullptr)) {
    bb_set_last_error_msg("bb_attention_fwd: null/unaligned pointer or stride not a multiple of 8 elements");
    return BB_ERR_INVALID_ARG;
  }
  AttnParams p = {};
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.out = (__nv_bfloat16*)out;
  p.lse = lse; p.stride_qkv = stride_qkv; p.stride_o = stride_o; p.B = B; p.H = H; p.S = S; p.causal = causal; p.scale = scale;
  if (use_tc_path(q, k, v, H, D, stride_qkv, true))
    return bb_attention_tc_fwd(q, out, lse, B, H, S, D, stride_qkv, stride_o, causal, scale, (cudaStream_t)stream);
  if (D == 64) return launch_fwd<64>(p, (cudaStream_t)stream);
  if (D == 128) return launch_fwd<128>(p, (cudaStream_t)stream);
  bb_set_last_error_msg("bb_attention_fwd: head dimension must be 64 or 128");
  return BB_ERR_UNSUPPORTED;
}

namespace {
// workspace: delta [B, H, S] fp32, then (256-byte aligned) the fp32 dQ accumulator [B, H, S, 64] of
// the fused tcgen05 backward (head dimension 64; the size does not depend on the head dimension
// because this query has none)
long long attn_ws_delta_bytes(int B, int H, int S) { return (((long long)B * H * S * (long long)sizeof(float)) + 255) & ~255LL; }
}  // namespace

extern "C" long long bb_attention_bwd_workspace_bytes(int B, int H, int S) {
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  return attn_ws_delta_bytes(B, H, S) + (long long)B * H * S * 64 * (long long)sizeof(float);
}

extern "C" int bb_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out, const float* lse,
                                void* dq, void* dk, void* dv, void* workspace, long long workspace_bytes, int B, int H, int S,
                                int D, long long stride_qkv, long long stride_o, long long stride_dqkv, int causal, float scale,
                                void* stream) {
  if (!q || !k || !v || !out || !d_out || !lse || !dq || !dk || !dv || !workspace || B <= 0 || H <= 0 || S <= 0 ||
      bad_layout(stride_qkv, D, q, k, v) || bad_layout(stride_o, D, out, d_out, nullptr) || bad_layout(stride_dqkv, D, dq, dk, dv)) {
    bb_set_last_error_msg("bb_attention_bwd: null/unaligned pointer or stride not a multiple of 8 elements");
    return BB_ERR_INVALID_ARG;
  }
  if (workspace_bytes < bb_attention_bwd_workspace_bytes(B, H, S)) {
    bb_set_last_error_msg("bb_attention_bwd: workspace smaller than bb_attention_bwd_workspace_bytes()");
    return BB_ERR_INVALID_ARG;
  }
  AttnParams p = {};
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v;
  p.o = (const __nv_bfloat16*)out; p.d_o = (const __nv_bfloat16*)d_out;
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv;
  p.lse = const_cast<float*>(lse); p.delta = (float*)workspace;
  p.stride_qkv = stride_qkv; p.stride_o = stride_o; p.stride_dqkv = stride_dqkv;
  p.B = B; p.H = H; p.S = S; p.causal = causal; p.scale = scale;
  if (use_tc_path(q, k, v, H, D, stride_qkv, false))
    return bb_attention_tc_bwd(q, out, d_out, lse, dq, dk, dv, (float*)workspace,
                               (float*)((char*)workspace + attn_ws_delta_bytes(B, H, S)), B, H, S, stride_qkv, stride_o,
                               stride_dqkv, causal, scale, (cudaStream_t)stream);
  if (D == 64) return launch_bwd<64>(p, (cudaStream_t)stream);
  if (D == 128) return launch_bwd<128>(p, (cudaStream_t)stream);
  bb_set_last_error_msg("bb_attention_bwd: head dimension must be 64 or 128");
  return BB_ERR_UNSUPPORTED;
}
