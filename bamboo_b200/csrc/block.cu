// Half a transformer block per call: the host-side sequencing of the kernels that the layer
// modules would otherwise launch one foreign call at a time.  Nothing here runs on the device;
// every launch goes through the library's own entry points, so the arithmetic is theirs.
#include "common.cuh"
#include "bamboo_b200.h"

namespace {

inline long long align256(long long n) { return (n + 255) & ~255LL; }

// Layout of `saved` (forward -> backward) and `scratch` (backward only); all offsets 256-byte aligned.
struct AttnLayout {
  long long h1, qkv, att, lse, mean, rstd, saved_total;
  long long datt, dqkv, dh1, ws_ln, ws_attn, ws_colsum, scratch_total;
};
struct MlpLayout {
  long long h2, pre, act, mean, rstd, saved_total;
  long long dpre, dh2, ws_ln, ws_colsum, scratch_total;
};

AttnLayout attn_layout(const bb_block_desc* d) {
  AttnLayout L;
  const long long T = d->tokens, h = d->hidden;
  long long o = 0;
  L.h1 = o;   o += align256(T * h * 2);
  L.qkv = o;  o += align256(T * 3 * h * 2);
  L.att = o;  o += align256(T * h * 2);
  L.lse = o;  o += align256((long long)d->batch * d->heads * d->seq * 4);
  L.mean = o; o += align256(T * 4);
  L.rstd = o; o += align256(T * 4);
  L.saved_total = o;
  o = 0;
  L.datt = o; o += align256(T * h * 2);
  L.dqkv = o; o += align256(T * 3 * h * 2);
  L.dh1 = o;  o += align256(T * h * 2);
  L.ws_ln = o;     o += align256(bb_layernorm_bwd_res_workspace_bytes((int)T, (int)h));
  L.ws_attn = o;   o += align256(bb_attention_bwd_workspace_bytes(d->batch, d->heads, d->seq));
  L.ws_colsum = o; o += align256(bb_colsum_workspace_bytes((int)T, (int)(3 * h)));
  L.scratch_total = o;
  return L;
}

MlpLayout mlp_layout(const bb_block_desc* d) {
  MlpLayout L;
  const long long T = d->tokens, h = d->hidden, f = d->ffn;
  long long o = 0;
  L.h2 = o;   o += align256(T * h * 2);
  L.pre = o;  o += align256(T * f * 2);
  L.act = o;  o += align256(T * f * 2);
  L.mean = o; o += align256(T * 4);
  L.rstd = o; o += align256(T * 4);
  L.saved_total = o;
  o = 0;
  L.dpre = o; o += align256(T * f * 2);
  L.dh2 = o;  o += align256(T * h * 2);
  L.ws_ln = o;     o += align256(bb_layernorm_bwd_res_workspace_bytes((int)T, (int)h));
  L.ws_colsum = o; o += align256(bb_colsum_workspace_bytes((int)T, (int)f));
  L.scratch_total = o;
  return L;
}

int gemm(const bb_block_desc* d, int M, int N, int K, const void* A, long long lda, int a_mn, const void* B, long long ldb,
         int b_mn, void* D, long long ldd, int epi, const void* bias, void* D2, const void* aux, long long ld_aux,
         void* stream) {
  bb_gemm_desc g = {};
  g.M = M; g.N = N; g.K = K; g.A = A; g.lda = lda; g.a_mn_major = a_mn; g.B = B; g.ldb = ldb; g.b_mn_major = b_mn;
  g.D = D; g.ldd = ldd; g.epilogue = epi; g.bias = bias; g.D2 = D2; g.aux = aux; g.ld_aux = ld_aux;
  g.max_ctas = d->max_ctas;
  return bb_gemm_bf16(&g, stream);
}

// side stream waits for everything issued on `stream` so far (no-op when they are the same stream)
int fork_to(void* stream, void* side) {
  if (stream == side) return BB_OK;
  static cudaEvent_t ev[64] = {nullptr};
  const int dev = bb_current_device();
  if (dev < 0) { bb_set_last_error_msg("bb_block_half_bwd: no current device"); return BB_ERR_CUDA; }
  if (!ev[dev]) BB_CUDA_CHECK(cudaEventCreateWithFlags(&ev[dev], cudaEventDisableTiming));
  BB_CUDA_CHECK(cudaEventRecord(ev[dev], (cudaStream_t)stream));
  BB_CUDA_CHECK(cudaStreamWaitEvent((cudaStream_t)side, ev[dev], 0));
  return BB_OK;
}

#define BB_TRY(expr) do { int _rc = (expr); if (_rc != BB_OK) return _rc; } while (0)

bool bad_desc(const bb_block_desc* d, int half) {
  return !d || d->tokens <= 0 || d->hidden <= 0 || (d->hidden & 7) || !d->ln_w || !d->ln_b || !d->w1 || !d->b1 || !d->w2 ||
         !d->b2 || (half == BB_HALF_ATTENTION ? (d->batch <= 0 || d->seq <= 0 || d->heads <= 0 || d->head_dim <= 0 ||
                                                 d->heads * d->head_dim != d->hidden || d->batch * d->seq != d->tokens)
                                              : (d->ffn <= 0 || (d->ffn & 7))) ||
         (half != BB_HALF_ATTENTION && half != BB_HALF_MLP);
}

}  // namespace

extern "C" long long bb_block_saved_bytes(const bb_block_desc* d, int half) {
  if (bad_desc(d, half)) return -1;
  return half == BB_HALF_ATTENTION ? attn_layout(d).saved_total : mlp_layout(d).saved_total;
}

extern "C" long long bb_block_scratch_bytes(const bb_block_desc* d, int half) {
  if (bad_desc(d, half)) return -1;
  return half == BB_HALF_ATTENTION ? attn_layout(d).scratch_total : mlp_layout(d).scratch_total;
}

extern "C" int bb_block_half_fwd(const bb_block_desc* d, int half, const void* x, void* saved, void* out, void* stream) {
  if (bad_desc(d, half) || !x || !saved || !out) {
    bb_set_last_error_msg("bb_block_half_fwd: bad descriptor or null buffer");
    return BB_ERR_INVALID_ARG;
  }
  const int T = d->tokens, h = d->hidden;
  uint8_t* sv = static_cast<uint8_t*>(saved);
  if (half == BB_HALF_ATTENTION) {
    const AttnLayout L = attn_layout(d);
    void* h1 = sv + L.h1; uint8_t* qkv = sv + L.qkv; void* att = sv + L.att;
    float* lse = reinterpret_cast<float*>(sv + L.lse);
    float* mean = reinterpret_cast<float*>(sv + L.mean); float* rstd = reinterpret_cast<float*>(sv + L.rstd);
    BB_TRY(bb_layernorm_fwd(x, d->ln_w, d->ln_b, h1, mean, rstd, T, h, d->eps, stream));
    BB_TRY(gemm(d, T, 3 * h, h, h1, h, 0, d->w1, h, 0, qkv, 3LL * h, BB_EPI_BIAS, d->b1, nullptr, nullptr, 0, stream));
    BB_TRY(bb_attention_fwd(qkv, qkv + 2LL * h, qkv + 4LL * h, att, lse, d->batch, d->heads, d->seq, d->head_dim, 3LL * h, h,
                            d->causal, 1.0f / sqrtf((float)d->head_dim), stream));
    BB_TRY(gemm(d, T, h, h, att, h, 0, d->w2, h, 0, out, h, BB_EPI_BIAS_RESIDUAL, d->b2, nullptr, x, h, stream));
    return BB_OK;
  }
  const MlpLayout L = mlp_layout(d);
  const int f = d->ffn;
  void* h2 = sv + L.h2; void* pre = sv + L.pre; void* act = sv + L.act;
  float* mean = reinterpret_cast<float*>(sv + L.mean); float* rstd = reinterpret_cast<float*>(sv + L.rstd);
  BB_TRY(bb_layernorm_fwd(x, d->ln_w, d->ln_b, h2, mean, rstd, T, h, d->eps, stream));
  BB_TRY(gemm(d, T, f, h, h2, h, 0, d->w1, h, 0, act, f, BB_EPI_BIAS_GELU, d->b1, pre, nullptr, 0, stream));
  BB_TRY(gemm(d, T, h, f, act, f, 0, d->w2, f, 0, out, h, BB_EPI_BIAS_RESIDUAL, d->b2, nullptr, x, h, stream));
  return BB_OK;
}

extern "C" int bb_block_half_bwd(const bb_block_desc* d, int half, const void* x, const void* saved, const void* dout, void* dx,
                                 void* scratch, long long scratch_bytes, void* stream, void* side_stream) {
  if (bad_desc(d, half) || !x || !saved || !dout || !dx || !scratch || !d->g_ln_w || !d->g_ln_b || !d->g_w1 || !d->g_b1 ||
      !d->g_w2 || !d->g_b2) {
    bb_set_last_error_msg("bb_block_half_bwd: bad descriptor, null buffer or missing gradient pointer");
    return BB_ERR_INVALID_ARG;
  }
  if (scratch_bytes < bb_block_scratch_bytes(d, half)) {
    bb_set_last_error_msg("bb_block_half_bwd: scratch smaller than bb_block_scratch_bytes");
    return BB_ERR_INVALID_ARG;
  }
  const int T = d->tokens, h = d->hidden;
  const uint8_t* sv = static_cast<const uint8_t*>(saved);
  uint8_t* sc = static_cast<uint8_t*>(scratch);
  if (half == BB_HALF_ATTENTION) {
    const AttnLayout L = attn_layout(d);
    const void* h1 = sv + L.h1; const uint8_t* qkv = sv + L.qkv; const void* att = sv + L.att;
    const float* lse = reinterpret_cast<const float*>(sv + L.lse);
    const float* mean = reinterpret_cast<const float*>(sv + L.mean);
    const float* rstd = reinterpret_cast<const float*>(sv + L.rstd);
    void* datt = sc + L.datt; uint8_t* dqkv = sc + L.dqkv; void* dh1 = sc + L.dh1;
    // input gradients along the chain: proj, attention, qkv
    BB_TRY(gemm(d, T, h, h, dout, h, 0, d->w2, h, 1, datt, h, BB_EPI_STORE, nullptr, nullptr, nullptr, 0, stream));
    BB_TRY(bb_attention_bwd(qkv, qkv + 2LL * h, qkv + 4LL * h, att, datt, lse, dqkv, dqkv + 2LL * h, dqkv + 4LL * h, sc + L.ws_attn,
                            bb_attention_bwd_workspace_bytes(d->batch, d->heads, d->seq), d->batch, d->heads, d->seq,
                            d->head_dim, 3LL * h, h, 3LL * h, d->causal, 1.0f / sqrtf((float)d->head_dim), stream));
    BB_TRY(gemm(d, T, h, 3 * h, dqkv, 3LL * h, 0, d->w1, h, 1, dh1, h, BB_EPI_STORE, nullptr, nullptr, nullptr, 0, stream));
    // weight and bias gradients beside the chain
    BB_TRY(fork_to(stream, side_stream));
    BB_TRY(gemm(d, h, h, T, dout, h, 1, att, h, 1, d->g_w2, h, BB_EPI_ACCUM_F32, nullptr, nullptr, nullptr, 0, side_stream));
    BB_TRY(gemm(d, 3 * h, h, T, dqkv, 3LL * h, 1, h1, h, 1, d->g_w1, h, BB_EPI_ACCUM_F32, nullptr, nullptr, nullptr, 0, side_stream));
    BB_TRY(bb_colsum_accum(dqkv, 3LL * h, d->g_b1, sc + L.ws_colsum, bb_colsum_workspace_bytes(T, 3 * h), T, 3 * h, side_stream));
    // the LayerNorm backward reads dout as the residual gradient: the projection's bias gradient
    // (dout's column sums) comes out of the same pass
    BB_TRY(bb_layernorm_bwd_res(dh1, x, d->ln_w, mean, rstd, dout, dx, d->g_ln_w, d->g_ln_b, d->g_b2, sc + L.ws_ln,
                                bb_layernorm_bwd_res_workspace_bytes(T, h), T, h, stream));
    return BB_OK;
  }
  const MlpLayout L = mlp_layout(d);
  const int f = d->ffn;
  const void* h2 = sv + L.h2; const void* pre = sv + L.pre; const void* act = sv + L.act;
  const float* mean = reinterpret_cast<const float*>(sv + L.mean);
  const float* rstd = reinterpret_cast<const float*>(sv + L.rstd);
  void* dpre = sc + L.dpre; void* dh2 = sc + L.dh2;
  // d(pre) = (dout W2) * gelu'(pre) in the epilogue, then through fc1
  BB_TRY(gemm(d, T, f, h, dout, h, 0, d->w2, f, 1, dpre, f, BB_EPI_MUL_DGELU, nullptr, nullptr, pre, f, stream));
  BB_TRY(gemm(d, T, h, f, dpre, f, 0, d->w1, h, 1, dh2, h, BB_EPI_STORE, nullptr, nullptr, nullptr, 0, stream));
  BB_TRY(fork_to(stream, side_stream));
  BB_TRY(gemm(d, h, f, T, dout, h, 1, act, f, 1, d->g_w2, f, BB_EPI_ACCUM_F32, nullptr, nullptr, nullptr, 0, side_stream));
  BB_TRY(gemm(d, f, h, T, dpre, f, 1, h2, h, 1, d->g_w1, h, BB_EPI_ACCUM_F32, nullptr, nullptr, nullptr, 0, side_stream));
  BB_TRY(bb_colsum_accum(dpre, f, d->g_b1, sc + L.ws_colsum, bb_colsum_workspace_bytes(T, f), T, f, side_stream));
  BB_TRY(bb_layernorm_bwd_res(dh2, x, d->ln_w, mean, rstd, dout, dx, d->g_ln_w, d->g_ln_b, d->g_b2, sc + L.ws_ln,
                              bb_layernorm_bwd_res_workspace_bytes(T, h), T, h, stream));
  return BB_OK;
}
