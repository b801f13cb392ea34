/* C ABI of libbamboo_b200.so - the sm_100a kernels behind Bamboo's pipeline step.
 *
 * The reference (uclasystem/bamboo, patched DeepSpeed 0.5.2) has no C ABI for stage
 * compute or inter-stage transfer: its pipeline engine calls PyTorch/ATen (cuBLAS, eager
 * elementwise kernels), torch.distributed send/recv and two pybind11 modules
 * (fused Adam, flatten/unflatten).  Each entry point below names the reference call
 * site(s) whose GPU work it replaces.  Paths are relative to the reference checkout;
 * DS = external/deepspeed/deepspeed, CS = external/deepspeed/csrc,
 * EX = external/deepspeed/DeepSpeedExamples.
 *
 * Conventions: every function returns an int status (0 ok, >0 recoverable condition,
 * <0 caller error), takes raw device pointers and an explicit stream (a cudaStream_t
 * passed as void*), never allocates device memory, never synchronises the device and
 * never throws.  bb_last_error() describes the most recent failure on this thread.
 */
#ifndef BAMBOO_B200_H
#define BAMBOO_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BB_OK 0
#define BB_ERR_INVALID_ARG (-1)
#define BB_ERR_CUDA (-2)
#define BB_ERR_UNSUPPORTED (-3)
#define BB_ERR_TOO_LARGE (-4)
#define BB_STATUS_PEER_TIMEOUT 1        /* a bounded wait on a neighbour stage expired      */
#define BB_STATUS_KERNEL_WAIT_TIMEOUT 2 /* a bounded wait inside a kernel pipeline expired */

/* ---- library ------------------------------------------------------------------- */
int bb_version(void);
const char* bb_last_error(void);
/* Reads (synchronously) and clears the device status word kernels write when one of
 * their bounded waits runs out.  0 = healthy. */
int bb_read_status(int* out_status);

/* ---- GEMM ----------------------------------------------------------------------- */
enum {
  BB_EPI_STORE = 0,         /* D(bf16) = acc                                              */
  BB_EPI_BIAS = 1,          /* D(bf16) = acc + bias[n]                                    */
  BB_EPI_BIAS_GELU = 2,     /* D2(bf16) = acc + bias ; D(bf16) = gelu_tanh(D2)            */
  BB_EPI_ACCUM_F32 = 3,     /* D(f32) += acc                                              */
  BB_EPI_STORE_F32 = 4,     /* D(f32)  = acc                                              */
  BB_EPI_MUL_DGELU = 5,     /* D(bf16) = acc * gelu_tanh'(aux[m,n])                       */
  BB_EPI_BIAS_RESIDUAL = 6  /* D(bf16) = acc + bias[n] + aux[m,n]                         */
};

typedef struct bb_gemm_desc {
  int M, N, K;
  const void* A; long long lda; int a_mn_major; /* 0: A is [M,K] row-major; 1: stored [K,M] */
  const void* B; long long ldb; int b_mn_major; /* 0: B is [N,K] row-major; 1: stored [K,N] */
  void* D; long long ldd;
  int epilogue;
  const void* bias;                 /* bf16 [N]                                         */
  void* D2;                         /* second output of BB_EPI_BIAS_GELU, same ldd      */
  const void* aux; long long ld_aux;/* bf16 [M,N] operand of DGELU / RESIDUAL           */
  int tile_n;                       /* 0 = choose, else 128 or 256                      */
  int max_ctas;                     /* 0 = one persistent CTA per SM; > 0 = cap (leaves SMs to a concurrent stream);
                                       < 0 = one tile per CTA (short CTAs for a low-priority stream) */
  int split_k;                      /* BB_EPI_ACCUM_F32 only: 0 = choose, else number of K splits */
  int cta_pair;                     /* 0 = choose, 1 = CTA pairs (cta_group::2, 256 x 256 tiles), -1 = single CTAs */
  int epi_warps;                    /* epilogue warps per TMEM lane quarter: 0 = choose, 2, or 4 (bf16 outputs only) */
} bb_gemm_desc;

/* D[M,N] = op(A)[M,K] * op(B)[N,K]^T, bf16 operands, fp32 accumulation in tensor memory
 * (tcgen05.mma fed by TMA), fused epilogue.
 * Replaces: the nn.Linear / torch.matmul calls of the stage layers executed by
 * PipelineModule.forward (DS/runtime/pipe/module.py:516-574; layer bodies
 * EX/pipeline_parallelism/gpt2.py:66-121) and their autograd backward
 * (DS/runtime/pipe/engine.py:1680-1727), i.e. ATen -> cuBLAS GEMMs plus the separate
 * bias / activation / residual elementwise kernels. */
int bb_gemm_bf16(const bb_gemm_desc* desc, void* stream);

/* ---- LayerNorm -------------------------------------------------------------------- */
/* y = (x - mean) * rstd * gamma + beta over rows of h bf16 values; mean/rstd (fp32, per
 * row) are saved for the backward pass.  h % 8 == 0.
 * Replaces: the LayerNorm module of the reference transformer blocks, a chain of eager
 * mean/std/sub/div/mul/add kernels (EX/pipeline_parallelism/gpt2.py:20-32). */
int bb_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                     int rows, int h, float eps, void* stream);
/* dx = LN'(dy) (+ dres, the gradient arriving over the residual branch); dgamma/dbeta
 * (fp32) are accumulated (+=).  `workspace` holds per-CTA partial sums
 * (bb_layernorm_bwd_workspace_bytes) that a second kernel reduces in a fixed order.
 * Replaces: autograd's backward of the same module (DS/runtime/pipe/engine.py:1680-1727). */
long long bb_layernorm_bwd_workspace_bytes(int rows, int h);
int bb_layernorm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                     const void* dres, void* dx, float* dgamma, float* dbeta, void* workspace,
                     long long workspace_bytes, int rows, int h, void* stream);
/* The same, and dres_sum[h] (fp32) += the column sums of dres, from the same pass over dres.
 * In a pre-LayerNorm block out = x + Linear(...), so the gradient of `out` is both the residual
 * gradient of the block's LayerNorm and the row-wise gradient of that Linear's bias: its bias
 * gradient comes out of this call instead of a separate pass over `dres` (bb_colsum_accum).
 * dres and dres_sum are required; dx may alias dres.  Workspace:
 * bb_layernorm_bwd_res_workspace_bytes.
 * Replaces: the two autograd nodes above (LayerNorm backward and the bias-gradient reduction of
 * nn.Linear, EX/pipeline_parallelism/gpt2.py:20-32,52-64 via DS/runtime/pipe/engine.py:1680-1727). */
long long bb_layernorm_bwd_res_workspace_bytes(int rows, int h);
int bb_layernorm_bwd_res(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                         const void* dres, void* dx, float* dgamma, float* dbeta, float* dres_sum, void* workspace,
                         long long workspace_bytes, int rows, int h, void* stream);

/* LayerNorm backward for callers that must not allocate device memory - code running inside
 * a memory-pool callback, a fixed-footprint serving process, or any host that is not allowed to
 * call cudaMalloc once it is up.  Same arguments and results as bb_layernorm_bwd, minus the
 * workspace: the per-CTA partial sums go to an 8 MiB array built into the library's device
 * image (every GPU that loads the library holds it until the process exits).  This entry point
 * has no counterpart in the reference; it exists for those callers only.
 *  - Limit: bb_layernorm_bwd_workspace_bytes(rows, h) must not exceed
 *    bb_layernorm_bwd_static_capacity_bytes() (8 MiB; e.g. any row count up to h = 3456);
 *    larger problems return BB_ERR_TOO_LARGE and launch nothing.
 *  - The first call on a device resolves the array's device address (cudaGetSymbolAddress);
 *    make that first call outside any stream capture.  No call allocates or frees memory.
 *  - All calls on a device share the one array: two calls whose kernels may overlap on the
 *    GPU (different streams) race on it and must be ordered by the caller.  The array keeps
 *    the last call's partial sums; every call rewrites all it reads, nothing needs clearing. */
long long bb_layernorm_bwd_static_capacity_bytes(void);
int bb_layernorm_bwd_static(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd,
                            const void* dres, void* dx, float* dgamma, float* dbeta, int rows, int h, void* stream);

/* out[n] += sum_rows dy[row, n] : bias gradient of a linear layer (fp32 accumulate).  One
 * launch: per-CTA partial rows go to `workspace`, the CTA that finishes last for a block of 256
 * columns adds them in a fixed order (the result does not depend on scheduling).
 * Replaces: the bias-gradient reduction autograd runs for nn.Linear
 * (EX/pipeline_parallelism/gpt2.py:52-64 via DS/runtime/pipe/engine.py:1680-1727). */
long long bb_colsum_workspace_bytes(int rows, int n);
int bb_colsum_accum(const void* dy, long long ld, float* out, void* workspace, long long workspace_bytes,
                    int rows, int n, void* stream);

/* ---- embedding -------------------------------------------------------------------- */
/* out[t,:] = wte[tokens[t],:] + wpe[t % seq,:] (wpe may be NULL); gradient scatter into
 * fp32 dwte/dwpe.  The reference examples have no embedding (they train on random float
 * activations, EX/pipeline_parallelism/gpt2.py:283-295); the benchmark configurations add
 * token and learned position embeddings in front of stage 0, loaded by
 * _exec_load_micro_batch (DS/runtime/pipe/engine.py:1729-1779). */
int bb_embedding_fwd(const long long* tokens, const void* wte, const void* wpe, void* out, int n_tokens,
                     int seq, int h, int vocab, void* stream);
int bb_embedding_bwd(const long long* tokens, const void* dout, float* dwte, float* dwpe, int n_tokens, int seq,
                     int h, int vocab, void* stream);

/* ---- attention -------------------------------------------------------------------- */
/* softmax(scale * Q K^T [+ causal mask]) V without materialising the scores; q/k/v are
 * addressed as base + token*stride + head*D so a packed [tokens, 3*H*D] projection is
 * consumed in place.  lse: [B,H,S] fp32.  D in {64, 128}.
 * Replaces: the matmul / softmax / matmul chain of the reference attention
 * (EX/pipeline_parallelism/gpt2.py:66-75) and its autograd backward. */
int bb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int H, int S, int D,
                     long long stride_qkv, long long stride_o, int causal, float scale, void* stream);
/* Backward: dq, dk, dv in the layout of q, k, v.  The workspace holds the per-row sums delta and, for
 * head dimension 64, an fp32 accumulator [B, H, S, 64]: each CTA owns 128 keys, computes the scores
 * once and adds its dQ contributions with vector reductions, so dq can differ in the last bits
 * from run to run (the order of a row's additions is not fixed); dk and dv do not.
 * BB_ATTENTION_BWD=split in the environment selects kernels that keep every sum in a fixed order. */
long long bb_attention_bwd_workspace_bytes(int B, int H, int S);
int bb_attention_bwd(const void* q, const void* k, const void* v, const void* out, const void* d_out, const float* lse,
                     void* dq, void* dk, void* dv, void* workspace, long long workspace_bytes, int B, int H, int S,
                     int D, long long stride_qkv, long long stride_o, long long stride_dqkv, int causal, float scale,
                     void* stream);

/* ---- loss ------------------------------------------------------------------------- */
/* Token-level cross entropy over bf16 logits [rows, ld] with `vocab` valid columns:
 * lse/row_loss per row, loss_out[0] = mean over non-ignored rows, loss_out[1] = their count.
 * Replaces: loss_fn(outputs, labels) on the last stage (DS/runtime/pipe/engine.py:1650-1663). */
int bb_cross_entropy_fwd(const void* logits, long long ld, const long long* targets, float* lse, float* row_loss,
                         float* loss_out, int rows, int vocab, long long ignore_index, void* stream);
/* dlogits = (softmax - onehot) * grad_scale * (*grad_scale_dev, if given) / count, zero in
 * the padded columns vocab..cols; may run in place.
 * Replaces: the loss part of DeepSpeedEngine.backward (DS/runtime/engine.py:1416-1478). */
int bb_cross_entropy_bwd(const void* logits, long long ld, const long long* targets, const float* lse,
                         const float* loss_out, const float* grad_scale_dev, float grad_scale, void* dlogits,
                         long long ldd, int rows, int vocab, int cols, long long ignore_index, void* stream);

/* dx = dy * gelu'(pre) (tanh form), n bf16 elements, n a multiple of 8.  The activation gradient
 * where no GEMM follows to fuse it into: the masked-LM head transform (dense + GeLU +
 * LayerNorm) of the BERT-large configuration.  The reference runs this as ATen's GeLU backward
 * inside loss.backward() (DS/runtime/engine.py:1478); its own BERT example
 * (DeepSpeedExamples/pipeline_parallelism/bert.py:126-147) stops before the language-model head. */
int bb_gelu_bwd(const void* dy, const void* pre, void* dx, long long n, void* stream);

/* ---- whole transformer half-blocks ------------------------------------------------- */
/* One call issues every kernel of half a pre-LN transformer block, so the host pays for one
 * foreign call instead of one per kernel (the Python host of a pipeline stage otherwise spends
 * more time issuing a micro-batch than the GPU needs to run it).  Same kernels, same order and
 * same arithmetic as calling the entry points above one by one.
 *   attention half:  out = x + proj(attention(qkv(LN1(x))))
 *   MLP half:        out = x + fc2(gelu(fc1(LN2(x))))
 * `saved` (bb_block_saved_bytes) receives what the backward pass needs; the backward entry
 * points write dx, accumulate every weight / bias / LayerNorm gradient into the fp32 pointers of
 * the descriptor and use `scratch` (bb_block_scratch_bytes) for intermediates.  Weight gradients
 * are issued on `side_stream` behind an event recorded on `stream` (pass the same stream twice
 * to keep everything in order on one stream).
 * Replaces: one layer call of PipelineModule.forward (DS/runtime/pipe/module.py:516-574; block
 * body EX/pipeline_parallelism/gpt2.py:66-121) and its share of loss.backward()
 * (DS/runtime/pipe/engine.py:1680-1727). */
enum { BB_HALF_ATTENTION = 0, BB_HALF_MLP = 1 };
typedef struct bb_block_desc {
  int tokens, batch, seq, heads, head_dim, hidden, ffn, causal;
  float eps;
  int max_ctas;                      /* forwarded to every GEMM (see bb_gemm_desc.max_ctas) */
  /* bf16 parameters: LayerNorm gain/bias, then the two linear layers of the half
   * (attention: qkv [3h,h], proj [h,h]; MLP: fc1 [ffn,h], fc2 [h,ffn]) with their biases */
  const void *ln_w, *ln_b, *w1, *b1, *w2, *b2;
  /* fp32 gradient accumulators of the same parameters (backward only) */
  float *g_ln_w, *g_ln_b, *g_w1, *g_b1, *g_w2, *g_b2;
} bb_block_desc;
long long bb_block_saved_bytes(const bb_block_desc* d, int half);
long long bb_block_scratch_bytes(const bb_block_desc* d, int half);
int bb_block_half_fwd(const bb_block_desc* d, int half, const void* x, void* saved, void* out, void* stream);
int bb_block_half_bwd(const bb_block_desc* d, int half, const void* x, const void* saved, const void* dout, void* dx,
                      void* scratch, long long scratch_bytes, void* stream, void* side_stream);

/* ---- convolutional stages (channels-last) ----------------------------------------- */
/* ResNet-152 stage compute, bf16 NHWC.  A convolution is bb_gemm_bf16 over a patch matrix:
 * rows = output pixels (n, ho, wo), columns = (tap r, tap s, input channel), weight stored
 * [Cout, k, k, Cin]; a 1 x 1 / stride 1 convolution reads the activation tensor itself as that
 * matrix.  bb_im2col_nhwc builds the patch matrix (zero padding), bb_col2im_nhwc is its adjoint
 * (input gradient from the patch-matrix gradient; gather form, fixed summation order).  C and
 * ld_col (elements per patch-matrix row, >= k*k*C) are multiples of 8; Ho = (H + 2 pad - k) /
 * stride + 1.
 * Replaces: torch.nn.Conv2d forward / backward (cuDNN) of torchvision's resnet152 as split by
 * join_resnet_layers (EX/osdi22-cv/resnet-exp.py:69-83; blocks EX/pipeline_parallelism/resnet.py:49-171). */
int bb_im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                   long long ld_col, void* stream);
int bb_col2im_nhwc(const void* dcol, void* dx, int N, int H, int W, int C, int k, int stride, int pad, int Ho, int Wo,
                   long long ld_col, void* stream);
/* Batch normalisation with batch statistics over the rows of y [rows, C] (rows = N*H*W), C = 8 x
 * a power of two <= 2048: bb_bn_stats -> mean / rstd (biased variance); bb_bn_apply -> z = (y -
 * mean) * rstd * gamma + beta (+ residual) (ReLU if relu != 0); bb_bn_bwd takes dz, masks it with
 * z > 0 when relu, writes dy (gradient w.r.t. the convolution output), optionally dres (the
 * masked gradient, for the residual branch) and accumulates dgamma / dbeta (fp32).  `workspace`:
 * bb_bn_workspace_bytes(rows, C).  Replaces: nn.BatchNorm2d (training mode) + ReLU + the residual
 * add of the bottleneck blocks and their autograd backward.  Running statistics are not kept
 * (they do not enter the training step). */
long long bb_bn_workspace_bytes(long long rows, int C);
int bb_bn_stats(const void* y, long long rows, int C, float eps, float* mean, float* rstd, void* workspace,
                long long workspace_bytes, void* stream);
int bb_bn_apply(const void* y, const float* mean, const float* rstd, const void* gamma, const void* beta,
                const void* residual, void* z, long long rows, int C, int relu, void* stream);
int bb_bn_bwd(const void* dz, const void* z, const void* y, const float* mean, const float* rstd, const void* gamma,
              void* dy, void* dres, float* dgamma, float* dbeta, long long rows, int C, int relu, void* workspace,
              long long workspace_bytes, void* stream);
/* One call per layer: convolution + batch norm (+ residual, + ReLU), forward and backward, issuing
 * the kernels above in order (patch gather, GEMM, statistics, normalise / batch-norm backward,
 * patch gather, weight-gradient GEMM, input-gradient GEMM, adjoint gather).  y is the
 * convolution output kept for the backward pass, z the layer output; dx / dres may be NULL.
 * `scratch`: bb_conv_bn_scratch_bytes(desc, backward, need_dx).  Replaces one Conv2d + BatchNorm2d
 * (+ add + ReLU) of a bottleneck block and their share of loss.backward(). */
typedef struct bb_conv_desc {
  int N, H, W, Cin, Cout, k, stride, pad, relu;
  float eps;
  int max_ctas;                       /* forwarded to every GEMM (see bb_gemm_desc.max_ctas) */
  const void *w, *gamma, *beta;       /* bf16: weight [Cout, k, k, Cin], batch-norm gain and bias */
  float *g_w, *g_gamma, *g_beta;      /* fp32 gradient accumulators (backward only) */
} bb_conv_desc;
long long bb_conv_bn_scratch_bytes(const bb_conv_desc* d, int backward, int need_dx);
int bb_conv_bn_fwd(const bb_conv_desc* d, const void* x, const void* residual, void* y, void* z, float* mean, float* rstd,
                   void* scratch, long long scratch_bytes, void* stream);
int bb_conv_bn_bwd(const bb_conv_desc* d, const void* x, const void* y, const void* z, const float* mean, const float* rstd,
                   const void* dz, void* dx, void* dres, void* scratch, long long scratch_bytes, void* stream);
/* 3 x 3 / stride 2 / padding 1 max pooling (argmax: 1 byte per output element, position 0..8 in
 * the window, first maximum wins) and global average pooling over HW pixels.
 * Replaces: model.maxpool / model.avgpool of the same layer list. */
int bb_maxpool3x3s2_fwd(const void* x, void* y, void* argmax, int N, int H, int W, int C, void* stream);
int bb_maxpool3x3s2_bwd(const void* dy, const void* argmax, void* dx, int N, int H, int W, int C, void* stream);
int bb_avgpool_fwd(const void* x, void* y, int N, int HW, int C, void* stream);
int bb_avgpool_bwd(const void* dy, void* dx, int N, int HW, int C, void* stream);

/* ---- optimizer -------------------------------------------------------------------- */
/* One Adam / AdamW step over a flat parameter arena: fp32 master weights, gradient and
 * moments; refreshes the bf16 working copy (may be NULL) and optionally clears the
 * gradient in the same pass.  grad_scale multiplies the gradient first (1/dp averaging).
 * Replaces: FusedAdam.step (DS/ops/adam/fused_adam.py:85-182) ->
 * multi_tensor_adam (CS/adam/multi_tensor_adam.cu:28-163) and zero_grad
 * (DS/runtime/engine.py:1526-1573). */
int bb_adam_step(float* master, float* grad, float* exp_avg, float* exp_avg_sq, void* param_bf16, long long n,
                 float lr, float beta1, float beta2, float eps, int step, int adam_w_mode, int bias_correction,
                 float weight_decay, float grad_scale, int zero_grad, void* stream);
/* dst(bf16) = src(fp32); used when a shadow stage is promoted or refreshed
 * (PipelineModule.build_layers(stage, buffer), DS/runtime/pipe/module.py:262-332). */
int bb_cast_f32_to_bf16(const float* src, void* dst, long long n, void* stream);

/* ---- inter-stage transfer --------------------------------------------------------- */
/* Set-up (these four are the only entry points that allocate or map device memory; call
 * them when a channel to a neighbour is created, not per message): a receive mailbox in
 * this GPU's memory with its 64-byte CUDA-IPC handle, and the mapping of a neighbour's. */
int bb_ipc_alloc(long long bytes, void** dev_ptr, void* handle_out64);
int bb_ipc_open(const void* handle64, void** dev_ptr);
int bb_ipc_close(void* dev_ptr);
int bb_ipc_free(void* dev_ptr);
/* Store `bytes` from local `src` into the neighbour's mailbox slot `dst_peer`, then release
 * `seq` into the slot's flag (`flag_peer`, 8 bytes in the neighbour's memory).
 * `done_counter`: 4 zero-initialised bytes of local device memory owned by the channel.
 * Replaces: p2p.send (DS/runtime/pipe/p2p_direct.py:11-13) as used by _exec_send_activations
 * / _exec_send_grads (DS/runtime/pipe/engine.py:1894-1997) - NCCL send - and the shape
 * handshake _send_tensor_meta (engine.py:1781-1841). */
int bb_p2p_put(void* dst_peer, const void* src, long long bytes, void* flag_peer, unsigned long long seq,
               void* done_counter, void* stream);
/* Wait (at most timeout_ns) until the local flag equals `seq`, then copy the local slot to
 * `dst`.  On expiry BB_STATUS_PEER_TIMEOUT is recorded in `status_word` (NULL: the
 * library's status word, see bb_read_status) and nothing is copied.  bytes may be 0 (ping).
 * Replaces: p2p.recv (p2p_direct.py:15-17) + the clone in _exec_recv_activations /
 * _exec_recv_grads (engine.py:1999-2082); the bounded wait stands in for NCCL_BLOCKING_WAIT. */
int bb_p2p_wait_copy(const void* slot, void* dst, long long bytes, const void* flag, unsigned long long seq,
                     unsigned long long timeout_ns, int* status_word, void* stream);
/* Release `seq` into a neighbour's flag without payload: the liveness ping of lazy
 * redundancy (buffer_id = -1, engine.py:1902-1905). */
int bb_p2p_signal(void* flag_peer, unsigned long long seq, void* stream);
/* Several slots of one mailbox delivered all-or-nothing: waits until each of the `n`
 * consecutive 8-byte flags at `flags` holds `seq`, then copies slot i to dsts[i]
 * (bytes[i], multiples of 16).  If the limit expires first nothing is copied and
 * BB_STATUS_PEER_TIMEOUT is recorded, so the destination never mixes two messages.
 * Carries the end-of-step refresh of a shadow stage (weights, exp_avg, exp_avg_sq) - a
 * transfer the reference declares but leaves empty (SendWeights/RecvWeights,
 * DS/runtime/pipe/engine.py:2084-2137: _exec_recv_weights returns at :2110-2112). */
#define BB_P2P_MAX_PIECES 4
int bb_p2p_wait_copy_multi(const void* const* slots, void* const* dsts, const long long* bytes, int n,
                           const void* flags, unsigned long long seq, unsigned long long timeout_ns,
                           int* status_word, void* stream);
/* Completion record for the host without a stream synchronisation: when the stream reaches
 * this point, one 8-byte store writes (status_word << 32) | ticket into `host_word`
 * (pinned, device-visible host memory, see bb_pinned_alloc), which the caller polls.
 * Replaces the implicit host blocking of p2p.recv (DS/runtime/pipe/p2p_direct.py:15-17):
 * the engine learns that a receive landed - or timed out - before it issues dependent work. */
int bb_p2p_notify(void* host_word, unsigned int ticket, void* stream);
/* Pinned, device-visible host memory for such records (set-up time; zero-filled). */
int bb_pinned_alloc(long long bytes, void** host_ptr);
int bb_pinned_free(void* host_ptr);
/* Clears the device status word in stream order (after a recorded timeout was handled). */
int bb_clear_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BAMBOO_B200_H */
