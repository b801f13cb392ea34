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
  int max_ctas;                     /* 0 = one per SM; else cap (leaves SMs to a concurrent stream) */
} bb_gemm_desc;

/* D[M,N] = op(A)[M,K] * op(B)[N,K]^T, bf16 operands, fp32 accumulation in tensor memory
 * (tcgen05.mma fed by TMA), fused epilogue.
 * Replaces: the nn.Linear / torch.matmul calls of the stage layers executed by
 * PipelineModule.forward (DS/runtime/pipe/module.py:516-574; layer bodies
 * EX/pipeline_parallelism/gpt2.py:66-121) and their autograd backward
 * (DS/runtime/pipe/engine.py:1680-1727), i.e. ATen -> cuBLAS GEMMs plus the separate
 * bias / activation / residual elementwise kernels. */
int bb_gemm_bf16(const bb_gemm_desc* desc, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BAMBOO_B200_H */
