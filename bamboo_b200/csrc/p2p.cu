// Inter-stage transfer over NVLink without NCCL: the sender stores the payload straight into
// the neighbour's receive mailbox (a CUDA-IPC mapping of the neighbour's memory) with
// 16-byte vector stores and then releases a sequence flag; the receiver waits - for a bounded
// time - on the flag in its own memory and copies the slot out.  Loads never touch peer
// memory; only plain stores cross the link.
#include "common.cuh"
#include <string.h>

namespace {

__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// dst (peer memory) <- src (local); the CTA that finishes last publishes the flag.
__global__ void __launch_bounds__(256)
put_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n16, unsigned long long* flag,
           unsigned long long seq, unsigned int* done_counter) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;  // ready for the next launch on this stream
      __threadfence_system();
      st_release_sys_u64(flag, seq);
    }
  }
}

// Wait until *flag == seq (bounded), then dst <- slot.  On timeout the status word (host
// visible) is set and nothing is copied.
__global__ void __launch_bounds__(256)
wait_copy_kernel(const uint4* __restrict__ slot, uint4* __restrict__ dst, long long n16, const unsigned long long* flag,
                 unsigned long long seq, unsigned long long timeout_ns, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 0;
    const unsigned long long t0 = bb::globaltimer_ns();
    unsigned int backoff = 32;
    for (;;) {
      const unsigned long long v = ld_acquire_sys_u64(flag);
      // a payload slot must hold exactly this message; a liveness ping (no payload) is a counter
      // that the sender may already have advanced past the one awaited
      if (v == seq || (n16 == 0 && v > seq)) { ok = 1; break; }
      if (bb::globaltimer_ns() - t0 > timeout_ns) {
        atomicCAS(status, 0, v > seq ? BB_ERR_INVALID_ARG : BB_STATUS_PEER_TIMEOUT);
        __threadfence_system();
        break;
      }
      __nanosleep(backoff);
      if (backoff < 2048) backoff <<= 1;
    }
  }
  __syncthreads();
  if (!ok) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) dst[i] = slot[i];
}

__global__ void signal_kernel(unsigned long long* flag, unsigned long long seq) {
  __threadfence_system();
  st_release_sys_u64(flag, seq);
}

int copy_grid(long long n16) {
  long long want = (n16 + 256 * 8 - 1) / (256 * 8);
  long long cap = bb_num_sms();
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace

extern "C" int bb_ipc_alloc(long long bytes, void** dev_ptr, void* handle_out64) {
  if (bytes <= 0 || !dev_ptr || !handle_out64) { bb_set_last_error_msg("bb_ipc_alloc: bad argument"); return BB_ERR_INVALID_ARG; }
  void* p = nullptr;
  BB_CUDA_CHECK(cudaMalloc(&p, (size_t)bytes));
  BB_CUDA_CHECK(cudaMemset(p, 0, (size_t)bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) { cudaFree(p); bb_set_last_error("cudaIpcGetMemHandle", e); return BB_ERR_CUDA; }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  memcpy(handle_out64, &h, 64);
  *dev_ptr = p;
  return BB_OK;
}

extern "C" int bb_ipc_open(const void* handle64, void** dev_ptr) {
  if (!handle64 || !dev_ptr) { bb_set_last_error_msg("bb_ipc_open: bad argument"); return BB_ERR_INVALID_ARG; }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  BB_CUDA_CHECK(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return BB_OK;
}

extern "C" int bb_ipc_close(void* dev_ptr) {
  if (dev_ptr) BB_CUDA_CHECK(cudaIpcCloseMemHandle(dev_ptr));
  return BB_OK;
}

extern "C" int bb_ipc_free(void* dev_ptr) {
  if (dev_ptr) BB_CUDA_CHECK(cudaFree(dev_ptr));
  return BB_OK;
}

extern "C" int bb_p2p_put(void* dst_peer, const void* src, long long bytes, void* flag_peer, unsigned long long seq,
                          void* done_counter, void* stream) {
  if (!dst_peer || !src || !flag_peer || !done_counter || bytes <= 0 || (bytes & 15) ||
      (((uintptr_t)dst_peer | (uintptr_t)src) & 15) || ((uintptr_t)flag_peer & 7)) {
    bb_set_last_error_msg("bb_p2p_put: null/unaligned pointer or size not a multiple of 16 bytes");
    return BB_ERR_INVALID_ARG;
  }
  const long long n16 = bytes >> 4;
  put_kernel<<<copy_grid(n16), 256, 0, (cudaStream_t)stream>>>((uint4*)dst_peer, (const uint4*)src, n16,
                                                               (unsigned long long*)flag_peer, seq, (unsigned int*)done_counter);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_p2p_wait_copy(const void* slot, void* dst, long long bytes, const void* flag, unsigned long long seq,
                                unsigned long long timeout_ns, int* status_word, void* stream) {
  if (!status_word) status_word = bb_device_status_word();
  if (!flag || !status_word || bytes < 0 || (bytes & 15) || (bytes > 0 && (!slot || !dst)) ||
      (((uintptr_t)slot | (uintptr_t)dst) & 15) || ((uintptr_t)flag & 7)) {
    bb_set_last_error_msg("bb_p2p_wait_copy: null/unaligned pointer or size not a multiple of 16 bytes");
    return BB_ERR_INVALID_ARG;
  }
  if (timeout_ns > 120000000000ull) timeout_ns = 120000000000ull;
  const long long n16 = bytes >> 4;
  wait_copy_kernel<<<copy_grid(n16), 256, 0, (cudaStream_t)stream>>>((const uint4*)slot, (uint4*)dst, n16,
                                                                     (const unsigned long long*)flag, seq, timeout_ns, status_word);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_p2p_signal(void* flag_peer, unsigned long long seq, void* stream) {
  if (!flag_peer || ((uintptr_t)flag_peer & 7)) { bb_set_last_error_msg("bb_p2p_signal: bad flag pointer"); return BB_ERR_INVALID_ARG; }
  signal_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((unsigned long long*)flag_peer, seq);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
