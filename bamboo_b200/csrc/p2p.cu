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

// Several slots of one mailbox delivered all-or-nothing: wait (bounded) until EVERY flag holds
// seq, then copy every slot out.  If one is missing when the limit expires nothing is copied,
// so the destination never holds pieces of two different messages.
struct MultiCopy {
  const uint4* slot[BB_P2P_MAX_PIECES];
  uint4* dst[BB_P2P_MAX_PIECES];
  long long n16[BB_P2P_MAX_PIECES];
  int n;
};

__global__ void __launch_bounds__(256)
wait_copy_multi_kernel(MultiCopy mc, const unsigned long long* flags, unsigned long long seq, unsigned long long timeout_ns,
                       int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 0;
    const unsigned long long t0 = bb::globaltimer_ns();
    unsigned int backoff = 32;
    for (;;) {
      bool all = true, ahead = false;
      for (int i = 0; i < mc.n; ++i) {
        const unsigned long long v = ld_acquire_sys_u64(flags + i);
        all = all && (v == seq);
        ahead = ahead || (v > seq);
      }
      if (all) { ok = 1; break; }
      if (ahead || bb::globaltimer_ns() - t0 > timeout_ns) {
        atomicCAS(status, 0, ahead ? BB_ERR_INVALID_ARG : BB_STATUS_PEER_TIMEOUT);
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
  for (int p = 0; p < mc.n; ++p)
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < mc.n16[p]; i += stride) mc.dst[p][i] = mc.slot[p][i];
}

// Completion record for the host: one 8-byte store into pinned host memory that the caller
// polls instead of synchronising with the stream.  Low half = the caller's ticket, high half =
// the device status word at that point of the stream (0 = every wait so far was answered).
__global__ void notify_kernel(unsigned long long* host_word, unsigned int ticket, const int* status) {
  const unsigned long long st = (unsigned long long)(unsigned int)(*status);
  __threadfence_system();
  *reinterpret_cast<volatile unsigned long long*>(host_word) = (st << 32) | ticket;
  __threadfence_system();
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

extern "C" int bb_p2p_wait_copy_multi(const void* const* slots, void* const* dsts, const long long* bytes, int n,
                                      const void* flags, unsigned long long seq, unsigned long long timeout_ns,
                                      int* status_word, void* stream) {
  if (!status_word) status_word = bb_device_status_word();
  if (!slots || !dsts || !bytes || !flags || !status_word || n < 1 || n > BB_P2P_MAX_PIECES || ((uintptr_t)flags & 7)) {
    bb_set_last_error_msg("bb_p2p_wait_copy_multi: null pointer or piece count outside 1..BB_P2P_MAX_PIECES");
    return BB_ERR_INVALID_ARG;
  }
  MultiCopy mc;
  mc.n = n;
  long long most = 0;
  for (int i = 0; i < BB_P2P_MAX_PIECES; ++i) { mc.slot[i] = nullptr; mc.dst[i] = nullptr; mc.n16[i] = 0; }
  for (int i = 0; i < n; ++i) {
    if (!slots[i] || !dsts[i] || bytes[i] <= 0 || (bytes[i] & 15) || (((uintptr_t)slots[i] | (uintptr_t)dsts[i]) & 15)) {
      bb_set_last_error_msg("bb_p2p_wait_copy_multi: null/unaligned piece or size not a multiple of 16 bytes");
      return BB_ERR_INVALID_ARG;
    }
    mc.slot[i] = (const uint4*)slots[i]; mc.dst[i] = (uint4*)dsts[i]; mc.n16[i] = bytes[i] >> 4;
    if (mc.n16[i] > most) most = mc.n16[i];
  }
  if (timeout_ns > 120000000000ull) timeout_ns = 120000000000ull;
  wait_copy_multi_kernel<<<copy_grid(most), 256, 0, (cudaStream_t)stream>>>(mc, (const unsigned long long*)flags, seq,
                                                                            timeout_ns, status_word);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_p2p_notify(void* host_word, unsigned int ticket, void* stream) {
  int* status_word = bb_device_status_word();
  if (!host_word || ((uintptr_t)host_word & 7) || !status_word) {
    bb_set_last_error_msg("bb_p2p_notify: null or unaligned host word");
    return BB_ERR_INVALID_ARG;
  }
  notify_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((unsigned long long*)host_word, ticket, status_word);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}

extern "C" int bb_pinned_alloc(long long bytes, void** host_ptr) {
  if (bytes <= 0 || !host_ptr) { bb_set_last_error_msg("bb_pinned_alloc: bad argument"); return BB_ERR_INVALID_ARG; }
  void* p = nullptr;
  BB_CUDA_CHECK(cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(p, 0, (size_t)bytes);
  *host_ptr = p;
  return BB_OK;
}

extern "C" int bb_pinned_free(void* host_ptr) {
  if (host_ptr) BB_CUDA_CHECK(cudaFreeHost(host_ptr));
  return BB_OK;
}

extern "C" int bb_clear_status(void* stream) {
  int* status_word = bb_device_status_word();
  if (!status_word) { bb_set_last_error_msg("bb_clear_status: no current device"); return BB_ERR_CUDA; }
  BB_CUDA_CHECK(cudaMemsetAsync(status_word, 0, sizeof(int), (cudaStream_t)stream));
  return BB_OK;
}

extern "C" int bb_p2p_signal(void* flag_peer, unsigned long long seq, void* stream) {
  if (!flag_peer || ((uintptr_t)flag_peer & 7)) { bb_set_last_error_msg("bb_p2p_signal: bad flag pointer"); return BB_ERR_INVALID_ARG; }
  signal_kernel<<<1, 1, 0, (cudaStream_t)stream>>>((unsigned long long*)flag_peer, seq);
  BB_CUDA_CHECK(cudaGetLastError());
  return BB_OK;
}
