// Library plumbing: version, per-thread error text, the device status word that kernels
// write when a bounded wait expires, cached device properties.
#include "common.cuh"
#include <stdio.h>
#include <string.h>

namespace {
thread_local char g_err[512] = "";
__device__ int g_status_word = 0;
}  // namespace

void bb_set_last_error(const char* what, cudaError_t e) {
  snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
}
void bb_set_last_error_msg(const char* msg) {
  strncpy(g_err, msg, sizeof(g_err) - 1);
  g_err[sizeof(g_err) - 1] = 0;
}

int* bb_device_status_word() {
  // resolved once per device; the symbol itself is only a host-side handle
  static int* ptr[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    ptr[dev] = static_cast<int*>(p);
  }
  return ptr[dev];
}

int bb_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -1;
  return dev;
}

int bb_num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!sms[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    sms[dev] = n;
  }
  return sms[dev];
}

extern "C" int bb_version(void) { return 100; }
extern "C" const char* bb_last_error(void) { return g_err; }

extern "C" int bb_read_status(int* out_status) {
  if (!out_status) return BB_ERR_INVALID_ARG;
  int v = 0;
  BB_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)));
  if (v != 0) {
    int zero = 0;
    BB_CUDA_CHECK(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
  }
  *out_status = v;
  return BB_OK;
}
