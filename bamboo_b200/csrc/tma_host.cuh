// Host-side helper shared by the TMA kernels: encode a 2-D tensor map (128-byte swizzle)
// through the driver entry point, resolved at run time so the library has no link-time
// dependency on libcuda.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <stdio.h>

namespace bbhost {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

// The driver call needs a context bound to the calling thread; a thread that has only ever
// set its device (autograd worker threads) has none yet.
inline int bind_context() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaError_t e = cudaFree(0);
    if (e != cudaSuccess) { bb_set_last_error("cudaFree(0)", e); return BB_ERR_CUDA; }
    bound = true;
  }
  return BB_OK;
}

// 2-D tensor map over a row-major [rows, cols] matrix (bf16, or fp32 when f32 != 0) with leading
// dimension ld (elements); box = box_cols x box_rows; 128-byte swizzle.
inline int encode_2d(CUtensorMap* tm, const void* base, long long rows, long long cols, long long ld, int box_cols,
                     int box_rows, int f32 = 0) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) { bb_set_last_error_msg("cuTensorMapEncodeTiled entry point not available"); return BB_ERR_CUDA; }
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * (f32 ? 4 : 2)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char msg[256];
    snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed with CUresult %d (base %p, rows %lld, cols %lld, ld %lld, box %dx%d, "
             "f32 %d); operands need a 16-byte aligned base and row pitch", (int)r, base, rows, cols, ld, box_cols, box_rows, f32);
    bb_set_last_error_msg(msg);
    return BB_ERR_INVALID_ARG;
  }
  return BB_OK;
}

}  // namespace bbhost
