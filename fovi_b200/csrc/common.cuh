// Shared host-side helpers of the fovi_b200 library (status, error capture, launch counter).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <atomic>
#include <string>

#include "../../include/fovi_b200.h"

namespace fovi {

extern thread_local std::string g_last_cuda_error;
extern std::atomic<int64_t> g_launch_count;

inline int cuda_fail(cudaError_t e, const char* what) {
  g_last_cuda_error = std::string(what) + ": " + cudaGetErrorString(e);
  return FOVI_ERR_CUDA;
}

#define FOVI_CUDA(call)                                         \
  do {                                                          \
    cudaError_t e__ = (call);                                   \
    if (e__ != cudaSuccess) return ::fovi::cuda_fail(e__, #call); \
  } while (0)

inline int after_launch(const char* name) {
  g_launch_count.fetch_add(1, std::memory_order_relaxed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, name);
  return FOVI_OK;
}

inline size_t dtype_size(int dt) { return dt == FOVI_BF16 ? 2 : 4; }
inline bool valid_dtype(int dt) { return dt == FOVI_F32 || dt == FOVI_BF16; }

// Number of SMs of the current device (cached per device id).
int sm_count();

}  // namespace fovi

// ---- device-side element access shared by the kernels
template <typename T> __device__ __forceinline__ float ld_as_float(const T* p);
template <> __device__ __forceinline__ float ld_as_float<float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld_as_float<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(__ldg(p));
}
template <> __device__ __forceinline__ float ld_as_float<unsigned char>(const unsigned char* p) { return (float)__ldg(p); }
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
