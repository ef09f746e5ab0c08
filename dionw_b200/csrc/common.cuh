// Shared helpers for the dionw_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/dionw_b200.h"

namespace dionw {

// Records the message returned by dionw_last_error() for the calling thread.
void set_error(const char* fmt, ...);

// Device-side status word: 0 while every bounded wait inside a kernel ended
// normally.  A kernel whose wait ran out stores a non-zero code here and leaves
// through its normal teardown path (no trap, the context stays usable).
int* device_status_word();

inline int check_cuda(cudaError_t err, const char* what) {
  if (err == cudaSuccess) return DIONW_OK;
  set_error("%s: %s", what, cudaGetErrorString(err));
  return DIONW_ERR_CUDA;
}

#define DIONW_CUDA(expr)                                   \
  do {                                                     \
    int _status = ::dionw::check_cuda((expr), #expr);      \
    if (_status != DIONW_OK) return _status;               \
  } while (0)

#define DIONW_REQUIRE(cond, ...)                           \
  do {                                                     \
    if (!(cond)) {                                         \
      ::dionw::set_error(__VA_ARGS__);                     \
      return DIONW_ERR_ARGUMENT;                           \
    }                                                      \
  } while (0)

// Adds one to the library's count of kernel launches (dionw_launch_count()).
void count_launch();

inline int launch_status(const char* what) {
  count_launch();
  return check_cuda(cudaGetLastError(), what);
}

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

}  // namespace dionw
