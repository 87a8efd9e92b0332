// Shared host/device helpers of the sm_100a library: status codes, error text, launch checks.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "smore_b200.h"

namespace smore {

constexpr int kWarp = 32;
constexpr int kNumSM = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this

char* last_error_buffer();
void count_launches(int n);  // kernels of this library enqueued so far (smore_kernel_launch_count)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int check_launch(const char* what, int kernels = 1) {
  count_launches(kernels);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(SMORE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return SMORE_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = kWarp / 2; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

}  // namespace smore
