// Shared host/device helpers of the sm_100a library: status codes, error text, launch checks.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "smore_b200.h"

namespace smore {

constexpr int kWarp = 32;
constexpr int kNumSMFull = 148;  // a whole B200: 2 dies x 74 SMs

// Multiprocessors of the current device (148 on a whole B200, fewer on a partitioned one); grids
// are sized in multiples of this.  Queried once per device.
int sm_count();

// Opt a kernel in to `bytes` of dynamic shared memory (and, if asked, the largest shared-memory
// carve-out) once per (kernel, device); thread-safe.
int allow_large_smem_impl(const void* kernel, int bytes, bool max_carveout);
template <class Kernel>
inline int allow_large_smem(Kernel kern, int bytes, bool max_carveout = true) {
  return allow_large_smem_impl(reinterpret_cast<const void*>(kern), bytes, max_carveout);
}

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

// Bits of the device status word that smore_async_status reports.
constexpr int kStatusCopyWait = 1;   // a bounded wait for a bulk copy gave up (distance kernels)
constexpr int kStatusPeerWait = 2;   // the same in the background row pull
constexpr int kStatusBadRowId = 4;   // a caller-supplied row id lay outside the table
constexpr int kStatusCapacity = 8;   // more work arrived than a fixed-size buffer holds (owner-side scoring)

// Row ids come from the caller.  One outside [0, n_rows) must never become an address: the load
// uses row 0 instead, the caller of this helper invalidates what the id belongs to (forward: NaN
// for the pair; backward: no gradient from it) and kStatusBadRowId is set in `status`.  Returns
// the id, or -1 for a bad one.  n_rows == 0 disables the check.
__device__ __forceinline__ long long checked_row_id(const int64_t* idx, size_t pos, long long n_rows, int* status) {
  const long long r = idx[pos];
  if (n_rows > 0 && (unsigned long long)r >= (unsigned long long)n_rows) {
    atomicOr(status, kStatusBadRowId);
    return -1;
  }
  return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = kWarp / 2; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

}  // namespace smore
