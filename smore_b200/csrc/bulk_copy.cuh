// Bulk asynchronous copies (the TMA engine's untiled form) and the mbarrier calls that track
// them, as inline PTX for sm_100a.  A copy moves one contiguous run of bytes between global and
// shared memory: both addresses 16-byte aligned, size a multiple of 16 bytes.  One thread issues
// it; completion of a load is signalled on an mbarrier in shared memory (transaction bytes),
// completion of a store through the issuing thread's bulk group.
//
// Every wait here is bounded: a wait that does not complete within kWaitCycles gives up and the
// caller records it in a status word instead of spinning on.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace smore {
namespace bulk {

constexpr long long kWaitCycles = 2000000000LL;  // about one second of SM clock

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void barrier_init(uint64_t* bar, unsigned arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// makes freshly initialised barriers visible to the copy engine
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// orders this thread's earlier shared-memory writes before later bulk copies that read them
__device__ __forceinline__ void fence_async_shared() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// one arrival that also announces `bytes` of copy traffic to wait for
__device__ __forceinline__ void barrier_expect(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void load(void* smem_dst, const void* gmem_src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

__device__ __forceinline__ void store(void* gmem_dst, const void* smem_src, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}

// element-wise fp32 add of a shared-memory run into global memory
__device__ __forceinline__ void reduce_add_f32(void* gmem_dst, const void* smem_src, unsigned bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// waits until at most N of this thread's bulk groups still READ their shared-memory source
template <int N>
__device__ __forceinline__ void wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

template <int N>
__device__ __forceinline__ void wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ bool barrier_try_wait(uint64_t* bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// true when the barrier's phase with the given parity completed; false after kWaitCycles
__device__ __forceinline__ bool barrier_wait(uint64_t* bar, unsigned parity) {
  if (barrier_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (!barrier_try_wait(bar, parity)) {
    if (clock64() - t0 > kWaitCycles) return false;   // (a __nanosleep back-off here measured slower)
  }
  return true;
}

}  // namespace bulk
}  // namespace smore
