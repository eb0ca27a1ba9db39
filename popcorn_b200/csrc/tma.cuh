// Bulk asynchronous copies (the 1-D form of the Tensor Memory Accelerator) and
// the mbarrier objects they complete on.  Only this CTA's own shared memory is
// ever a destination; no copy in this library is addressed to several CTAs.
//
// Alignment: both addresses and the size of a bulk copy must be multiples of
// 16 bytes; the callers check that on the host before choosing a kernel that
// uses these helpers.
//
// Every wait is bounded: a waiter gives up after kSpinLimit probes and the
// kernel then takes a slower path that does not depend on the copy (and counts
// the event in g_wait_timeouts) instead of spinning forever.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// Incremented by any kernel of the including source file whose bounded wait ran
// out (one counter per source file: the library is built without relocatable
// device code).  b200_wait_timeouts() adds the counters up.
static __device__ unsigned int g_wait_timeouts = 0;

// Host side: current value of this source file's counter (synchronises the device).
static inline unsigned int read_wait_timeouts() {
  unsigned int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_wait_timeouts, sizeof(value)) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return value;
}

constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// Makes freshly initialised barriers visible to the asynchronous proxy.
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// One arrival plus the number of bytes the barrier should expect from bulk copies.
__device__ __forceinline__ void mbar_arrive_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Returns false if the phase did not complete within kSpinLimit probes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicAdd(&g_wait_timeouts, 1u);
  return false;
}

// global -> this CTA's shared memory, completion counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// this CTA's shared memory -> global, tracked by the issuing thread's bulk groups.
__device__ __forceinline__ void bulk_store(void* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gmem_dst), "r"(smem_addr(smem_src)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }

// Blocks until at most N of this thread's committed bulk-store groups still READ shared memory.
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Blocks until at most N of this thread's committed bulk-store groups are incomplete.
template <int N>
__device__ __forceinline__ void bulk_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// Orders this thread's ordinary shared-memory writes before later asynchronous-proxy reads.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

}  // namespace b200
