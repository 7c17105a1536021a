// Bulk asynchronous copies (the TMA engine's untiled form) and the shared-memory
// barriers that track them, with bounded waits: a wait that runs out sets a
// status bit and gives up instead of hanging the GPU.
#pragma once

#include "common.cuh"

namespace mxb {

__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void barrier_init(uint64_t* barrier, int arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(shared_address(barrier)), "r"(arrivals) : "memory");
}

// Makes the initialised barriers visible to the asynchronous copy engine.
__device__ __forceinline__ void barrier_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
}

// One arrival that also announces `bytes` of copies to come.
__device__ __forceinline__ void barrier_arrive_expect(uint64_t* barrier, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(shared_address(barrier)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void barrier_arrive(uint64_t* barrier) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(shared_address(barrier)) : "memory");
}

// `bytes` (a multiple of 16) from global to shared memory, both 16-byte
// aligned; completion is counted on `barrier`.
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* barrier) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
               ::"r"(shared_address(dst)), "l"(src), "r"(bytes), "r"(shared_address(barrier)) : "memory");
}

constexpr int kBarrierSpins = 1 << 20;  // each try already waits a while in hardware

// Waits for the phase of parity `parity` to complete. False (and a status
// bit) if it does not within the spin limit.
__device__ __forceinline__ bool barrier_wait(uint64_t* barrier, uint32_t parity, int* status) {
  const uint32_t address = shared_address(barrier);
  for (int spin = 0; spin < kBarrierSpins; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done) : "r"(address), "r"(parity) : "memory");
    if (done) return true;
  }
  atomicOr(status, kStatusWaitTimeout);
  return false;
}

}  // namespace mxb
