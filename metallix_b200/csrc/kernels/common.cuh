// Shared device helpers for the hand-written kernels: element types, loads
// that widen to float, warp and block reductions with a fixed order.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mxb {

// Element type codes of the C interface.
enum DType : int { kF32 = 0, kBF16 = 1 };

// Bits of the device status word that kernels set instead of trapping.
enum StatusBit : int {
  kStatusBadTokenId = 1,    // a token id outside the vocabulary
  kStatusBadSlot = 2,       // a cache slot outside the pool
  kStatusBadPage = 4,       // a block-table entry outside the pool
  kStatusNonFinite = 8,     // a non-finite logit where a token was picked
  kStatusWaitTimeout = 16,  // a bounded wait (mbarrier) ran out
};

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. The
// order of additions depends only on the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < warps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Programmatic dependent launch: a kernel launched through launch_chained()
// may start while its predecessor in the stream is still running. It calls
// chain_wait() before it touches anything the predecessor writes (the wait
// returns once the predecessor has finished and its writes are visible), and
// chain_release() as early as it likes to let its own successor start. What
// runs before the wait (index arithmetic, fetching weights no kernel writes)
// overlaps the predecessor. Without the launch attribute both are no-ops.
#ifndef MXB_TIMELINE
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#define MXB_TIMELINE_EXPORT(name)
#else
// A build with -DMXB_TIMELINE (METALLIX_B200_TIMELINE=1) records when the
// first thread of the first block of every chained kernel got past its wait,
// i.e. when the kernel ahead of it had finished: the differences are the time
// each kernel holds the chain, measured on the device while the step runs as
// it always does (captured graph, overlapped launches). Every source file has
// counters of its own, read through the function MXB_TIMELINE_EXPORT defines.
constexpr unsigned kTimelineSlots = 8192;
static __device__ unsigned long long timeline_times[kTimelineSlots];
static __device__ unsigned timeline_count;
__device__ __forceinline__ void chain_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    const unsigned slot = atomicAdd(&timeline_count, 1u);
    if (slot < kTimelineSlots) timeline_times[slot] = now;
  }
}
// int name(unsigned long long* out, int reset): copies the recorded times (ns)
// to `out` (room for 8192, may be null), optionally clears them, returns how many.
#define MXB_TIMELINE_EXPORT(name)                                                                        \
  extern "C" __attribute__((visibility("default"))) int name(unsigned long long* out, int reset) {       \
    unsigned count = 0;                                                                                  \
    cudaMemcpyFromSymbol(&count, mxb::timeline_count, sizeof(count));                                    \
    if (count > mxb::kTimelineSlots) count = mxb::kTimelineSlots;                                        \
    if (out != nullptr && count > 0)                                                                     \
      cudaMemcpyFromSymbol(out, mxb::timeline_times, count * sizeof(unsigned long long));                \
    if (reset) {                                                                                         \
      const unsigned zero = 0;                                                                           \
      cudaMemcpyToSymbol(mxb::timeline_count, &zero, sizeof(zero));                                      \
    }                                                                                                    \
    return static_cast<int>(count);                                                                      \
  }
#endif
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A kernel that launch_chained() starts lives before the kernel ahead of it
// has written its output, so the promise a const __restrict__ parameter makes
// (nobody changes this memory while the kernel runs) does not hold for that
// output, and the compiler, trusting it, may move a load above chain_wait().
// behind_wait(), called after chain_wait(), gives the pointer back with that
// promise taken off: loads through the result stay behind the wait.
template <typename T> __device__ __forceinline__ T* behind_wait(T* p) {
  asm volatile("" : "+l"(p));
  return p;
}

bool chained_launches();      // whether launch_chained() asks for the overlap (csrc/kernels/embed_norm.cu)
unsigned chained_block_limit();            // ... for grids of up to this many blocks
unsigned long long chained_byte_limit();   // ... and kernels that stream up to this many bytes

// Whether a launch of `grid` that reads `bytes` (0: not known, small) asks for
// the overlap. The overlap pays where a kernel is short: it hides the start-up
// and lets weights be fetched ahead. A kernel that streams tens of megabytes
// gains nothing from starting a few microseconds early, and a step made of
// such kernels ran a third slower with the overlap than without (the layers
// of an 8B- or 32B-shaped model at 1 to 8 rows), so those are launched the
// ordinary way.
inline bool chain_this(dim3 grid, unsigned long long bytes = 0) {
  return chained_launches() && bytes <= chained_byte_limit() &&
         static_cast<unsigned long long>(grid.x) * grid.y * grid.z <= chained_block_limit();
}

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chained_sized(unsigned long long bytes, void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                                        size_t shared, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = chain_this(grid, bytes) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared,
                                  cudaStream_t stream, Args... args) {
  return launch_chained_sized(0ull, kernel, grid, block, shared, stream, args...);
}

// The same for a kernel whose blocks run as clusters of `cluster_x` along x
// (grid.x a multiple of it): the blocks of a cluster are resident together and
// read one another's shared memory.
template <typename... KernelArgs, typename... Args>
inline cudaError_t launch_chained_clusters(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t shared,
                                           unsigned cluster_x, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster_x;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = chain_this(grid) ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

}  // namespace mxb

#define MXB_API extern "C" __attribute__((visibility("default")))
