// Copies whole pages (or state slots) inside a pool: what a forked request
// needs of its parent's partly filled last page. The reference copies a shared
// partial block before a sequence writes into it
// (crates/core/engine/src/manager.rs:749-763, the copy itself being the
// caller's); here the copy is one launch over every entry (layer) of the group.
//
// The pool is [entries, units, unit_bytes]: a unit is a page of one layer
// (keys and values of every head) or one request's slot of a state tensor.
#include "common.cuh"

namespace mxb {

// Block (pair, entry) copies unit pairs[pair].x to unit pairs[pair].y of one
// entry, in the widest words the unit's size and the pool's address allow.
template <typename Word>
__global__ void __launch_bounds__(256) copy_units_kernel(
    unsigned char* __restrict__ pool, const int2* __restrict__ pairs, long long unit_bytes, int units,
    int* __restrict__ status) {
  const int2 pair = pairs[blockIdx.x];
  if (pair.x < 0 || pair.x >= units || pair.y < 0 || pair.y >= units) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadPage);
    return;
  }
  if (pair.x == pair.y) return;
  unsigned char* entry = pool + static_cast<size_t>(blockIdx.y) * units * unit_bytes;
  const Word* from = reinterpret_cast<const Word*>(entry + static_cast<size_t>(pair.x) * unit_bytes);
  Word* to = reinterpret_cast<Word*>(entry + static_cast<size_t>(pair.y) * unit_bytes);
  const long long words = unit_bytes / static_cast<long long>(sizeof(Word));
  for (long long i = threadIdx.x; i < words; i += blockDim.x) to[i] = from[i];
}

}  // namespace mxb

using namespace mxb;

// pool: [entries, units, unit_bytes] bytes on the device; pairs: [count] (source
// unit, target unit) on the device. Source and target units of one call must
// not overlap each other's targets (a target is never another pair's source).
MXB_API int mxb_copy_units(void* pool, int entries, int units, long long unit_bytes, const void* pairs,
                           int count, int* status, cudaStream_t stream) {
  if (count <= 0 || entries <= 0 || unit_bytes <= 0) return 0;
  if (entries > 65535) return static_cast<int>(cudaErrorInvalidValue);
  unsigned char* bytes = static_cast<unsigned char*>(pool);
  const int2* list = static_cast<const int2*>(pairs);
  const dim3 grid(static_cast<unsigned>(count), static_cast<unsigned>(entries));
  const uintptr_t address = reinterpret_cast<uintptr_t>(pool);
  if (unit_bytes % 16 == 0 && address % 16 == 0)
    copy_units_kernel<uint4><<<grid, 256, 0, stream>>>(bytes, list, unit_bytes, units, status);
  else if (unit_bytes % 4 == 0 && address % 4 == 0)
    copy_units_kernel<uint32_t><<<grid, 256, 0, stream>>>(bytes, list, unit_bytes, units, status);
  else
    copy_units_kernel<unsigned char><<<grid, 256, 0, stream>>>(bytes, list, unit_bytes, units, status);
  return static_cast<int>(cudaGetLastError());
}
