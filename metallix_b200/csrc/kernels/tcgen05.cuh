// The pieces every tcgen05 kernel here is made of: TMA tile loads, shared-
// memory matrix descriptors and instruction descriptors, the MMA, commit, and
// tensor-memory load/store instructions as inline PTX, and the host helper
// that encodes (and keeps) TMA tensor maps.
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "async_copy.cuh"
#include "common.cuh"

namespace mxb {

constexpr int kTmaColumns = 64;  // bfloat16 per TMA box row: one 128-byte swizzle row

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* barrier) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
               ::"r"(shared_address(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(shared_address(barrier)),
                 "r"(x), "r"(y) : "memory");
}

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle:
// rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t tc_smem_descriptor(uint32_t address) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((address >> 4) & 0x3FFF);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                   // leading byte offset (unused with a swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;           // stride between 8-row groups
  d |= static_cast<uint64_t>(1) << 46;                   // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                   // 128-byte swizzle
  return d;
}

// Instruction descriptor: bfloat16 x bfloat16 -> float32, both operands K-major.
__host__ __device__ constexpr uint32_t tc_instruction_descriptor(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n"
      "}\n"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// The barrier gets one arrival when every MMA issued so far has finished.
__device__ __forceinline__ void tc_commit(uint64_t* barrier) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
               ::"r"(shared_address(barrier)) : "memory");
}

__device__ __forceinline__ void tc_load_32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void tc_load_16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_load(uint32_t taddr, uint32_t (&r)[32]) { tc_load_32(taddr, r); }
__device__ __forceinline__ void tc_load(uint32_t taddr, uint32_t (&r)[16]) { tc_load_16(taddr, r); }

// The same for an MN-major tile (the contracted index runs over rows): rows of
// 64 contiguous values of the free index (128 bytes), 8 rows to a 1024-byte
// group, groups one after the other; the next 64 values of the free index lie
// `free_stride` bytes further.
__device__ __forceinline__ uint64_t tc_smem_descriptor_mn(uint32_t address, uint32_t free_stride) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((address >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((free_stride >> 4) & 0x3FFF) << 16;  // leading byte offset: between 64-value blocks
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                     // stride between groups of 8 rows
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// As tc_instruction_descriptor, with B MN-major.
__host__ __device__ constexpr uint32_t tc_instruction_descriptor_b_mn(int m, int n) {
  return tc_instruction_descriptor(m, n) | (1u << 16);
}

// D[tmem] (+)= A[tmem] * B[smem]: A is read from tensor memory, one row per
// lane, two bfloat16 per 32-bit column.
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n"
      "}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}

// 16 registers of this thread to 16 columns of its lane of tensor memory.
__device__ __forceinline__ void tc_store_16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};\n"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tc_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiled encode_tiled() {
  static EncodeTiled function = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* symbol = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess)
      function = reinterpret_cast<EncodeTiled>(symbol);
  });
  return function;
}

inline bool encode_map(CUtensorMap* map, const void* base, int rows, int k, long long ld, int box_rows) {
  EncodeTiled encode = encode_tiled();
  if (encode == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(kTmaColumns), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t element_strides[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// A [rows, k] bfloat16 matrix with row stride ld (elements), read in boxes of
// box_rows x 64 with the 128-byte swizzle; what lies outside reads as zero.
// Encoded maps are kept: weights never move and the allocator hands the same
// activation buffers out again and again.
inline bool make_map(CUtensorMap* map, const void* base, int rows, int k, long long ld, int box_rows) {
  using Key = std::tuple<const void*, int, int, long long, int>;
  static std::map<Key, CUtensorMap> known;
  static std::mutex guard;
  const Key key(base, rows, k, ld, box_rows);
  {
    std::lock_guard<std::mutex> lock(guard);
    auto found = known.find(key);
    if (found != known.end()) {
      *map = found->second;
      return true;
    }
  }
  if (!encode_map(map, base, rows, k, ld, box_rows)) return false;
  std::lock_guard<std::mutex> lock(guard);
  if (known.size() > 4096) known.clear();
  known.emplace(key, *map);
  return true;
}

}  // namespace mxb
