// Causal grouped-query flash attention for prompt portions in bfloat16, over
// the paged cache (which already holds this step's own keys and values).
//
// One block of four warps takes up to 64 consecutive query tokens of one
// request and one query head (half a tile of the caller's list). It walks the request's keys in tiles of 64
// absolute positions, fetched page by page through the block table with
// 16-byte asynchronous copies into swizzled shared memory (two stages), forms
// q k^T and p v on the tensor cores (mma.sync m16n8k16, bfloat16 in, float32
// accumulate) and keeps scores, running maximum, running sum and the output
// accumulator in float32. Key tiles start at multiples of 64 of the absolute
// position and a row's arithmetic does not depend on the other rows of its
// tile, so a position's result is the same however the prompt was cut.
//
// Replaces the reference's gather of the whole context plus
// fast::scaled_dot_product_attention with a causal mask aligned to the last
// key (crates/models/qwen/src/forward/paged.rs:1143-1148, :1176-1184;
// crates/models/qwen/src/forward.rs:1967-1989).
#include "common.cuh"

namespace mxb {

constexpr int kFlashQueries = 64;
constexpr int kFlashKeys = 64;
constexpr int kFlashThreads = 128;

__device__ __forceinline__ uint32_t smem_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16 bytes global -> shared; src_bytes == 0 writes zeros.
__device__ __forceinline__ void copy_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void copy_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 2^x on the special-function unit (relative error about 2^-22); -inf gives 0.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a [rows][HD] bfloat16
// tile whose chunks are XOR-swizzled by the row so that ldmatrix meets no
// bank conflict.
template <int HD> __device__ __forceinline__ uint32_t tile_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(kFlashThreads, 3)
flash_prefill_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                     __nv_bfloat16* __restrict__ out, const int* __restrict__ block_tables, int max_pages,
                     const int* __restrict__ tile_request, const int* __restrict__ tile_start,
                     const int* __restrict__ tile_length, const int* __restrict__ positions, int heads,
                     int kv_heads, int page_tokens, int num_pages, int window, float scale, int* status) {
  constexpr int CHUNKS = HD / 8;                      // 16-byte chunks per row
  constexpr int TILE_BYTES = kFlashKeys * HD * 2;
  extern __shared__ __align__(128) unsigned char shared[];
  unsigned char* sK = shared;                          // 2 x [64][HD]
  unsigned char* sV = sK + 2 * TILE_BYTES;             // 2 x [64][HD]
  unsigned char* sQ = sK + TILE_BYTES;                 // [64][HD]: the query tile borrows the second key
                                                       // stage until its fragments sit in registers

  // Tile lists hold up to 128 tokens a tile: two blocks take 64 each.
  const int head = blockIdx.x, tile = blockIdx.y >> 1;  // heads of one tile run side by side and share its keys in L2
  const int kv = head / (heads / kv_heads);
  const int t0 = tile_start[tile] + (blockIdx.y & 1) * kFlashQueries;
  const int n = min(kFlashQueries, tile_length[tile] - static_cast<int>(blockIdx.y & 1) * kFlashQueries);
  if (n <= 0) return;
  const int pos0 = positions[t0];
  const int last_pos = pos0 + n - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int* table = block_tables + static_cast<size_t>(tile_request[tile]) * max_pages;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const size_t page_stride = static_cast<size_t>(2) * kv_heads * page_tokens * HD;
  const size_t v_offset = static_cast<size_t>(kv_heads) * page_tokens * HD;
  const __nv_bfloat16* head_base = cache + static_cast<size_t>(kv) * page_tokens * HD;

  // ---- the query tile
  for (int i = tid; i < kFlashQueries * CHUNKS; i += kFlashThreads) {
    const int row = i / CHUNKS, chunk = i - row * CHUNKS;
    const bool valid = row < n;
    const __nv_bfloat16* src = q + (static_cast<size_t>(t0 + (valid ? row : 0)) * heads + head) * HD + chunk * 8;
    copy_async_16(smem_address(sQ + tile_offset<HD>(row, chunk)), src, valid ? 16 : 0);
  }
  copy_async_commit();

  // Two threads per key row: one block-table lookup each, then their half of
  // the row's 16-byte chunks of K and of V.
  auto load_keys = [&](int key_tile, int stage) {
    const int row = tid >> 1, half = tid & 1;
    const int key = key_tile * kFlashKeys + row;
    bool valid = key >= first_key && key <= last_pos;
    int page = 0;
    if (valid) {
      page = table[key / page_tokens];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, kStatusBadPage);
        valid = false;
        page = 0;
      }
    }
    const __nv_bfloat16* src = head_base + page * page_stride + static_cast<size_t>(valid ? key % page_tokens : 0) * HD;
    const int bytes = valid ? 16 : 0;
#pragma unroll
    for (int c = 0; c < CHUNKS / 2; ++c) {
      const int chunk = half * (CHUNKS / 2) + c;
      const uint32_t offset = stage * TILE_BYTES + tile_offset<HD>(row, chunk);
      copy_async_16(smem_address(sK + offset), src + chunk * 8, bytes);
      copy_async_16(smem_address(sV + offset), src + v_offset + chunk * 8, bytes);
    }
    copy_async_commit();
  };

  const int tile_begin = first_key / kFlashKeys, tile_end = last_pos / kFlashKeys;
  load_keys(tile_begin, 0);

  // Each warp owns 16 query rows; a thread owns rows g and g + 8 of them.
  const int g = lane >> 2, t = lane & 3;
  const int row_lo = warp * 16 + g, row_hi = row_lo + 8;
  const int pos_lo = pos0 + row_lo, pos_hi = pos0 + row_hi;
  const bool valid_lo = row_lo < n, valid_hi = row_hi < n;
  const float scale_log2 = scale * 1.4426950408889634f;

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  uint32_t qf[HD / 16][4];

  // The query fragments move to registers before the second stage is filled.
  copy_async_wait<1>();  // the query tile (the first group) has landed
  __syncthreads();
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    ldmatrix_x4(qf[ks], smem_address(sQ + tile_offset<HD>(row, ks * 2 + (lane >> 4))));
  }
  __syncthreads();

  for (int kt = tile_begin; kt <= tile_end; ++kt) {
    const int stage = (kt - tile_begin) & 1;
    if (kt < tile_end) {
      load_keys(kt + 1, stage ^ 1);
      copy_async_wait<1>();
    } else {
      copy_async_wait<0>();
    }
    __syncthreads();
    const unsigned char* k_tile = sK + stage * TILE_BYTES;
    const unsigned char* v_tile = sV + stage * TILE_BYTES;

    // ---- s = q k^T for this warp's 16 rows and the tile's 64 keys
    float s[kFlashKeys / 8][4];
#pragma unroll
    for (int i = 0; i < kFlashKeys / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int nb = 0; nb < kFlashKeys / 16; ++nb) {  // two 8-key blocks per ldmatrix
        uint32_t kf[4];
        const int row = nb * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(kf, smem_address(k_tile + tile_offset<HD>(row, ks * 2 + ((lane >> 3) & 1))));
        mma_bf16_16816(s[2 * nb], qf[ks], kf[0], kf[1]);
        mma_bf16_16816(s[2 * nb + 1], qf[ks], kf[2], kf[3]);
      }
    }

    // ---- mask, running maximum and sum (float32). m_* hold the running
    // maximum already multiplied by scale * log2(e).
    const int key0 = kt * kFlashKeys;
    const bool all_seen = window <= 0 && n == kFlashQueries && key0 + kFlashKeys - 1 <= pos0;
    if (!all_seen) {
#pragma unroll
      for (int nb = 0; nb < kFlashKeys / 8; ++nb) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int key = key0 + nb * 8 + 2 * t + j;
          const bool seen_lo = valid_lo && key <= pos_lo && key >= first_key && (window <= 0 || key > pos_lo - window);
          const bool seen_hi = valid_hi && key <= pos_hi && key >= first_key && (window <= 0 || key > pos_hi - window);
          if (!seen_lo) s[nb][j] = -INFINITY;
          if (!seen_hi) s[nb][2 + j] = -INFINITY;
        }
      }
    }
    float max_lo = -INFINITY, max_hi = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < kFlashKeys / 8; ++nb) {
      max_lo = fmaxf(max_lo, fmaxf(s[nb][0], s[nb][1]));
      max_hi = fmaxf(max_hi, fmaxf(s[nb][2], s[nb][3]));
    }
    max_lo = fmaxf(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, 1));
    max_lo = fmaxf(max_lo, __shfl_xor_sync(0xffffffffu, max_lo, 2));
    max_hi = fmaxf(max_hi, __shfl_xor_sync(0xffffffffu, max_hi, 1));
    max_hi = fmaxf(max_hi, __shfl_xor_sync(0xffffffffu, max_hi, 2));
    max_lo = fmaxf(m_lo, max_lo * scale_log2);  // scale > 0 keeps the order
    max_hi = fmaxf(m_hi, max_hi * scale_log2);
    // A row that has seen no key yet keeps a finite reference so that no
    // inf - inf appears.
    const float ref_lo = max_lo == -INFINITY ? 0.0f : max_lo;
    const float ref_hi = max_hi == -INFINITY ? 0.0f : max_hi;
    const float alpha_lo = fast_exp2(m_lo - ref_lo), alpha_hi = fast_exp2(m_hi - ref_hi);
    float sum_lo = 0.0f, sum_hi = 0.0f;
    uint32_t pf[kFlashKeys / 16][4];
#pragma unroll
    for (int nb = 0; nb < kFlashKeys / 8; ++nb) {
      const float p0 = fast_exp2(fmaf(s[nb][0], scale_log2, -ref_lo)), p1 = fast_exp2(fmaf(s[nb][1], scale_log2, -ref_lo));
      const float p2 = fast_exp2(fmaf(s[nb][2], scale_log2, -ref_hi)), p3 = fast_exp2(fmaf(s[nb][3], scale_log2, -ref_hi));
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 1);
    sum_lo += __shfl_xor_sync(0xffffffffu, sum_lo, 2);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 1);
    sum_hi += __shfl_xor_sync(0xffffffffu, sum_hi, 2);
    l_lo = l_lo * alpha_lo + sum_lo;
    l_hi = l_hi * alpha_hi + sum_hi;
    m_lo = max_lo;
    m_hi = max_hi;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      o[i][0] *= alpha_lo; o[i][1] *= alpha_lo;
      o[i][2] *= alpha_hi; o[i][3] *= alpha_hi;
    }

    // ---- o += p v
#pragma unroll
    for (int ks = 0; ks < kFlashKeys / 16; ++ks) {
#pragma unroll
      for (int nb = 0; nb < HD / 16; ++nb) {
        uint32_t vf[4];
        const int row = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(vf, smem_address(v_tile + tile_offset<HD>(row, nb * 2 + (lane >> 4))));
        mma_bf16_16816(o[2 * nb], pf[ks], vf[0], vf[1]);
        mma_bf16_16816(o[2 * nb + 1], pf[ks], vf[2], vf[3]);
      }
    }
    __syncthreads();  // this stage may be refilled by the next iteration's copies
  }

  const float inv_lo = valid_lo ? 1.0f / l_lo : 0.0f, inv_hi = valid_hi ? 1.0f / l_hi : 0.0f;
  __nv_bfloat16* out_lo = out + (static_cast<size_t>(t0 + row_lo) * heads + head) * HD;
  __nv_bfloat16* out_hi = out + (static_cast<size_t>(t0 + row_hi) * heads + head) * HD;
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) {
    const int d = i * 8 + 2 * t;
    if (valid_lo) *reinterpret_cast<uint32_t*>(out_lo + d) = pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
    if (valid_hi) *reinterpret_cast<uint32_t*>(out_hi + d) = pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
  }
}

template <int HD>
static int launch_flash(const void* q, const void* cache, void* out, const int* block_tables, int max_pages,
                        const int* tile_request, const int* tile_start, const int* tile_length,
                        const int* positions, int tiles, int heads, int kv_heads, int page_tokens,
                        int num_pages, int window, float scale, int* status, cudaStream_t stream) {
  const int shared = 4 * kFlashKeys * HD * 2;
  auto kernel = flash_prefill_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(heads, 2 * tiles);
  kernel<<<grid, kFlashThreads, shared, stream>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(cache),
      static_cast<__nv_bfloat16*>(out), block_tables, max_pages, tile_request, tile_start, tile_length,
      positions, heads, kv_heads, page_tokens, num_pages, window, scale, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// bfloat16 with head_dim 64 or 128; everything else goes through the general
// tile kernel.
MXB_API int mxb_flash_prefill_supported(int head_dim, int heads, int kv_heads, int dtype) {
  if (kv_heads <= 0 || heads % kv_heads != 0 || dtype != kBF16) return 0;
  return head_dim == 64 || head_dim == 128 ? 1 : 0;
}

MXB_API int mxb_flash_prefill_tile() { return 2 * kFlashQueries; }

// Query tiles as for the general kernel, but up to 128 tokens each.
MXB_API int mxb_flash_prefill(const void* q, const void* cache, void* out, const int* block_tables,
                              int max_pages, const int* tile_request, const int* tile_start,
                              const int* tile_length, const int* positions, int tiles, int heads,
                              int kv_heads, int head_dim, int page_tokens, int num_pages, int window,
                              float scale, int dtype, int* status, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (!mxb_flash_prefill_supported(head_dim, heads, kv_heads, dtype)) return static_cast<int>(cudaErrorInvalidValue);
  if (head_dim == 64)
    return launch_flash<64>(q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length,
                            positions, tiles, heads, kv_heads, page_tokens, num_pages, window, scale, status, stream);
  return launch_flash<128>(q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length,
                           positions, tiles, heads, kv_heads, page_tokens, num_pages, window, scale, status, stream);
}
