// Causal grouped-query attention for prompt portions in bfloat16 on the
// fifth-generation tensor cores, over the paged cache (which already holds
// this step's own keys and values).
//
// One block takes up to 128 consecutive query tokens of one request and one
// query head and walks the request's keys in tiles of 128 absolute positions.
//   warp 0      fetches: the query tile once, then for every key tile the
//               pages the block table names, K and V, as TMA boxes of one page
//               x 64 values with the 128-byte swizzle (so a tile of K is a
//               K-major operand and a tile of V an MN-major one, as they lie
//               in the cache);
//   warp 1      owns tensor memory and issues the MMAs: S = Q K^T into one of
//               two score buffers, and O_tile = P V into one of two output
//               buffers, with P read from tensor memory where the softmax
//               warps left it (over the scores it came from);
//   warps 2..5  one thread per query row: mask, running maximum and sum in
//               float32, P = exp2(...) back to tensor memory as bfloat16, and
//               the row's output accumulator in registers: acc = acc * alpha +
//               O_tile, read back with tcgen05.ld.
// The MMAs of tile j + 1's scores run while the softmax of tile j does, and
// the accumulation of tile j - 1 while P_j V_j runs.
//
// Key tiles start at multiples of 128 of the absolute position and a row's
// arithmetic does not depend on the other rows of its tile, so a position's
// result is the same however the prompt was cut.
//
// Replaces the reference's gather of the whole context plus
// fast::scaled_dot_product_attention with a causal mask aligned to the last
// key (crates/models/qwen/src/forward/paged.rs:1143-1148, :1176-1184;
// crates/models/qwen/src/forward.rs:1967-1989).
//
// Every wait on a barrier is bounded: if one runs out, the status word gets a
// bit, the block stops issuing work, frees its tensor memory and leaves.
#include "tcgen05.cuh"

namespace mxb {

constexpr int kFaRows = 128;     // query rows of a block
constexpr int kFaKeys = 128;     // keys of a tile
constexpr int kFaThreads = 192;
constexpr int kFaTmemColumns = 512;
constexpr int kFaHalfBytes = 128 * kTmaColumns * 2;  // a [128 x 64] bfloat16 operand block: 16 KiB

template <int HD> struct FaConfig {
  static constexpr int kHalves = HD / kTmaColumns;
  static constexpr int kTileBytes = kHalves * kFaHalfBytes;    // Q, a K stage or a V stage
  static constexpr int kStages = HD == 64 ? 4 : 2;             // one block per SM either way
  static constexpr int kSharedBytes = (1 + 2 * kStages) * kTileBytes + 1024;
  static constexpr int kScoreColumns = kFaKeys;                // two buffers of 128 columns
  static constexpr int kOutputBase = 2 * kFaKeys;              // then two buffers of HD columns
};

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
  __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&pair);
}

template <int HD>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_cache,
                             __nv_bfloat16* __restrict__ out, const int* __restrict__ block_tables, int max_pages,
                             const int* __restrict__ tile_request, const int* __restrict__ tile_start,
                             const int* __restrict__ tile_length, const int* __restrict__ positions, int heads,
                             int kv_heads, int page_tokens, int num_pages, int window, float scale, int* status) {
  using Config = FaConfig<HD>;
  constexpr int STAGES = Config::kStages;
  constexpr int HALVES = Config::kHalves;
  extern __shared__ unsigned char fa_shared_raw[];
  __shared__ __align__(8) uint64_t q_full;
  __shared__ __align__(8) uint64_t k_full[STAGES], k_empty[STAGES], v_full[STAGES], v_empty[STAGES];
  __shared__ __align__(8) uint64_t s_full[2], p_full[2], o_full[2], o_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  unsigned char* q_tile = fa_shared_raw + ((1024 - (shared_address(fa_shared_raw) & 1023)) & 1023);
  unsigned char* k_tiles = q_tile + Config::kTileBytes;
  unsigned char* v_tiles = k_tiles + STAGES * Config::kTileBytes;

  const int head = blockIdx.x, tile = blockIdx.y;  // heads of one tile run side by side and share its keys in L2
  const int kv = head / (heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = tile_start[tile], n = tile_length[tile];
  const int pos0 = positions[t0];
  const int last_pos = pos0 + n - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int tile_begin = first_key / kFaKeys, tile_end = last_pos / kFaKeys;
  const int key_tiles = tile_end - tile_begin + 1;

  if (threadIdx.x == 0) {
    barrier_init(&q_full, 1);
    for (int s = 0; s < STAGES; ++s) {
      barrier_init(&k_full[s], 1);
      barrier_init(&k_empty[s], 1);
      barrier_init(&v_full[s], 1);
      barrier_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(&s_full[b], 1);
      barrier_init(&p_full[b], kFaRows);   // every softmax thread arrives
      barrier_init(&o_full[b], 1);
      barrier_init(&o_empty[b], kFaRows);
    }
    barrier_init_fence();
    failed = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(shared_address(&tmem_base_slot)), "r"(kFaTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---- fetch: Q once, then K and V of every key tile, page by page
    const int* table = block_tables + static_cast<size_t>(tile_request[tile]) * max_pages;
    if (lane == 0) {
      barrier_arrive_expect(&q_full, Config::kTileBytes);
      for (int half = 0; half < HALVES; ++half)
        tma_load_2d(q_tile + half * kFaHalfBytes, &map_q, head * HD + half * kTmaColumns, t0, &q_full);
    }
    const int pages_per_tile = kFaKeys / page_tokens;
    const int copies = 2 * pages_per_tile * HALVES;  // K and V, every page, every 64-value half
    for (int i = 0; i < key_tiles && !failed; ++i) {
      const int stage = i % STAGES;
      const uint32_t parity = (i / STAGES) & 1;
      const int key0 = (tile_begin + i) * kFaKeys;
      bool ok = barrier_wait(&k_empty[stage], parity ^ 1, status);
      ok = ok && barrier_wait(&v_empty[stage], parity ^ 1, status);
      if (!ok) { failed = 1; break; }
      if (lane == 0) {
        barrier_arrive_expect(&k_full[stage], Config::kTileBytes);
        barrier_arrive_expect(&v_full[stage], Config::kTileBytes);
      }
      __syncwarp();
      for (int copy = lane; copy < copies; copy += 32) {
        const int half = copy % HALVES;
        const int which = (copy / HALVES) % 2;  // 0 K, 1 V
        const int slot = copy / (2 * HALVES);   // page of the tile
        const int page_key = key0 + slot * page_tokens;
        // Pages no row of the tile can see are not looked up: page 0 stands
        // in (its values are finite and every such key is masked).
        int page = 0;
        if (page_key <= last_pos && page_key + page_tokens > first_key && page_key / page_tokens < max_pages) {
          page = table[page_key / page_tokens];
          if (page < 0 || page >= num_pages) {
            atomicOr(status, kStatusBadPage);
            page = 0;
          }
        }
        const int row = ((page * 2 + which) * kv_heads + kv) * page_tokens;
        unsigned char* dst = (which ? v_tiles : k_tiles) + stage * Config::kTileBytes + half * kFaHalfBytes +
                             slot * page_tokens * (kTmaColumns * 2);
        tma_load_2d(dst, &map_cache, half * kTmaColumns, row, which ? &v_full[stage] : &k_full[stage]);
      }
    }
  } else if (warp == 1) {
    // ---- one thread issues every MMA
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc_instruction_descriptor(kFaRows, kFaKeys);
      constexpr uint32_t idesc_o = tc_instruction_descriptor_b_mn(kFaRows, HD);
      const uint32_t q_address = shared_address(q_tile);
      bool ok = barrier_wait(&q_full, 0, status);
      auto scores = [&](int i) {  // S_i = Q K_i^T
        const int stage = i % STAGES;
        if (!barrier_wait(&k_full[stage], (i / STAGES) & 1, status)) return false;
        tc_fence_after_sync();
        const uint32_t k_address = shared_address(k_tiles + stage * Config::kTileBytes);
        const uint32_t tmem_s = tmem_base + (i & 1) * Config::kScoreColumns;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t offset = (kk / 4) * kFaHalfBytes + (kk % 4) * 32;
          tc_mma(tmem_s, tc_smem_descriptor(q_address + offset), tc_smem_descriptor(k_address + offset), idesc_s,
                 kk > 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[stage]);
        tc_commit(&s_full[i & 1]);
        return true;
      };
      auto outputs = [&](int i) {  // O_tile_i = P_i V_i
        const int stage = i % STAGES, buffer = i & 1;
        if (!barrier_wait(&v_full[stage], (i / STAGES) & 1, status)) return false;
        if (!barrier_wait(&o_empty[buffer], ((i >> 1) & 1) ^ 1, status)) return false;
        if (!barrier_wait(&p_full[buffer], (i >> 1) & 1, status)) return false;
        tc_fence_after_sync();
        const uint32_t v_address = shared_address(v_tiles + stage * Config::kTileBytes);
        const uint32_t tmem_p = tmem_base + buffer * Config::kScoreColumns;
        const uint32_t tmem_o = tmem_base + Config::kOutputBase + buffer * HD;
#pragma unroll
        for (int kk = 0; kk < kFaKeys / 16; ++kk) {  // 16 keys per instruction: two 8-row groups of V, 8 columns of P
          tc_mma_ts(tmem_o, tmem_p + kk * 8, tc_smem_descriptor_mn(v_address + kk * 2048, kFaHalfBytes), idesc_o,
                    kk > 0 ? 1u : 0u);
        }
        tc_commit(&v_empty[stage]);
        tc_commit(&o_full[buffer]);
        return true;
      };
      ok = ok && scores(0);
      for (int i = 0; i < key_tiles && ok && !failed; ++i) {
        if (i + 1 < key_tiles) ok = scores(i + 1);
        ok = ok && outputs(i);
      }
      if (!ok) failed = 1;
    }
  } else {
    // ---- softmax and accumulation: one thread per query row
    const int lane_base = (warp & 3) * 32;
    const int row = lane_base + lane;
    const bool valid = row < n;
    const int pos = pos0 + row;
    const int key_hi = valid ? pos : -1;                                   // last key this row sees
    const int key_lo = window > 0 ? max(0, pos - window + 1) : 0;          // first key this row sees
    const float scale_log2 = scale * 1.4426950408889634f;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
    float acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f, alpha_pending = 0.0f;
    bool ok = true;

    auto accumulate = [&](int i, float alpha) {  // acc = acc * alpha + O_tile_i
      const int buffer = i & 1;
      if (!barrier_wait(&o_full[buffer], (i >> 1) & 1, status)) return false;
      tc_fence_after_sync();
      const uint32_t tmem_o = tmem_lane + Config::kOutputBase + buffer * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t o[32];
        tc_load_32(tmem_o + c, o);
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[c + j] = fmaf(acc[c + j], alpha, __uint_as_float(o[j]));
      }
      tc_fence_before_sync();
      barrier_arrive(&o_empty[buffer]);
      return true;
    };

    for (int i = 0; i < key_tiles; ++i) {
      const int buffer = i & 1;
      const int key0 = (tile_begin + i) * kFaKeys;
      if (!barrier_wait(&s_full[buffer], (i >> 1) & 1, status) || failed) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tmem_s = tmem_lane + buffer * Config::kScoreColumns;
      const bool all_seen = key0 >= key_lo && key0 + kFaKeys - 1 <= key_hi;
      // Running maximum, already multiplied by scale * log2(e) (scale > 0 keeps the order).
      float tile_max = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < kFaKeys; c += 32) {
        uint32_t s[32];
        tc_load_32(tmem_s + c, s);
        if (all_seen) {
#pragma unroll
          for (int j = 0; j < 32; ++j) tile_max = fmaxf(tile_max, __uint_as_float(s[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int key = key0 + c + j;
            if (key >= key_lo && key <= key_hi) tile_max = fmaxf(tile_max, __uint_as_float(s[j]));
          }
        }
      }
      const float m_new = fmaxf(m, tile_max * scale_log2);
      // A row that has seen no key yet keeps a finite reference so that no inf - inf appears.
      const float ref = m_new == -INFINITY ? 0.0f : m_new;
      const float alpha = fa_exp2(m - ref);
      float sum = 0.0f;
#pragma unroll 1
      for (int c = 0; c < kFaKeys; c += 32) {
        uint32_t s[32];
        tc_load_32(tmem_s + c, s);
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          float p0 = fa_exp2(fmaf(__uint_as_float(s[j]), scale_log2, -ref));
          float p1 = fa_exp2(fmaf(__uint_as_float(s[j + 1]), scale_log2, -ref));
          if (!all_seen) {
            const int key = key0 + c + j;
            if (key < key_lo || key > key_hi) p0 = 0.0f;
            if (key + 1 < key_lo || key + 1 > key_hi) p1 = 0.0f;
          }
          sum += p0 + p1;
          packed[j >> 1] = fa_pack(p0, p1);
        }
        // P lies over the scores it came from: columns this thread has already read.
        tc_store_16(tmem_s + (c >> 1), packed);
      }
      tc_store_wait();
      tc_fence_before_sync();
      barrier_arrive(&p_full[buffer]);
      l = fmaf(l, alpha, sum);
      m = m_new;
      if (i > 0 && !accumulate(i - 1, alpha_pending)) { ok = false; break; }
      alpha_pending = alpha;
    }
    if (ok && !failed) ok = accumulate(key_tiles - 1, alpha_pending);
    if (!ok) failed = 1;
    if (ok && valid) {
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = out + (static_cast<size_t>(t0 + row) * heads + head) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        *reinterpret_cast<uint4*>(dst + c) =
            make_uint4(fa_pack(acc[c] * inv, acc[c + 1] * inv), fa_pack(acc[c + 2] * inv, acc[c + 3] * inv),
                       fa_pack(acc[c + 4] * inv, acc[c + 5] * inv), fa_pack(acc[c + 6] * inv, acc[c + 7] * inv));
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (failed && threadIdx.x == 0) {
    // A wait ran out somewhere. Give loads that may still be in flight a
    // millisecond before the block's shared memory goes back.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kFaTmemColumns) : "memory");
  }
}

template <int HD>
static int launch_flash_tc(const void* q, const void* cache, void* out, const int* block_tables, int max_pages,
                           const int* tile_request, const int* tile_start, const int* tile_length,
                           const int* positions, int tokens, int tiles, int heads, int kv_heads, int page_tokens,
                           int num_pages, int window, float scale, int* status, cudaStream_t stream) {
  using Config = FaConfig<HD>;
  CUtensorMap map_q, map_cache;
  // q as [tokens, heads * HD]; the cache as [pages * 2 * kv_heads * page_tokens, HD].
  const long long cache_rows = static_cast<long long>(num_pages) * 2 * kv_heads * page_tokens;
  if (cache_rows > 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
  if (!make_map(&map_q, q, tokens, heads * HD, static_cast<long long>(heads) * HD, kFaRows) ||
      !make_map(&map_cache, cache, static_cast<int>(cache_rows), HD, HD, page_tokens))
    return static_cast<int>(cudaErrorInvalidValue);
  auto kernel = flash_prefill_tcgen05_kernel<HD>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Config::kSharedBytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(heads, tiles);
  kernel<<<grid, kFaThreads, Config::kSharedBytes, stream>>>(
      map_q, map_cache, static_cast<__nv_bfloat16*>(out), block_tables, max_pages, tile_request, tile_start,
      tile_length, positions, heads, kv_heads, page_tokens, num_pages, window, scale, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// bfloat16, head_dim 64 or 128, pages of 8, 16, 32, 64 or 128 tokens (a page
// must fill whole 8-row groups of the swizzled tile and divide a key tile).
MXB_API int mxb_flash_prefill_tcgen05_supported(int head_dim, int heads, int kv_heads, int page_tokens, int dtype) {
  if (kv_heads <= 0 || heads % kv_heads != 0 || dtype != kBF16) return 0;
  if (head_dim != 64 && head_dim != 128) return 0;
  if (page_tokens < 8 || page_tokens > kFaKeys || kFaKeys % page_tokens != 0) return 0;
  return 1;
}

MXB_API int mxb_flash_prefill_tcgen05_tile() { return kFaRows; }

// Query tiles of up to 128 tokens each; q and out are [tokens, heads, head_dim].
MXB_API int mxb_flash_prefill_tcgen05(const void* q, const void* cache, void* out, const int* block_tables,
                                      int max_pages, const int* tile_request, const int* tile_start,
                                      const int* tile_length, const int* positions, int tokens, int tiles,
                                      int heads, int kv_heads, int head_dim, int page_tokens, int num_pages,
                                      int window, float scale, int dtype, int* status, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (!mxb_flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page_tokens, dtype))
    return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  if (head_dim == 64)
    return launch_flash_tc<64>(q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length,
                               positions, tokens, tiles, heads, kv_heads, page_tokens, num_pages, window, scale,
                               status, stream);
  return launch_flash_tc<128>(q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length,
                              positions, tokens, tiles, heads, kv_heads, page_tokens, num_pages, window, scale,
                              status, stream);
}
