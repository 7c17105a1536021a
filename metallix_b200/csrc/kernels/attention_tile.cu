// Attention over the paged cache for any mix of prompt portions and decoded
// tokens: the general kernel of both precisions.
//
// One block takes up to 16 consecutive query tokens of one request and one
// query head, walks the request's keys in tiles of 32 absolute positions
// through its block table, and keeps scores, running maximum, running sum and
// the output accumulator in float32. Key tiles start at multiples of 32 of the
// absolute position, and a row's arithmetic touches only its own keys in
// ascending order, so the result at a position is bit-identical however the
// tokens were cut into steps or batched.
//
// Replaces the reference's gather of the whole context plus
// fast::scaled_dot_product_attention (crates/models/qwen/src/forward/paged.rs:329-342,
// :1067-1076, :1176-1184): s = (q k^T) * scale, causal with the diagonal at the
// query's own position, optional window (key > position - window), softmax
// over keys, query head j reads key/value head j / (heads / kv_heads).
#include "common.cuh"

namespace mxb {

constexpr int kTileQueries = 16;
constexpr int kTileKeys = 32;
constexpr int kTileThreads = 128;
constexpr float kMinusHuge = -1.0e30f;

template <typename T, int DPT>
__global__ void __launch_bounds__(kTileThreads)
paged_attention_tile_kernel(const T* __restrict__ q, const T* __restrict__ cache, T* __restrict__ out,
                            const int* __restrict__ block_tables, int max_pages,
                            const int* __restrict__ tile_request, const int* __restrict__ tile_start,
                            const int* __restrict__ tile_length, const int* __restrict__ positions,
                            int heads, int kv_heads, int head_dim, int page_tokens, int num_pages,
                            int window, float scale, int* status) {
  extern __shared__ float shared[];
  float* sQ = shared;                                   // [16][head_dim]
  float* sK = sQ + kTileQueries * head_dim;             // [32][head_dim + 1]
  float* sV = sK + kTileKeys * (head_dim + 1);          // [32][head_dim]
  float* sP = sV + kTileKeys * head_dim;                // [16][32]

  const int tile = blockIdx.x, head = blockIdx.y;
  const int kv = head / (heads / kv_heads);
  const int request = tile_request[tile];
  const int t0 = tile_start[tile];
  const int n = tile_length[tile];
  const int pos0 = positions[t0];
  const int last_pos = pos0 + n - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  const int tid = threadIdx.x;
  const int r = tid >> 3, lane8 = tid & 7;
  const int my_pos = pos0 + r;
  const bool row_valid = r < n;
  const int* table = block_tables + static_cast<size_t>(request) * max_pages;

  for (int i = tid; i < kTileQueries * head_dim; i += kTileThreads) {
    const int row = i / head_dim, d = i - row * head_dim;
    sQ[i] = row < n ? to_float(q[(static_cast<size_t>(t0 + row) * heads + head) * head_dim + d]) : 0.0f;
  }

  float m = kMinusHuge, l = 0.0f;
  float acc[DPT];
#pragma unroll
  for (int j = 0; j < DPT; ++j) acc[j] = 0.0f;

  const int tile_begin = first_key / kTileKeys, tile_end = last_pos / kTileKeys;
  for (int kt = tile_begin; kt <= tile_end; ++kt) {
    const int key0 = kt * kTileKeys;
    __syncthreads();  // the previous tile's K, V and P are no longer read
    for (int i = tid; i < kTileKeys * head_dim; i += kTileThreads) {
      const int kk = i / head_dim, d = i - kk * head_dim;
      const int key = key0 + kk;
      float kval = 0.0f, vval = 0.0f;
      if (key >= first_key && key <= last_pos) {
        const int page = table[key / page_tokens];
        if (page < 0 || page >= num_pages) {
          atomicOr(status, kStatusBadPage);
        } else {
          const size_t base = ((static_cast<size_t>(page) * 2 * kv_heads + kv) * page_tokens + key % page_tokens) * head_dim + d;
          kval = to_float(cache[base]);
          vval = to_float(cache[base + static_cast<size_t>(kv_heads) * page_tokens * head_dim]);
        }
      }
      sK[kk * (head_dim + 1) + d] = kval;
      sV[kk * head_dim + d] = vval;
    }
    __syncthreads();

    float s[4];
    bool visible[4];
    float tile_max = kMinusHuge;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = lane8 + 8 * j;
      const int key = key0 + c;
      float dot = 0.0f;
      const float* qrow = sQ + r * head_dim;
      const float* krow = sK + c * (head_dim + 1);
      for (int d = 0; d < head_dim; ++d) dot = fmaf(qrow[d], krow[d], dot);
      visible[j] = row_valid && key <= my_pos && key >= first_key && (window <= 0 || key > my_pos - window);
      s[j] = visible[j] ? dot * scale : kMinusHuge;
      tile_max = fmaxf(tile_max, s[j]);
    }
#pragma unroll
    for (int offset = 1; offset < 8; offset <<= 1)
      tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, offset));
    const float m_new = fmaxf(m, tile_max);
    const float alpha = expf(m - m_new);
    float psum = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p = visible[j] ? expf(s[j] - m_new) : 0.0f;
      sP[r * kTileKeys + lane8 + 8 * j] = p;
      psum += p;
    }
#pragma unroll
    for (int offset = 1; offset < 8; offset <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, offset);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();  // a row's 8 threads sit in one warp

    const float* prow = sP + r * kTileKeys;
#pragma unroll
    for (int j = 0; j < DPT; ++j) {
      const int d = lane8 + 8 * j;
      if (d < head_dim) {
        float sum = 0.0f;
        for (int k = 0; k < kTileKeys; ++k) sum = fmaf(prow[k], sV[k * head_dim + d], sum);
        acc[j] = acc[j] * alpha + sum;
      }
    }
  }

  if (row_valid) {
    const float inv = 1.0f / l;
    T* dst = out + (static_cast<size_t>(t0 + r) * heads + head) * head_dim;
#pragma unroll
    for (int j = 0; j < DPT; ++j) {
      const int d = lane8 + 8 * j;
      if (d < head_dim) dst[d] = from_float<T>(acc[j] * inv);
    }
  }
}

template <typename T, int DPT>
static int launch_tile(const void* q, const void* cache, void* out, const int* block_tables,
                       int max_pages, const int* tile_request, const int* tile_start,
                       const int* tile_length, const int* positions, int tiles, int heads,
                       int kv_heads, int head_dim, int page_tokens, int num_pages, int window,
                       float scale, int* status, cudaStream_t stream) {
  const size_t shared = sizeof(float) * (static_cast<size_t>(kTileQueries) * head_dim +
                                         static_cast<size_t>(kTileKeys) * (head_dim + 1) +
                                         static_cast<size_t>(kTileKeys) * head_dim +
                                         kTileQueries * kTileKeys);
  auto kernel = paged_attention_tile_kernel<T, DPT>;
  if (shared > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  dim3 grid(tiles, heads);
  kernel<<<grid, kTileThreads, shared, stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(cache), static_cast<T*>(out), block_tables,
      max_pages, tile_request, tile_start, tile_length, positions, heads, kv_heads, head_dim,
      page_tokens, num_pages, window, scale, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// Query tiles are listed by the caller: tile i covers tokens tile_start[i] ..
// tile_start[i] + tile_length[i] - 1 (at most 16, consecutive positions of
// request row tile_request[i]).
MXB_API int mxb_paged_attention_tile(const void* q, const void* cache, void* out,
                                     const int* block_tables, int max_pages,
                                     const int* tile_request, const int* tile_start,
                                     const int* tile_length, const int* positions, int tiles,
                                     int heads, int kv_heads, int head_dim, int page_tokens,
                                     int num_pages, int window, float scale, int dtype, int* status,
                                     cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (head_dim <= 0 || head_dim > 256 || heads % kv_heads != 0) return static_cast<int>(cudaErrorInvalidValue);
#define ARGS q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length, positions, \
             tiles, heads, kv_heads, head_dim, page_tokens, num_pages, window, scale, status, stream
#define DISPATCH(T)                                           \
  if (head_dim <= 16) return launch_tile<T, 2>(ARGS);         \
  if (head_dim <= 32) return launch_tile<T, 4>(ARGS);         \
  if (head_dim <= 64) return launch_tile<T, 8>(ARGS);         \
  if (head_dim <= 128) return launch_tile<T, 16>(ARGS);       \
  return launch_tile<T, 32>(ARGS);
  if (dtype == kF32) { DISPATCH(float) }
  if (dtype == kBF16) { DISPATCH(__nv_bfloat16) }
#undef DISPATCH
#undef ARGS
  return static_cast<int>(cudaErrorInvalidValue);
}
