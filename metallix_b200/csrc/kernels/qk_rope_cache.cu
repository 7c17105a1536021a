// Per-head q/k RMSNorm, rotate-half RoPE and the write of K and V into the
// paged cache, in one pass over the projected q, k and v.
//
// Replaces, per layer, the reference's two fast::rms_norm calls, two
// fast::rope calls (crates/models/qwen/src/forward.rs:2031-2062) and the pool
// scatter (crates/models/qwen/src/forward/paged.rs:300-325). Norm and rotation
// run in float32; cos and sin come from a table built in float64.
//
// Cache layout of one layer: [pages, 2 (K, V), kv_heads, page_tokens, head_dim];
// position p of a request lives in page table[p / page_tokens] at row
// p % page_tokens, which the caller passes flattened as slot = page *
// page_tokens + row.
#include "common.cuh"

namespace mxb {

template <typename T>
__global__ void qk_norm_rope_cache_kernel(
    const T* __restrict__ q_in, const T* __restrict__ k_in, const T* __restrict__ v_in,
    long long q_stride, long long k_stride, long long v_stride,  // row strides in elements
    T* __restrict__ q_out,                                        // [tokens, heads, head_dim]
    T* __restrict__ cache, const int* __restrict__ slots,         // slots may be null: no write
    const int* __restrict__ positions,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight,  // null: no norm
    const float* __restrict__ cos_table, const float* __restrict__ sin_table,  // null: no rotation
    int table_positions, int rotary_dim, int heads, int kv_heads, int head_dim, int page_tokens,
    int num_pages, float eps, int* status) {
  extern __shared__ float head[];  // head_dim values
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int h = blockIdx.y;  // 0..heads-1: q, then kv_heads of k, then kv_heads of v
  const bool is_q = h < heads;
  const bool is_k = !is_q && h < heads + kv_heads;
  const int kv = is_q ? 0 : (is_k ? h - heads : h - heads - kv_heads);

  const T* src = is_q ? q_in + t * q_stride + static_cast<long long>(h) * head_dim
               : is_k ? k_in + t * k_stride + static_cast<long long>(kv) * head_dim
                      : v_in + t * v_stride + static_cast<long long>(kv) * head_dim;

  T* dst = nullptr;
  if (is_q) {
    if (q_out == nullptr) return;
    dst = q_out + (static_cast<size_t>(t) * heads + h) * head_dim;
  } else {
    if (slots == nullptr || cache == nullptr) return;
    const int slot = slots[t];
    if (slot < 0) return;  // this token does not write the cache
    const int page = slot / page_tokens, row = slot - page * page_tokens;
    if (page >= num_pages) {
      if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
      return;
    }
    dst = cache + (((static_cast<size_t>(page) * 2 + (is_k ? 0 : 1)) * kv_heads + kv) * page_tokens + row) * head_dim;
  }

  if (!is_q && !is_k) {  // values are stored as projected
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) dst[i] = src[i];
    return;
  }

  const float* weight = is_q ? q_weight : k_weight;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
    const float v = to_float(src[i]);
    head[i] = v;
    sum += v * v;
  }
  if (weight != nullptr) {
    sum = block_sum(sum, scratch);
    const float scale = rsqrtf(sum / static_cast<float>(head_dim) + eps);
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) head[i] = head[i] * scale * weight[i];
  }
  __syncthreads();

  const int half = rotary_dim >> 1;
  int pos = positions[t];
  const bool rotate = cos_table != nullptr;
  if (rotate && (pos < 0 || pos >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, kStatusBadSlot);
    pos = 0;
  }
  for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
    float out = head[i];
    if (rotate && i < rotary_dim) {
      const int j = i < half ? i : i - half;
      const float c = cos_table[static_cast<size_t>(pos) * half + j];
      const float s = sin_table[static_cast<size_t>(pos) * half + j];
      // out[i] = x[i] cos - x[i + half] sin; out[i + half] = x[i + half] cos + x[i] sin
      out = i < half ? head[i] * c - head[i + half] * s : head[i] * c + head[i - half] * s;
    }
    dst[i] = from_float<T>(out);
  }
}

// V values of type T moved as one access of V * sizeof(T) bytes.
template <typename T, int V> struct alignas(sizeof(T) * V) Pack { T v[V]; };

// The same work without shared memory, for head sizes 64, 128 and 256 with
// the rotation over the whole head. Every access is 16 bytes: a lane holds V
// = 16 / sizeof(T) consecutive values of the lower half of a head and the
// same of the upper half, so the rotation partner of element i (i +- head_dim
// / 2) sits in the same lane; head_dim / (2 V) lanes make up a head, a warp
// takes 32 / that many heads at once, and the sum of squares runs over a
// head's lanes only.
template <typename T, int HD>
__global__ void __launch_bounds__(256)
qk_norm_rope_cache_warp_kernel(
    const T* __restrict__ q_in, const T* __restrict__ k_in, const T* __restrict__ v_in,
    long long q_stride, long long k_stride, long long v_stride, T* __restrict__ q_out,
    T* __restrict__ cache, const int* __restrict__ slots, const int* __restrict__ positions,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight,
    const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions,
    int tokens, int heads, int kv_heads, int page_tokens, int num_pages, float eps, int* status) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr int HALF = HD / 2;
  constexpr int LANES = HALF / V;          // lanes of a head
  constexpr int HEADS = 32 / LANES;        // heads of a warp
  static_assert(LANES >= 1 && LANES <= 32 && (LANES & (LANES - 1)) == 0, "a head's lanes must divide a warp");
  using Values = Pack<T, V>;
  using Floats = Pack<float, 4>;
  chain_release();
  // Up to chain_wait(): only the step's integers, the norm weights and the
  // cos/sin tables, none of which a kernel of this step writes.
  const int lane = threadIdx.x & 31, sub = lane % LANES;
  const int per_token = heads + 2 * kv_heads;
  // The launcher keeps tokens * per_token below 2^31: 32-bit division, which
  // is a fraction of the instructions the 64-bit one takes.
  const unsigned total = static_cast<unsigned>(tokens) * static_cast<unsigned>(per_token);
  const unsigned item = (blockIdx.x * 8u + (threadIdx.x >> 5)) * HEADS + lane / LANES;
  // Lanes without work stay to the end: the sums below shuffle within a head's lanes.
  bool active = item < total;
  const int t = active ? static_cast<int>(item / static_cast<unsigned>(per_token)) : 0;
  const int h = active ? static_cast<int>(item - static_cast<unsigned>(t) * static_cast<unsigned>(per_token)) : 0;
  const bool is_q = h < heads;
  const bool is_k = !is_q && h < heads + kv_heads;
  const int kv = is_q ? 0 : (is_k ? h - heads : h - heads - kv_heads);
  const T* src = is_q ? q_in + t * q_stride + static_cast<long long>(h) * HD
               : is_k ? k_in + t * k_stride + static_cast<long long>(kv) * HD
                      : v_in + t * v_stride + static_cast<long long>(kv) * HD;
  T* dst = nullptr;
  if (is_q) {
    if (q_out == nullptr) active = false;
    else dst = q_out + (static_cast<size_t>(t) * heads + h) * HD;
  } else if (slots == nullptr || cache == nullptr) {
    active = false;
  } else if (active) {
    const int slot = slots[t];
    const int page = slot / page_tokens, row = slot - page * page_tokens;
    if (slot < 0) {
      active = false;
    } else if (page >= num_pages) {
      if (sub == 0) atomicOr(status, kStatusBadSlot);
      active = false;
    } else {
      dst = cache + (((static_cast<size_t>(page) * 2 + (is_k ? 0 : 1)) * kv_heads + kv) * page_tokens + row) * HD;
    }
  }
  const bool plain_copy = !is_q && !is_k;   // values: no norm, no rotation
  const float* weight = is_q ? q_weight : k_weight;
  float gain[2 * V], c[V], sn[V];
#pragma unroll
  for (int j = 0; j < 2 * V; ++j) gain[j] = 1.0f;
#pragma unroll
  for (int j = 0; j < V; ++j) { c[j] = 1.0f; sn[j] = 0.0f; }
  if (active && !plain_copy && weight != nullptr) {
#pragma unroll
    for (int q4 = 0; q4 < V / 4; ++q4) {
      const Floats lo = reinterpret_cast<const Floats*>(weight + V * sub)[q4];
      const Floats hi = reinterpret_cast<const Floats*>(weight + HALF + V * sub)[q4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        gain[q4 * 4 + j] = lo.v[j];
        gain[V + q4 * 4 + j] = hi.v[j];
      }
    }
  }
  if (active && !plain_copy && cos_table != nullptr) {
    int pos = positions[t];
    if (pos < 0 || pos >= table_positions) {
      if (sub == 0) atomicOr(status, kStatusBadSlot);
      pos = 0;
    }
#pragma unroll
    for (int q4 = 0; q4 < V / 4; ++q4) {
      const Floats cs = reinterpret_cast<const Floats*>(cos_table + static_cast<size_t>(pos) * HALF + V * sub)[q4];
      const Floats ss = reinterpret_cast<const Floats*>(sin_table + static_cast<size_t>(pos) * HALF + V * sub)[q4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        c[q4 * 4 + j] = cs.v[j];
        sn[q4 * 4 + j] = ss.v[j];
      }
    }
  }
  chain_wait();
  src = behind_wait(src);  // written by the kernel ahead of this one
  Values in_lo = {}, in_hi = {};
  if (active) {
    in_lo = reinterpret_cast<const Values*>(src)[sub];
    in_hi = reinterpret_cast<const Values*>(src + HALF)[sub];
  }
  if (plain_copy) {   // the same for every lane of a head; other heads of the warp go on below
    if (active) {
      reinterpret_cast<Values*>(dst)[sub] = in_lo;
      reinterpret_cast<Values*>(dst + HALF)[sub] = in_hi;
    }
    active = false;
  }
  // A warp whose heads are all values (or past the end) has nothing left to do.
  if (__all_sync(0xffffffffu, !active)) return;
  float x[2 * V];
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    x[j] = to_float(in_lo.v[j]);
    x[V + j] = to_float(in_hi.v[j]);
  }
#pragma unroll
  for (int j = 0; j < 2 * V; ++j) sum += x[j] * x[j];
#pragma unroll
  for (int offset = LANES / 2; offset > 0; offset >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
  if (weight != nullptr) {
    const float scale = rsqrtf(sum / static_cast<float>(HD) + eps);
#pragma unroll
    for (int j = 0; j < 2 * V; ++j) x[j] = x[j] * scale * gain[j];
  }
  if (cos_table != nullptr) {
#pragma unroll
    for (int j = 0; j < V; ++j) {
      // element V sub + j (below HALF) and its partner HALF further, x[V + j]
      const float lo = x[j], hi = x[V + j];
      x[j] = lo * c[j] - hi * sn[j];
      x[V + j] = hi * c[j] + lo * sn[j];
    }
  }
  if (!active) return;
  Values out_lo, out_hi;
#pragma unroll
  for (int j = 0; j < V; ++j) {
    out_lo.v[j] = from_float<T>(x[j]);
    out_hi.v[j] = from_float<T>(x[V + j]);
  }
  reinterpret_cast<Values*>(dst)[sub] = out_lo;
  reinterpret_cast<Values*>(dst + HALF)[sub] = out_hi;
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_qk_norm_rope_cache(
    const void* q_in, const void* k_in, const void* v_in, long long q_stride, long long k_stride,
    long long v_stride, void* q_out, void* cache, const int* slots, const int* positions,
    const float* q_weight, const float* k_weight, const float* cos_table, const float* sin_table,
    int table_positions, int rotary_dim, int tokens, int heads, int kv_heads, int head_dim,
    int page_tokens, int num_pages, float eps, int dtype, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return static_cast<int>(cudaErrorInvalidValue);
  // The warp kernel moves 16 bytes per access: rows and bases must be aligned to that.
  const int element = dtype == kF32 ? 4 : 2;
  auto aligned = [&](const void* p, long long stride) {
    return p == nullptr || (reinterpret_cast<uintptr_t>(p) % 16 == 0 && (stride * element) % 16 == 0);
  };
  const bool vector_ok = aligned(q_in, q_stride) && aligned(k_in, k_stride) && aligned(v_in, v_stride) &&
                         aligned(q_out, 0) && aligned(cache, 0) && aligned(q_weight, 0) && aligned(k_weight, 0) &&
                         aligned(cos_table, 0) && aligned(sin_table, 0);
  if ((head_dim == 64 || head_dim == 128 || head_dim == 256) && (cos_table == nullptr || rotary_dim == head_dim) &&
      vector_ok && (dtype == kF32 || dtype == kBF16)) {
    const long long items = static_cast<long long>(tokens) * (heads + 2 * kv_heads);
    if (items >= 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
    const int heads_per_warp = 32 / (head_dim / 2 / (16 / element));
    const unsigned blocks = static_cast<unsigned>((items + 8 * heads_per_warp - 1) / (8 * heads_per_warp));
    cudaError_t launch_status = cudaSuccess;
#define WARP_LAUNCH(T, HD) launch_status = launch_chained(qk_norm_rope_cache_warp_kernel<T, HD>, dim3(blocks), dim3(256), 0, stream, \
        static_cast<const T*>(q_in), static_cast<const T*>(k_in), static_cast<const T*>(v_in), q_stride, k_stride, \
        v_stride, static_cast<T*>(q_out), static_cast<T*>(cache), slots, positions, q_weight, k_weight, cos_table, \
        sin_table, table_positions, tokens, heads, kv_heads, page_tokens, num_pages, eps, status)
    if (dtype == kF32) {
      if (head_dim == 64) WARP_LAUNCH(float, 64); else if (head_dim == 128) WARP_LAUNCH(float, 128); else WARP_LAUNCH(float, 256);
    } else {
      if (head_dim == 64) WARP_LAUNCH(__nv_bfloat16, 64); else if (head_dim == 128) WARP_LAUNCH(__nv_bfloat16, 128); else WARP_LAUNCH(__nv_bfloat16, 256);
    }
#undef WARP_LAUNCH
    return static_cast<int>(launch_status);
  }
  int threads = 32;
  while (threads < head_dim && threads < 256) threads <<= 1;
  dim3 grid(tokens, heads + 2 * kv_heads);
  const size_t shared = static_cast<size_t>(head_dim) * sizeof(float);
  if (dtype == kF32)
    qk_norm_rope_cache_kernel<float><<<grid, threads, shared, stream>>>(
        static_cast<const float*>(q_in), static_cast<const float*>(k_in), static_cast<const float*>(v_in),
        q_stride, k_stride, v_stride, static_cast<float*>(q_out), static_cast<float*>(cache), slots,
        positions, q_weight, k_weight, cos_table, sin_table, table_positions, rotary_dim, heads,
        kv_heads, head_dim, page_tokens, num_pages, eps, status);
  else if (dtype == kBF16)
    qk_norm_rope_cache_kernel<__nv_bfloat16><<<grid, threads, shared, stream>>>(
        static_cast<const __nv_bfloat16*>(q_in), static_cast<const __nv_bfloat16*>(k_in),
        static_cast<const __nv_bfloat16*>(v_in), q_stride, k_stride, v_stride,
        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(cache), slots, positions,
        q_weight, k_weight, cos_table, sin_table, table_positions, rotary_dim, heads, kv_heads,
        head_dim, page_tokens, num_pages, eps, status);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}

MXB_TIMELINE_EXPORT(mxb_timeline_qk_rope)
