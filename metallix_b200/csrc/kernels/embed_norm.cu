// Token embedding, RMSNorm and the fused residual-sum + RMSNorm.
//
// The residual stream is float32 in both precisions; the sum of squares and
// the scale are float32 always. Replaces the reference's take_axis
// (crates/models/qwen/src/forward/projection.rs:208-216) and
// fast::rms_norm (crates/models/qwen/src/forward.rs:2442-2449) calls.
#include "common.cuh"

namespace mxb {

static bool g_chained_launches = false;
static unsigned g_chained_block_limit = 0xffffffffu;
static unsigned long long g_chained_byte_limit = 24ull << 20;
bool chained_launches() { return g_chained_launches; }
unsigned chained_block_limit() { return g_chained_block_limit; }
unsigned long long chained_byte_limit() { return g_chained_byte_limit; }

// out[t, :] = table[ids[t], :] as float32. A bad id sets the status word and
// writes zeros.
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int hidden, int vocab, int* status) {
  chain_release();
  chain_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  if (!ok && threadIdx.x == 0) atomicOr(status, kStatusBadTokenId);
  const T* row = table + static_cast<size_t>(ok ? id : 0) * hidden;
  float* dst = out + static_cast<size_t>(t) * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_float(row[i]) : 0.0f;
}

// y[r, :] = x[src(r), :] * rsqrt(mean(x^2) + eps) * w, one block per row.
// rows_index (optional) gathers the rows to normalise.
template <typename TIn, typename TOut>
__global__ void rmsnorm_kernel(TOut* __restrict__ y, const TIn* __restrict__ x,
                               const float* __restrict__ w, const int* __restrict__ rows_index,
                               int size, float eps) {
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  const size_t src = rows_index ? static_cast<size_t>(rows_index[r]) : static_cast<size_t>(r);
  const TIn* row = x + src * size;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float v = to_float(row[i]);
    sum += v * v;
  }
  sum = block_sum(sum, scratch);
  const float scale = rsqrtf(sum / static_cast<float>(size) + eps);
  TOut* dst = y + static_cast<size_t>(r) * size;
  for (int i = threadIdx.x; i < size; i += blockDim.x)
    dst[i] = from_float<TOut>(to_float(row[i]) * scale * w[i]);
}

// x[r, :] += delta[r, :] (float32 sum), then y[r, :] = RMSNorm(x[r, :]) * w.
template <typename TDelta, typename TOut>
__global__ void add_rmsnorm_kernel(float* __restrict__ x, const TDelta* __restrict__ delta,
                                   TOut* __restrict__ y, const float* __restrict__ w, int size,
                                   float eps) {
  __shared__ float scratch[33];
  const size_t base = static_cast<size_t>(blockIdx.x) * size;
  float sum = 0.0f;
  for (int i = threadIdx.x; i < size; i += blockDim.x) {
    const float v = x[base + i] + to_float(delta[base + i]);
    x[base + i] = v;
    sum += v * v;
  }
  sum = block_sum(sum, scratch);
  const float scale = rsqrtf(sum / static_cast<float>(size) + eps);
  for (int i = threadIdx.x; i < size; i += blockDim.x)
    y[base + i] = from_float<TOut>(x[base + i] * scale * w[i]);
}

// Four values per thread at a time (rows whose width is a multiple of 4 and
// that start on 16-byte boundaries).
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  return make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                     __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&lo);
  raw.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same sums in the same order per thread as the scalar kernels would make
// with a quarter of the threads: thread t owns elements 4t .. 4t + 3 of every
// stride.
template <typename TDelta, typename TOut, bool ADD>
__global__ void add_rmsnorm_vec4_kernel(float* __restrict__ x, const TDelta* __restrict__ delta,
                                        TOut* __restrict__ y, const float* __restrict__ w,
                                        const int* __restrict__ rows_index, int size, float eps) {
  __shared__ float scratch[33];
  chain_release();
  const size_t src = rows_index ? static_cast<size_t>(rows_index[blockIdx.x]) : static_cast<size_t>(blockIdx.x);
  float* row = x + src * size;
  const int first = threadIdx.x * 4;
  // The thread's first four values stay in registers between the two passes
  // (for rows up to 4 * blockDim.x wide that is all of them); the norm weights
  // are fetched before waiting for the kernel that produces x.
  float4 held = make_float4(0.0f, 0.0f, 0.0f, 0.0f), held_gain = held;
  if (first < size) held_gain = load4(w + first);
  chain_wait();
  row = behind_wait(row);      // both written by kernels ahead of this one
  delta = behind_wait(delta);
  float sum = 0.0f;
  for (int i = first; i < size; i += blockDim.x * 4) {
    float4 v = load4(row + i);
    if (ADD) {
      const float4 d = load4(delta + src * size + i);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      store4(row + i, v);
    }
    if (i == first) held = v;
    sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  sum = block_sum(sum, scratch);
  const float scale = rsqrtf(sum / static_cast<float>(size) + eps);
  TOut* dst = y + static_cast<size_t>(blockIdx.x) * size;
  for (int i = first; i < size; i += blockDim.x * 4) {
    const float4 v = i == first ? held : load4(row + i);
    const float4 g = i == first ? held_gain : load4(w + i);
    store4(dst + i, make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w));
  }
}

// x += summands[0] + summands[1] + ... (in that order), then the norm: the
// summands are [parts, rows, size] float32, what a producer left that splits
// its sum over k into parts (the output projection taken head by head).
template <typename TOut, bool VEC4>
__global__ void __launch_bounds__(256)   // what norm_threads() gives at most: room for a batch of loads in registers
add_summands_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ summands, int parts,
                                            size_t part_stride, TOut* __restrict__ y, const float* __restrict__ w,
                                            int size, float eps) {
  __shared__ float scratch[33];
  chain_release();
  constexpr int V = VEC4 ? 4 : 1;
  constexpr int BATCH = 16;  // parts whose loads are on their way before the first of them is added
  float* row = x + static_cast<size_t>(blockIdx.x) * size;
  const int first = threadIdx.x * V;
  // As in the kernel above: the thread's first values stay in registers
  // between the passes, the norm weights come before the wait.
  float4 held = make_float4(0.0f, 0.0f, 0.0f, 0.0f), held_gain = held;
  if (VEC4 && first < size) held_gain = load4(w + first);
  chain_wait();
  row = behind_wait(row);      // both written by kernels ahead of this one
  summands = behind_wait(summands) + static_cast<size_t>(blockIdx.x) * size;
  float sum = 0.0f;
  for (int i = first; i < size; i += blockDim.x * V) {
    if (VEC4) {
      // The adds wait for their loads in order: a loop of one load and one add
      // would make a trip to memory per part.
      float4 v = load4(row + i);
      float4 d = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      for (int part = 0; part < parts; part += BATCH) {
        float4 more[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j)
          more[j] = load4(summands + min(part + j, parts - 1) * part_stride + i);   // no branch around a load
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
          if (part + j < parts) {
            d.x += more[j].x; d.y += more[j].y; d.z += more[j].z; d.w += more[j].w;
          }
        }
      }
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
      store4(row + i, v);
      if (i == first) held = v;
      sum += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    } else {
      float d = 0.0f;
      for (int part = 0; part < parts; part += BATCH) {
        float more[BATCH];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) more[j] = summands[min(part + j, parts - 1) * part_stride + i];
#pragma unroll
        for (int j = 0; j < BATCH; ++j)
          if (part + j < parts) d += more[j];
      }
      const float v = row[i] + d;
      row[i] = v;
      sum += v * v;
    }
  }
  sum = block_sum(sum, scratch);
  const float scale = rsqrtf(sum / static_cast<float>(size) + eps);
  TOut* dst = y + static_cast<size_t>(blockIdx.x) * size;
  for (int i = first; i < size; i += blockDim.x * V) {
    if (VEC4) {
      const float4 v = i == first ? held : load4(row + i);
      const float4 g = i == first ? held_gain : load4(w + i);
      store4(dst + i, make_float4(v.x * scale * g.x, v.y * scale * g.y, v.z * scale * g.z, v.w * scale * g.w));
    } else {
      dst[i] = from_float<TOut>(row[i] * scale * w[i]);
    }
  }
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

// x[r, :] += delta[r, :] alone (the last residual sum of a model).
template <typename TDelta>
__global__ void add_kernel(float* __restrict__ x, const TDelta* __restrict__ delta, size_t count) {
  chain_release();
  chain_wait();
  x = behind_wait(x);
  delta = behind_wait(delta);
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) x[i] += to_float(delta[i]);
}

static int norm_threads(int size) {
  int threads = 32;
  while (threads < size && threads < 1024) threads <<= 1;
  // A fixed block size per row width keeps the order of additions, and so the
  // result, the same whatever else is in the batch.
  return threads > 256 ? 256 : threads;
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_embed(float* out, const void* table, int table_dtype, const int* ids, int tokens,
                      int hidden, int vocab, int* status, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int threads = hidden >= 256 ? 256 : 128;
  if (table_dtype == kF32)
    return static_cast<int>(launch_chained(embed_kernel<float>, dim3(tokens), dim3(threads), 0, stream, out,
                                           static_cast<const float*>(table), ids, hidden, vocab, status));
  return static_cast<int>(launch_chained(embed_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, out,
                                         static_cast<const __nv_bfloat16*>(table), ids, hidden, vocab, status));
}

MXB_API int mxb_rmsnorm(void* y, int y_dtype, const void* x, int x_dtype, const float* w,
                        const int* rows_index, int rows, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (x_dtype == kF32 && size % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(w)) {
    const int vec_threads = norm_threads(size / 4);
    float* xs = const_cast<float*>(static_cast<const float*>(x));  // read only: ADD is false
    if (y_dtype == kF32)
      return static_cast<int>(launch_chained(add_rmsnorm_vec4_kernel<float, float, false>, dim3(rows), dim3(vec_threads), 0,
                                             stream, xs, static_cast<const float*>(nullptr), static_cast<float*>(y), w, rows_index, size, eps));
    if (y_dtype == kBF16)
      return static_cast<int>(launch_chained(add_rmsnorm_vec4_kernel<float, __nv_bfloat16, false>, dim3(rows), dim3(vec_threads), 0,
                                             stream, xs, static_cast<const float*>(nullptr), static_cast<__nv_bfloat16*>(y), w, rows_index, size, eps));
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const int threads = norm_threads(size);
#define LAUNCH(TI, TO) rmsnorm_kernel<TI, TO><<<rows, threads, 0, stream>>>( \
      static_cast<TO*>(y), static_cast<const TI*>(x), w, rows_index, size, eps)
  if (x_dtype == kF32 && y_dtype == kF32) LAUNCH(float, float);
  else if (x_dtype == kF32 && y_dtype == kBF16) LAUNCH(float, __nv_bfloat16);
  else if (x_dtype == kBF16 && y_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == kBF16 && y_dtype == kF32) LAUNCH(__nv_bfloat16, float);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_add_rmsnorm(float* x, const void* delta, int delta_dtype, void* y, int y_dtype,
                            const float* w, int rows, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (size % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(w) && aligned16(delta) &&
      (delta_dtype == kF32 || size % 8 == 0)) {
    const int vec_threads = norm_threads(size / 4);
#define VEC(TD, TO) return static_cast<int>(launch_chained(add_rmsnorm_vec4_kernel<TD, TO, true>, dim3(rows), dim3(vec_threads), \
        0, stream, x, static_cast<const TD*>(delta), static_cast<TO*>(y), w, static_cast<const int*>(nullptr), size, eps))
    if (delta_dtype == kF32 && y_dtype == kF32) VEC(float, float);
    if (delta_dtype == kBF16 && y_dtype == kBF16) VEC(__nv_bfloat16, __nv_bfloat16);
    if (delta_dtype == kF32 && y_dtype == kBF16) VEC(float, __nv_bfloat16);
    if (delta_dtype == kBF16 && y_dtype == kF32) VEC(__nv_bfloat16, float);
#undef VEC
    return static_cast<int>(cudaErrorInvalidValue);
  }
  const int threads = norm_threads(size);
#define LAUNCH(TD, TO) add_rmsnorm_kernel<TD, TO><<<rows, threads, 0, stream>>>( \
      x, static_cast<const TD*>(delta), static_cast<TO*>(y), w, size, eps)
  if (delta_dtype == kF32 && y_dtype == kF32) LAUNCH(float, float);
  else if (delta_dtype == kBF16 && y_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == kF32 && y_dtype == kBF16) LAUNCH(float, __nv_bfloat16);
  else if (delta_dtype == kBF16 && y_dtype == kF32) LAUNCH(__nv_bfloat16, float);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

// x[r, :] += sum over parts of summands[part, r, :], y = RMSNorm(x) * w.
MXB_API int mxb_add_summands_rmsnorm(float* x, const float* summands, int parts, void* y, int y_dtype,
                                     const float* w, int rows, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (parts <= 0 || size <= 0 || (y_dtype != kF32 && y_dtype != kBF16)) return static_cast<int>(cudaErrorInvalidValue);
  const size_t part_stride = static_cast<size_t>(rows) * size;
  const bool vec4 = size % 4 == 0 && aligned16(x) && aligned16(summands) && aligned16(w) &&
                    (y_dtype == kF32 ? aligned16(y) : reinterpret_cast<uintptr_t>(y) % 8 == 0);
  int threads = norm_threads(vec4 ? size / 4 : size);
  if (vec4 && threads < 32) threads = 32;
#define LAUNCH(TO, VEC) launch_chained(add_summands_rmsnorm_kernel<TO, VEC>, dim3(rows), dim3(threads), 0, stream, x, \
                                       summands, parts, part_stride, static_cast<TO*>(y), w, size, eps)
  cudaError_t e;
  if (y_dtype == kF32) e = vec4 ? LAUNCH(float, true) : LAUNCH(float, false);
  else e = vec4 ? LAUNCH(__nv_bfloat16, true) : LAUNCH(__nv_bfloat16, false);
#undef LAUNCH
  return static_cast<int>(e);
}

MXB_API int mxb_add(float* x, const void* delta, int delta_dtype, long long count,
                    cudaStream_t stream) {
  if (count <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((count + threads - 1) / threads);
  if (delta_dtype == kF32)
    return static_cast<int>(launch_chained(add_kernel<float>, dim3(blocks), dim3(threads), 0, stream, x,
                                           static_cast<const float*>(delta), static_cast<size_t>(count)));
  return static_cast<int>(launch_chained(add_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, stream, x,
                                         static_cast<const __nv_bfloat16*>(delta), static_cast<size_t>(count)));
}

// Turns the overlap of consecutive kernels (programmatic dependent launch) on
// or off for every kernel of this library that supports it.
MXB_API void mxb_set_chained_launches(int enabled) { mxb::g_chained_launches = enabled != 0; }
// Grids of more blocks than `blocks`, and kernels that say they stream more
// than `megabytes`, are launched without the overlap (0: no limit).
MXB_API void mxb_set_chained_limits(unsigned blocks, unsigned megabytes) {
  mxb::g_chained_block_limit = blocks == 0 ? 0xffffffffu : blocks;
  mxb::g_chained_byte_limit = megabytes == 0 ? ~0ull : static_cast<unsigned long long>(megabytes) << 20;
}

MXB_TIMELINE_EXPORT(mxb_timeline_norms)
