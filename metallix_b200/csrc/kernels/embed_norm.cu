// Token embedding, RMSNorm and the fused residual-sum + RMSNorm.
//
// The residual stream is float32 in both precisions; the sum of squares and
// the scale are float32 always. Replaces the reference's take_axis
// (crates/models/qwen/src/forward/projection.rs:208-216) and
// fast::rms_norm (crates/models/qwen/src/forward.rs:2442-2449) calls.
#include "common.cuh"

namespace mxb {

// out[t, :] = table[ids[t], :] as float32. A bad id sets the status word and
// writes zeros.
template <typename T>
__global__ void embed_kernel(float* __restrict__ out, const T* __restrict__ table,
                             const int* __restrict__ ids, int hidden, int vocab, int* status) {
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

// x[r, :] += delta[r, :] alone (the last residual sum of a model).
template <typename TDelta>
__global__ void add_kernel(float* __restrict__ x, const TDelta* __restrict__ delta, size_t count) {
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
    embed_kernel<float><<<tokens, threads, 0, stream>>>(out, static_cast<const float*>(table), ids, hidden, vocab, status);
  else
    embed_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(out, static_cast<const __nv_bfloat16*>(table), ids, hidden, vocab, status);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_rmsnorm(void* y, int y_dtype, const void* x, int x_dtype, const float* w,
                        const int* rows_index, int rows, int size, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
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

MXB_API int mxb_add(float* x, const void* delta, int delta_dtype, long long count,
                    cudaStream_t stream) {
  if (count <= 0) return 0;
  const int threads = 256;
  const unsigned blocks = static_cast<unsigned>((count + threads - 1) / threads);
  if (delta_dtype == kF32)
    add_kernel<float><<<blocks, threads, 0, stream>>>(x, static_cast<const float*>(delta), static_cast<size_t>(count));
  else
    add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(x, static_cast<const __nv_bfloat16*>(delta), static_cast<size_t>(count));
  return static_cast<int>(cudaGetLastError());
}
