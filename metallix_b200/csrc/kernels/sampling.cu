// Token picking on the device: greedy argmax with a finite check, inverse-CDF
// temperature sampling in token-id order, and Gumbel-max ("race") sampling.
//
// Definitions follow the reference's host samplers:
//  * greedy: first maximum, a non-finite row is an error
//    (crates/app/cli/src/qwen_forward.rs:1546-1557, forward/picks.rs:286-296);
//  * inverse CDF: weights exp((f64(logit) - max) / T) in float64, target =
//    u * sum, the first id whose cumulative weight exceeds the target, else the
//    last id of positive weight (crates/core/engine/src/sampling.rs:56-103);
//  * race: argmax of f64(logit) / T + Gumbel noise from Philox4x32-10 keyed by
//    (seed, choice, generated position, id), lowest id on ties
//    (crates/core/engine/src/sampling/race.rs:1-17, :40-105).
// The uniform of the inverse-CDF sampler is a counter-based function of
// (seed, stream, generated position), so a request's tokens do not depend on
// what else is in the batch or on whether it was computed again.
#include "common.cuh"

namespace mxb {

constexpr int kPickThreads = 1024;

__device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                              uint32_t k0, uint32_t k1, uint32_t out[4]) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int round = 0; round < 10; ++round) {
    if (round > 0) { k0 += W0; k1 += W1; }
    const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
    const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
    const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
    c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// The uniform in [0, 1) of one generated position: Philox words 0 (high) and
// 1 (low), key = the seed's halves, counter = (position, stream low, stream
// high, "icdf"); the top 53 bits over 2^53 (qwen_forward.rs:551-559).
__device__ __forceinline__ double request_uniform(uint64_t seed, uint64_t stream, uint32_t position) {
  uint32_t w[4];
  philox4x32_10(position, static_cast<uint32_t>(stream), static_cast<uint32_t>(stream >> 32), 0x69636466u,
                static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32), w);
  const uint64_t word = (static_cast<uint64_t>(w[0]) << 32) | w[1];
  return static_cast<double>(word >> 11) * (1.0 / 9007199254740992.0);
}

__device__ __forceinline__ double gumbel_from_bits(uint64_t bits) {
  const double two_to_minus_64 = 1.0 / 18446744073709551616.0;
  double exponential;
  if (bits < (1ull << 63)) exponential = -log1p(-((static_cast<double>(bits) + 0.5) * two_to_minus_64));
  else exponential = -log((static_cast<double>(~bits) + 0.5) * two_to_minus_64);
  return -log(exponential);
}

struct Best {
  float value;
  int index;
};

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// ids[r] = lowest index of the row maximum; a non-finite row sets the status
// word and ids[r] = -1.
__global__ void __launch_bounds__(kPickThreads)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int* __restrict__ ids,
              int* status) {
  __shared__ float s_value[32];
  __shared__ int s_index[32];
  __shared__ int s_bad;
  const float* row = logits + blockIdx.x * row_stride;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
    const float v = row[i];
    bad = bad || !isfinite(v);
    if (better(v, i, best, best_i)) { best = v; best_i = i; }
  }
  if (bad) s_bad = 1;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_value[warp] = best; s_index[warp] = best_i; }
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    best = lane < warps ? s_value[lane] : -INFINITY;
    best_i = lane < warps ? s_index[lane] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) {
      if (s_bad) { atomicOr(status, kStatusNonFinite); ids[blockIdx.x] = -1; }
      else ids[blockIdx.x] = best_i;
    }
  }
}

// Inverse-CDF sampling of one row per block. Thread t owns the contiguous ids
// [t * chunk, (t + 1) * chunk), sums its weights in id order in float64, the
// block scans the chunk sums in thread order, and the owner of the target
// walks its chunk again.
__global__ void __launch_bounds__(kPickThreads)
sample_icdf_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                   const double* __restrict__ temperature, const unsigned long long* __restrict__ seed,
                   const unsigned long long* __restrict__ stream, const int* __restrict__ position,
                   const unsigned char* __restrict__ legal, int* __restrict__ ids, int* status) {
  __shared__ double s_sum[kPickThreads];
  __shared__ float s_max[32];
  __shared__ int s_flag[3];  // bad row, owner thread, last positive id
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + r * row_stride;
  const unsigned char* mask = legal ? legal + static_cast<size_t>(r) * vocab : nullptr;
  if (tid == 0) { s_flag[0] = 0; s_flag[1] = 0x7fffffff; s_flag[2] = -1; }
  __syncthreads();

  float local_max = -INFINITY;
  bool bad = false;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    bad = bad || !isfinite(v);
    if (!mask || mask[i]) local_max = fmaxf(local_max, v);
  }
  if (bad) s_flag[0] = 1;
  local_max = warp_max(local_max);
  if ((tid & 31) == 0) s_max[tid >> 5] = local_max;
  __syncthreads();
  if (tid < 32) {
    float v = tid < (blockDim.x >> 5) ? s_max[tid] : -INFINITY;
    v = warp_max(v);
    if (tid == 0) s_max[0] = v;
  }
  __syncthreads();
  if (s_flag[0] || s_max[0] == -INFINITY) {  // non-finite logits or an empty legal set
    if (tid == 0) { atomicOr(status, kStatusNonFinite); ids[r] = -1; }
    return;
  }
  const double maximum = static_cast<double>(s_max[0]);
  const double inv_t = 1.0 / temperature[r];
  const int chunk = (vocab + blockDim.x - 1) / blockDim.x;
  const int begin = min(vocab, tid * chunk), end = min(vocab, begin + chunk);

  double sum = 0.0;
  int last_positive = -1;
  for (int i = begin; i < end; ++i) {
    if (mask && !mask[i]) continue;
    const double w = exp((static_cast<double>(row[i]) - maximum) * inv_t);
    sum += w;
    if (w > 0.0) last_positive = i;
  }
  s_sum[tid] = sum;
  if (last_positive >= 0) atomicMax(&s_flag[2], last_positive);
  __syncthreads();
  // Exclusive prefix of the chunk sums in thread order (one thread: 1024
  // additions, the same order for every row and batch).
  __shared__ double s_total;
  if (tid == 0) {
    double running = 0.0;
    for (int t = 0; t < blockDim.x; ++t) {
      const double v = s_sum[t];
      s_sum[t] = running;
      running += v;
    }
    s_total = running;
  }
  __syncthreads();
  const double target = request_uniform(seed[r], stream[r], static_cast<uint32_t>(position[r])) * s_total;
  const double before = s_sum[tid];
  if (sum > 0.0 && target < before + sum) atomicMin(&s_flag[1], tid);
  __syncthreads();
  if (s_flag[1] == 0x7fffffff) {  // rounding left the target beyond the total
    if (tid == 0) ids[r] = s_flag[2];
    return;
  }
  if (tid != s_flag[1]) return;
  double cumulative = before;
  int picked = last_positive;
  for (int i = begin; i < end; ++i) {
    if (mask && !mask[i]) continue;
    cumulative += exp((static_cast<double>(row[i]) - maximum) * inv_t);
    if (target < cumulative) { picked = i; break; }
  }
  ids[r] = picked;
}

// Gumbel-max sampling of one row per block.
__global__ void __launch_bounds__(kPickThreads)
sample_race_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                   const double* __restrict__ temperature, const unsigned long long* __restrict__ seed,
                   const int* __restrict__ position, const unsigned char* __restrict__ legal,
                   int* __restrict__ ids, int* status) {
  __shared__ double s_value[32];
  __shared__ int s_index[32];
  __shared__ int s_bad;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + r * row_stride;
  const unsigned char* mask = legal ? legal + static_cast<size_t>(r) * vocab : nullptr;
  if (tid == 0) s_bad = 0;
  __syncthreads();
  const double inv_t = 1.0 / temperature[r];
  const uint32_t k0 = static_cast<uint32_t>(seed[r]), k1 = static_cast<uint32_t>(seed[r] >> 32);
  const uint32_t pos = static_cast<uint32_t>(position[r]);
  double best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    bad = bad || !isfinite(v);
    if (mask && !mask[i]) continue;
    uint32_t w[4];
    philox4x32_10(static_cast<uint32_t>(i) >> 1, pos, 0u, 0x72616365u, k0, k1, w);
    const uint64_t bits = (i & 1) ? ((static_cast<uint64_t>(w[2]) << 32) | w[3])
                                  : ((static_cast<uint64_t>(w[0]) << 32) | w[1]);
    const double score = static_cast<double>(v) * inv_t + gumbel_from_bits(bits);
    if (score > best || (score == best && i < best_i)) { best = score; best_i = i; }
  }
  if (bad) s_bad = 1;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const double ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
  }
  if ((tid & 31) == 0) { s_value[tid >> 5] = best; s_index[tid >> 5] = best_i; }
  __syncthreads();
  if (tid < 32) {
    const int warps = blockDim.x >> 5;
    best = tid < warps ? s_value[tid] : -INFINITY;
    best_i = tid < warps ? s_index[tid] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const double ov = __shfl_xor_sync(0xffffffffu, best, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if (tid == 0) {
      if (s_bad || best_i == 0x7fffffff) { atomicOr(status, kStatusNonFinite); ids[r] = -1; }
      else ids[r] = best_i;
    }
  }
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_argmax(const float* logits, long long row_stride, int rows, int vocab, int* ids,
                       int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  argmax_kernel<<<rows, kPickThreads, 0, stream>>>(logits, row_stride, vocab, ids, status);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_sample_icdf(const float* logits, long long row_stride, int rows, int vocab,
                            const double* temperature, const unsigned long long* seed,
                            const unsigned long long* stream_id, const int* position,
                            const unsigned char* legal, int* ids, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  sample_icdf_kernel<<<rows, kPickThreads, 0, stream>>>(logits, row_stride, vocab, temperature, seed,
                                                        stream_id, position, legal, ids, status);
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_sample_race(const float* logits, long long row_stride, int rows, int vocab,
                            const double* temperature, const unsigned long long* seed,
                            const int* position, const unsigned char* legal, int* ids, int* status,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  sample_race_kernel<<<rows, kPickThreads, 0, stream>>>(logits, row_stride, vocab, temperature, seed,
                                                        position, legal, ids, status);
  return static_cast<int>(cudaGetLastError());
}
