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
// word and ids[r] = -1. Two kernels: a row is cut into pieces, a block finds
// the first maximum of its piece (one block per row read a 150,000-word row
// at a fraction of what memory gives: 64 us for eight rows), and one warp per
// row picks among the pieces' results. Both are launched through
// launch_chained(): the logits are the output of the kernel ahead.
constexpr int kArgmaxThreads = 256;
constexpr int kArgmaxPieces = 64;   // at most; pieces[row][piece] = (value, index), index -1: a non-finite value

__device__ __forceinline__ void take(float v, int i, float& best, int& best_i, bool& bad) {
  bad = bad || !isfinite(v);
  if (better(v, i, best, best_i)) { best = v; best_i = i; }
}

__global__ void __launch_bounds__(kArgmaxThreads)
argmax_pieces_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int piece_size,
                     Best* __restrict__ pieces) {
  __shared__ float s_value[kArgmaxThreads / 32];
  __shared__ int s_index[kArgmaxThreads / 32];
  __shared__ int s_bad;
  chain_release();
  const int begin = blockIdx.x * piece_size;   // a multiple of 4
  const int end = min(vocab, begin + piece_size);
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  chain_wait();
  const float* row = behind_wait(logits) + blockIdx.y * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const int whole = begin + (end - begin) / 4 * 4;
    for (int i = begin + threadIdx.x * 4; i < whole; i += kArgmaxThreads * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      take(v.x, i, best, best_i, bad);
      take(v.y, i + 1, best, best_i, bad);
      take(v.z, i + 2, best, best_i, bad);
      take(v.w, i + 3, best, best_i, bad);
    }
    for (int i = whole + threadIdx.x; i < end; i += kArgmaxThreads) take(row[i], i, best, best_i, bad);
  } else {
    for (int i = begin + threadIdx.x; i < end; i += kArgmaxThreads) take(row[i], i, best, best_i, bad);
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
    best = lane < kArgmaxThreads / 32 ? s_value[lane] : -INFINITY;
    best_i = lane < kArgmaxThreads / 32 ? s_index[lane] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (lane == 0) {
      Best result;
      result.value = best;
      result.index = s_bad ? -1 : best_i;
      pieces[blockIdx.y * gridDim.x + blockIdx.x] = result;
    }
  }
}

__global__ void __launch_bounds__(32)
argmax_pick_kernel(const Best* __restrict__ pieces, int piece_count, int* __restrict__ ids, int* status) {
  chain_release();
  chain_wait();
  const Best* mine = behind_wait(pieces) + blockIdx.x * piece_count;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int p = threadIdx.x; p < piece_count; p += 32) {
    const Best piece = mine[p];
    bad = bad || piece.index < 0;
    if (piece.index >= 0 && better(piece.value, piece.index, best, best_i)) { best = piece.value; best_i = piece.index; }
  }
  bad = __any_sync(0xffffffffu, bad);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (better(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  if (threadIdx.x == 0) {
    if (bad) { atomicOr(status, kStatusNonFinite); ids[blockIdx.x] = -1; }
    else ids[blockIdx.x] = best_i;
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

// Pieces a row is cut into: enough blocks to fill the device twice over, at
// least 1,024 values each, at most kArgmaxPieces.
MXB_API int mxb_argmax_pieces(int rows, int vocab) {
  int pieces = (2 * 148 + rows - 1) / (rows > 0 ? rows : 1);
  const int most = vocab / 1024 > 1 ? vocab / 1024 : 1;
  if (pieces > most) pieces = most;
  if (pieces > kArgmaxPieces) pieces = kArgmaxPieces;
  return pieces < 1 ? 1 : pieces;
}

// scratch: rows * mxb_argmax_pieces(rows, vocab) pairs of (float, int), 8-byte aligned.
MXB_API int mxb_argmax(const float* logits, long long row_stride, int rows, int vocab, int* ids, void* scratch,
                       int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || scratch == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  const int pieces = mxb_argmax_pieces(rows, vocab);
  const int piece_size = ((vocab + pieces - 1) / pieces + 3) / 4 * 4;
  cudaError_t e = launch_chained(argmax_pieces_kernel, dim3(pieces, rows), dim3(kArgmaxThreads), 0, stream, logits,
                                 row_stride, vocab, piece_size, static_cast<Best*>(scratch));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_chained(argmax_pick_kernel, dim3(rows), dim3(32), 0, stream,
                                         static_cast<const Best*>(scratch), pieces, ids, status));
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
