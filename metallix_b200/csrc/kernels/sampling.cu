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

// Inverse-CDF sampling. A row is cut into pieces of kIcdfPiece ids, whatever
// the batch is, so that the grouping of the float64 sums, and with it every
// rounding, is a function of the row alone. Three kernels: the maximum over
// the legal ids of every piece; the weight of every piece (thread t of a
// block owns kIcdfPiece / 256 consecutive ids and adds their weights in id
// order, thread 0 adds the threads' sums in thread order); and the pick: one
// thread walks the pieces' sums in order up to the piece that holds the
// target, the block repeats that piece's sums and the thread that holds the
// target walks its ids.
constexpr int kIcdfPiece = 2048;
constexpr int kIcdfThreads = 256;
constexpr int kIcdfOwn = kIcdfPiece / kIcdfThreads;   // ids of a thread

__global__ void __launch_bounds__(kIcdfThreads)
icdf_max_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                const unsigned char* __restrict__ legal, Best* __restrict__ maxima) {
  __shared__ float s_max[kIcdfThreads / 32];
  __shared__ int s_bad;
  chain_release();
  const int r = blockIdx.y, tid = threadIdx.x;
  if (tid == 0) s_bad = 0;
  __syncthreads();
  chain_wait();
  const float* row = behind_wait(logits) + r * row_stride;
  const unsigned char* mask = legal ? behind_wait(legal) + static_cast<size_t>(r) * vocab : nullptr;
  const int begin = blockIdx.x * kIcdfPiece, end = min(vocab, begin + kIcdfPiece);
  float local_max = -INFINITY;
  bool bad = false;
  for (int i = begin + tid; i < end; i += kIcdfThreads) {
    const float v = row[i];
    bad = bad || !isfinite(v);
    if (!mask || mask[i]) local_max = fmaxf(local_max, v);
  }
  if (bad) s_bad = 1;
  local_max = warp_max(local_max);
  if ((tid & 31) == 0) s_max[tid >> 5] = local_max;
  __syncthreads();
  if (tid < 32) {
    float v = tid < kIcdfThreads / 32 ? s_max[tid] : -INFINITY;
    v = warp_max(v);
    if (tid == 0) {
      Best result;
      result.value = v;
      result.index = s_bad ? -1 : 0;
      maxima[r * gridDim.x + blockIdx.x] = result;
    }
  }
}

// The row's maximum over its legal ids from the pieces' maxima; false for a
// row with a non-finite logit or without a legal id. Every thread of the
// block gets the same answer.
__device__ __forceinline__ bool icdf_row_maximum(const Best* maxima, int pieces, float& maximum) {
  float best = -INFINITY;
  bool bad = false;
  for (int p = 0; p < pieces; ++p) {
    const Best piece = maxima[p];
    bad = bad || piece.index < 0;
    best = fmaxf(best, piece.value);
  }
  maximum = best;
  return !bad && best != -INFINITY;
}

// This thread's ids of the piece: their weights' sum in id order and the last id of positive weight.
__device__ __forceinline__ double icdf_own_sum(const float* row, const unsigned char* mask, int begin, int end,
                                               double maximum, double inv_t, int& last_positive) {
  double sum = 0.0;
  last_positive = -1;
  for (int i = begin; i < end; ++i) {
    if (mask && !mask[i]) continue;
    const double w = exp((static_cast<double>(row[i]) - maximum) * inv_t);
    sum += w;
    if (w > 0.0) last_positive = i;
  }
  return sum;
}

__global__ void __launch_bounds__(kIcdfThreads)
icdf_sum_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                const double* __restrict__ temperature, const unsigned char* __restrict__ legal,
                const Best* __restrict__ maxima, double* __restrict__ sums, int* __restrict__ lasts) {
  __shared__ double s_sum[kIcdfThreads];
  __shared__ int s_last;
  chain_release();
  const int r = blockIdx.y, tid = threadIdx.x, pieces = gridDim.x;
  if (tid == 0) s_last = -1;
  __syncthreads();
  chain_wait();
  float maximum;
  if (!icdf_row_maximum(behind_wait(maxima) + r * pieces, pieces, maximum)) return;   // the pick reports it
  const float* row = behind_wait(logits) + r * row_stride;
  const unsigned char* mask = legal ? behind_wait(legal) + static_cast<size_t>(r) * vocab : nullptr;
  const int begin = min(vocab, blockIdx.x * kIcdfPiece + tid * kIcdfOwn);
  const int end = min(vocab, begin + kIcdfOwn);
  int last_positive;
  s_sum[tid] = icdf_own_sum(row, mask, begin, end, static_cast<double>(maximum), 1.0 / temperature[r], last_positive);
  if (last_positive >= 0) atomicMax(&s_last, last_positive);
  __syncthreads();
  if (tid == 0) {
    double running = 0.0;
    for (int t = 0; t < kIcdfThreads; ++t) running += s_sum[t];   // thread order: one order of additions
    sums[r * pieces + blockIdx.x] = running;
    lasts[r * pieces + blockIdx.x] = s_last;
  }
}

__global__ void __launch_bounds__(kIcdfThreads)
icdf_pick_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int pieces,
                 const double* __restrict__ temperature, const unsigned long long* __restrict__ seed,
                 const unsigned long long* __restrict__ stream, const int* __restrict__ position,
                 const unsigned char* __restrict__ legal, const Best* __restrict__ maxima,
                 const double* __restrict__ sums, const int* __restrict__ lasts, int* __restrict__ ids,
                 int* status) {
  __shared__ double s_sum[kIcdfThreads];
  __shared__ double s_target, s_before;
  __shared__ int s_piece, s_owner, s_last;
  chain_release();
  const int r = blockIdx.x, tid = threadIdx.x;
  chain_wait();
  float maximum;
  if (!icdf_row_maximum(behind_wait(maxima) + r * pieces, pieces, maximum)) {  // non-finite logits or an empty legal set
    if (tid == 0) { atomicOr(status, kStatusNonFinite); ids[r] = -1; }
    return;
  }
  const double* row_sums = behind_wait(sums) + r * pieces;
  const int* row_lasts = behind_wait(lasts) + r * pieces;
  // The pieces' sums into shared memory, all threads at once: the one thread
  // that walks them would otherwise wait for memory at every step it takes.
  extern __shared__ double s_piece_sums[];   // [pieces]
  int last_here = -1;
  for (int p = tid; p < pieces; p += kIcdfThreads) {
    s_piece_sums[p] = row_sums[p];
    last_here = max(last_here, row_lasts[p]);
  }
  if (tid == 0) s_last = -1;
  __syncthreads();
  if (last_here >= 0) atomicMax(&s_last, last_here);
  __syncthreads();
  if (tid == 0) {
    double total = 0.0;
    for (int p = 0; p < pieces; ++p) total += s_piece_sums[p];   // piece order: one order of additions
    const double target = request_uniform(seed[r], stream[r], static_cast<uint32_t>(position[r])) * total;
    double before = 0.0;
    int piece = -1;
    for (int p = 0; p < pieces; ++p) {
      const double sum = s_piece_sums[p];
      if (sum > 0.0 && target < before + sum) { piece = p; break; }
      before += sum;
    }
    s_target = target;
    s_before = before;
    s_piece = piece;
    s_owner = 0x7fffffff;
  }
  __syncthreads();
  if (s_piece < 0) {  // rounding left the target beyond the total: the last id of positive weight
    if (tid == 0) ids[r] = s_last;
    return;
  }
  const float* row = logits + r * row_stride;
  const unsigned char* mask = legal ? legal + static_cast<size_t>(r) * vocab : nullptr;
  const double inv_t = 1.0 / temperature[r];
  const int begin = min(vocab, s_piece * kIcdfPiece + tid * kIcdfOwn);
  const int end = min(vocab, begin + kIcdfOwn);
  int last_positive;
  const double sum = icdf_own_sum(row, mask, begin, end, static_cast<double>(maximum), inv_t, last_positive);
  s_sum[tid] = sum;
  __syncthreads();
  if (tid == 0) {
    double running = s_before;
    for (int t = 0; t < kIcdfThreads; ++t) {
      const double v = s_sum[t];
      s_sum[t] = running;   // what lies in front of thread t
      if (s_owner == 0x7fffffff && v > 0.0 && s_target < running + v) s_owner = t;
      running += v;
    }
  }
  __syncthreads();
  if (s_owner == 0x7fffffff) {  // the same rounding inside the piece: its last id of positive weight
    if (tid == 0) ids[r] = row_lasts[s_piece];
    return;
  }
  if (tid != s_owner) return;
  double cumulative = s_sum[tid];
  int picked = last_positive;
  for (int i = begin; i < end; ++i) {
    if (mask && !mask[i]) continue;
    cumulative += exp((static_cast<double>(row[i]) - static_cast<double>(maximum)) * inv_t);
    if (s_target < cumulative) { picked = i; break; }
  }
  ids[r] = picked;
}

// Gumbel-max sampling, in pieces like the greedy pick: a block finds the best
// score of its piece, one warp per row picks among the pieces. One Philox call
// yields the noise of an even id and of the odd id after it.
struct BestScore {
  double value;
  int index;   // -1: a non-finite logit in the piece; 0x7fffffff: no legal id in it
  int unused;
};

__device__ __forceinline__ bool better_score(double v, int i, double bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

__global__ void __launch_bounds__(kArgmaxThreads)
race_pieces_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int piece_size,
                   const double* __restrict__ temperature, const unsigned long long* __restrict__ seed,
                   const int* __restrict__ position, const unsigned char* __restrict__ legal,
                   BestScore* __restrict__ pieces) {
  __shared__ double s_value[kArgmaxThreads / 32];
  __shared__ int s_index[kArgmaxThreads / 32];
  __shared__ int s_bad;
  chain_release();
  const int r = blockIdx.y, tid = threadIdx.x;
  if (tid == 0) s_bad = 0;
  __syncthreads();
  const double inv_t = 1.0 / temperature[r];
  const uint32_t k0 = static_cast<uint32_t>(seed[r]), k1 = static_cast<uint32_t>(seed[r] >> 32);
  const uint32_t pos = static_cast<uint32_t>(position[r]);
  const int begin = blockIdx.x * piece_size, end = min(vocab, begin + piece_size);   // begin is even
  chain_wait();
  const float* row = behind_wait(logits) + r * row_stride;
  const unsigned char* mask = legal ? behind_wait(legal) + static_cast<size_t>(r) * vocab : nullptr;
  double best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int i = begin + 2 * tid; i < end; i += 2 * kArgmaxThreads) {
    uint32_t w[4];
    philox4x32_10(static_cast<uint32_t>(i) >> 1, pos, 0u, 0x72616365u, k0, k1, w);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int id = i + half;
      if (id >= end) break;
      const float v = row[id];
      bad = bad || !isfinite(v);
      if (mask && !mask[id]) continue;
      const uint64_t bits = (static_cast<uint64_t>(w[2 * half]) << 32) | w[2 * half + 1];
      const double score = static_cast<double>(v) * inv_t + gumbel_from_bits(bits);
      if (better_score(score, id, best, best_i)) { best = score; best_i = id; }
    }
  }
  if (bad) s_bad = 1;
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const double ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (better_score(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  if ((tid & 31) == 0) { s_value[tid >> 5] = best; s_index[tid >> 5] = best_i; }
  __syncthreads();
  if (tid < 32) {
    best = tid < kArgmaxThreads / 32 ? s_value[tid] : -INFINITY;
    best_i = tid < kArgmaxThreads / 32 ? s_index[tid] : 0x7fffffff;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const double ov = __shfl_xor_sync(0xffffffffu, best, offset);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
      if (better_score(ov, oi, best, best_i)) { best = ov; best_i = oi; }
    }
    if (tid == 0) {
      BestScore result;
      result.value = best;
      result.index = s_bad ? -1 : best_i;
      result.unused = 0;
      pieces[r * gridDim.x + blockIdx.x] = result;
    }
  }
}

__global__ void __launch_bounds__(32)
race_pick_kernel(const BestScore* __restrict__ pieces, int piece_count, int* __restrict__ ids, int* status) {
  chain_release();
  chain_wait();
  const BestScore* mine = behind_wait(pieces) + blockIdx.x * piece_count;
  double best = -INFINITY;
  int best_i = 0x7fffffff;
  bool bad = false;
  for (int p = threadIdx.x; p < piece_count; p += 32) {
    const BestScore piece = mine[p];
    bad = bad || piece.index < 0;
    if (piece.index >= 0 && better_score(piece.value, piece.index, best, best_i)) { best = piece.value; best_i = piece.index; }
  }
  bad = __any_sync(0xffffffffu, bad);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const double ov = __shfl_xor_sync(0xffffffffu, best, offset);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, offset);
    if (better_score(ov, oi, best, best_i)) { best = ov; best_i = oi; }
  }
  if (threadIdx.x == 0) {
    if (bad || best_i == 0x7fffffff) { atomicOr(status, kStatusNonFinite); ids[blockIdx.x] = -1; }   // or no legal id at all
    else ids[blockIdx.x] = best_i;
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

// Pieces of a row in the inverse-CDF sampler.
MXB_API int mxb_icdf_pieces(int vocab) { return (vocab + kIcdfPiece - 1) / kIcdfPiece; }

// scratch: rows * mxb_icdf_pieces(vocab) * 3 words of 8 bytes, 8-byte aligned
// (the pieces' maxima, their sums, their last ids of positive weight).
MXB_API int mxb_sample_icdf(const float* logits, long long row_stride, int rows, int vocab,
                            const double* temperature, const unsigned long long* seed,
                            const unsigned long long* stream_id, const int* position,
                            const unsigned char* legal, int* ids, void* scratch, int* status,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || scratch == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  const int pieces = mxb_icdf_pieces(vocab);
  const size_t slots = static_cast<size_t>(rows) * pieces;
  Best* maxima = static_cast<Best*>(scratch);
  double* sums = reinterpret_cast<double*>(maxima + slots);
  int* lasts = reinterpret_cast<int*>(sums + slots);
  cudaError_t e = launch_chained(icdf_max_kernel, dim3(pieces, rows), dim3(kIcdfThreads), 0, stream, logits,
                                 row_stride, vocab, legal, maxima);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = launch_chained(icdf_sum_kernel, dim3(pieces, rows), dim3(kIcdfThreads), 0, stream, logits, row_stride, vocab,
                     temperature, legal, static_cast<const Best*>(maxima), sums, lasts);
  if (e != cudaSuccess) return static_cast<int>(e);
  const size_t pick_shared = static_cast<size_t>(pieces) * sizeof(double);
  if (pick_shared > 48 * 1024) {
    e = cudaFuncSetAttribute(icdf_pick_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pick_shared));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return static_cast<int>(launch_chained(icdf_pick_kernel, dim3(rows), dim3(kIcdfThreads), pick_shared, stream, logits,
                                         row_stride, vocab, pieces, temperature, seed, stream_id, position, legal,
                                         static_cast<const Best*>(maxima), static_cast<const double*>(sums),
                                         static_cast<const int*>(lasts), ids, status));
}

// scratch: rows * mxb_argmax_pieces(rows, vocab) * 2 words of 8 bytes, 8-byte aligned.
MXB_API int mxb_sample_race(const float* logits, long long row_stride, int rows, int vocab,
                            const double* temperature, const unsigned long long* seed, const int* position,
                            const unsigned char* legal, int* ids, void* scratch, int* status,
                            cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || scratch == nullptr) return static_cast<int>(cudaErrorInvalidValue);
  const int pieces = mxb_argmax_pieces(rows, vocab);
  const int piece_size = ((vocab + pieces - 1) / pieces + 3) / 4 * 4;
  cudaError_t e = launch_chained(race_pieces_kernel, dim3(pieces, rows), dim3(kArgmaxThreads), 0, stream, logits,
                                 row_stride, vocab, piece_size, temperature, seed, position, legal,
                                 static_cast<BestScore*>(scratch));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_chained(race_pick_kernel, dim3(rows), dim3(32), 0, stream,
                                         static_cast<const BestScore*>(scratch), pieces, ids, status));
}
