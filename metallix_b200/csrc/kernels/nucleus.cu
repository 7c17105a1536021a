// The legal set of top-k then top-p sampling: a cluster of eight blocks per row.
//
// Definition (crates/app/cli/src/qwen_forward.rs:474-549): order the tokens by
// descending logit, lower id first on ties; keep the first top_k; of those,
// keep the shortest prefix whose weight exp((logit - max) / T) reaches top_p
// of the kept weight. The reference sorts on the host. Here nothing is sorted:
// a token's place in that order is one integer (the ordered bit pattern of its
// logit above the complement of its id, larger first), and both cuts are the
// same question about it, "the largest c such that the tokens with place >= c
// weigh at least the target": weight 1 and target top_k for the first cut, the
// token's weight and top_p of the kept weight for the second.
//
// A row is split over the eight blocks of a cluster, each with its part of
// the row in shared memory where it fits. The question is answered in two
// steps. First the row's range of values is cut into 1,024 equal bins (the
// bin of a value never falls as the value grows, so whole bins lie in front
// of one another): every block fills a histogram of its part, and after a
// cluster barrier every block adds up the eight histograms over distributed
// shared memory and walks them from the top to the bin where the weight
// reaches the target. Then the few tokens of that bin are gathered, again over
// distributed shared memory, into every block, which settles the rest alone,
// eleven bits of the place at a time. A bin that holds more tokens than the
// gathering has room for (a row of equal logits) takes the slow road: eleven
// bits at a time over the whole row, a cluster barrier per step.
//
// Weights are fixed-point integers (exp(..) scaled by a power of two so that a
// whole row still fits 62 bits): integer sums do not depend on the order of
// additions, so the mask is the same whatever else runs and however the
// atomics fall.
#include "common.cuh"

namespace mxb {

constexpr int kNucleusBlocks = 8;     // blocks of a cluster: parts of a row
constexpr int kNucleusThreads = 512;
constexpr int kNucleusWarps = kNucleusThreads / 32;
constexpr int kDigitBits = 11;
constexpr int kBins = 1 << kDigitBits;
constexpr int kBinsPerThread = kBins / kNucleusThreads;   // 4
constexpr int kValueBins = 1024;      // of the first step, two per thread
constexpr int kOwnEntries = 256;      // tokens of the chosen bin a block can hand over
constexpr int kAllEntries = kNucleusBlocks * kOwnEntries;
constexpr int kNucleusSharedLimit = 200 * 1024;
using u64 = unsigned long long;

// Order-preserving map from a finite float to an unsigned key.
__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ void nucleus_meet() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n"
               "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

// The 8 bytes at this block's shared address `address`, read from block `rank` of the cluster.
__device__ __forceinline__ u64 nucleus_remote(uint32_t address, uint32_t rank) {
  uint32_t remote;
  u64 value;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(address), "r"(rank));
  asm volatile("ld.shared::cluster.u64 %0, [%1];\n" : "=l"(value) : "r"(remote) : "memory");
  return value;
}

// Two neighbours of 8 bytes in one access (the address is a multiple of 16).
__device__ __forceinline__ void nucleus_remote_pair(uint32_t address, uint32_t rank, u64& first, u64& second) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(address), "r"(rank));
  asm volatile("ld.shared::cluster.v2.u64 {%0, %1}, [%2];\n" : "=l"(first), "=l"(second) : "r"(remote) : "memory");
}

struct NucleusSmall {
  // the first 16 bytes are read by the other blocks, in one access or as two halves
  float maximum;   // of this block's part
  int bad;         // a non-finite logit in this block's part
  float minimum;
  int own_count;   // tokens of the chosen bin in this block's part (more than kOwnEntries: too many)
  u64 warp_sums[kNucleusWarps];
  u64 remaining;
  int digit;
  float warp_maxima[kNucleusWarps];
  float warp_minima[kNucleusWarps];
};
static_assert(sizeof(NucleusSmall) % 16 == 0 || sizeof(NucleusSmall) % 8 == 0, "what follows holds floats");

struct Entry {   // a token of the chosen bin
  u64 place;
  u64 weight;
};

// What the blocks agree on bit by bit: a token's place in the order, its
// 32 + id_bits bits shifted up to a multiple of eleven.
struct Order {
  int id_bits, pad_bits;
  __device__ __forceinline__ u64 place(float v, int id) const {
    return ((static_cast<u64>(ordered_key(v)) << id_bits) | static_cast<u64>(((1u << id_bits) - 1u) - static_cast<uint32_t>(id)))
           << pad_bits;
  }
};

// Sum of `mine` over the threads after this one (an exclusive scan from the
// last thread down) and, in `total`, over all threads.
__device__ __forceinline__ u64 sum_of_later_threads(u64 mine, NucleusSmall* small, u64& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  u64 inclusive = mine;
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const u64 other = __shfl_down_sync(0xffffffffu, inclusive, offset);
    if (lane + offset < 32) inclusive += other;
  }
  __syncthreads();   // the sums of an earlier call have been read
  if (lane == 0) small->warp_sums[warp] = inclusive;
  __syncthreads();
  u64 later_warps = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kNucleusWarps; ++w) {
    const u64 s = small->warp_sums[w];
    all += s;
    if (w > warp) later_warps += s;
  }
  total = all;
  return inclusive - mine + later_warps;
}

// What a question is asked about: this block's part of the row (indexed by
// token id, begin <= id < end), which tokens count (place >= eligible) and
// what a token weighs: 1, or exp((logit - maximum) * inv_t) * scale.
struct Asked {
  const float* values;
  int begin, end;
  Order order;
  int levels;
  u64 eligible;
  bool weighted;
  double maximum, inv_t, scale;
  __device__ __forceinline__ u64 weight(float v) const {
    return weighted ? static_cast<u64>(exp((static_cast<double>(v) - maximum) * inv_t) * scale) : 1ull;
  }
};

// This thread's bins (thread 0 the lowest) hold `bins`; the bin where the
// weight, summed from the top bin down, reaches `target` lands in
// small->digit and what of the target is left inside it in small->remaining;
// `total` gets the weight of all bins. Every thread of the block calls it.
template <int PER_THREAD>
__device__ __forceinline__ void walk_bins(const u64 (&bins)[PER_THREAD], u64 target, bool find, NucleusSmall* small,
                                          u64& total) {
  u64 mine = 0;
#pragma unroll
  for (int b = 0; b < PER_THREAD; ++b) mine += bins[b];
  u64 above = sum_of_later_threads(mine, small, total);
  if (threadIdx.x == 0) { small->digit = 0; small->remaining = target; }   // kept if no bin is found: an empty row
  __syncthreads();
  if (find) {
#pragma unroll
    for (int b = PER_THREAD - 1; b >= 0; --b) {
      if (above < target && above + bins[b] >= target) {   // true for one bin of one thread
        small->digit = threadIdx.x * PER_THREAD + b;
        small->remaining = target - above;
      }
      above += bins[b];
    }
  }
  __syncthreads();
}

// Bins PER_THREAD * t ... of the histograms of all eight blocks, added up.
template <int PER_THREAD>
__device__ __forceinline__ void gather_bins(const u64* histogram, u64 (&bins)[PER_THREAD]) {
  // All loads first, then the sums: a sum that waited for its load would hold up the loads behind it.
  u64 fetched[kNucleusBlocks][PER_THREAD];
  const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(histogram + threadIdx.x * PER_THREAD));
#pragma unroll
  for (uint32_t rank = 0; rank < kNucleusBlocks; ++rank)
#pragma unroll
    for (int b = 0; b < PER_THREAD; b += 2) nucleus_remote_pair(address + b * 8, rank, fetched[rank][b], fetched[rank][b + 1]);
#pragma unroll
  for (int b = 0; b < PER_THREAD; ++b) {
    bins[b] = 0;
#pragma unroll
    for (int rank = 0; rank < kNucleusBlocks; ++rank) bins[b] += fetched[rank][b];
  }
}

// The slow road: eleven bits of the place at a time over the whole row, the
// histograms of the eight blocks added up behind a cluster barrier at every
// step. `round` counts those barriers, which picks the histogram buffer.
__device__ u64 nucleus_cut_over_the_row(const Asked& asked, u64 target, u64* histograms, NucleusSmall* small,
                                        int& round) {
  u64 prefix = 0;
  for (int level = 0; level < asked.levels; ++level) {
    const int shift = kDigitBits * (asked.levels - 1 - level);
    u64* histogram = histograms + (round & 1) * kBins;
    for (int b = threadIdx.x; b < kBins; b += kNucleusThreads) histogram[b] = 0;
    __syncthreads();
    for (int id = asked.begin + threadIdx.x; id < asked.end; id += kNucleusThreads) {
      const float v = asked.values[id];
      const u64 place = asked.order.place(v, id);
      if (place < asked.eligible) continue;
      if (level > 0 && (place >> (shift + kDigitBits)) != prefix) continue;
      const u64 weight = asked.weight(v);
      if (weight) atomicAdd(&histogram[(place >> shift) & (kBins - 1)], weight);
    }
    nucleus_meet();
    ++round;
    u64 bins[kBinsPerThread], total;
    gather_bins<kBinsPerThread>(histogram, bins);
    walk_bins<kBinsPerThread>(bins, target, true, small, total);
    prefix = (prefix << kDigitBits) | static_cast<u64>(small->digit);
    target = small->remaining;
  }
  return prefix;
}

// The same over the gathered tokens of one bin, which every block holds: no barrier between blocks.
__device__ u64 nucleus_cut_among(const Entry* entries, int count, int levels, u64 target, u64* histogram,
                                 NucleusSmall* small) {
  u64 prefix = 0;
  for (int level = 0; level < levels; ++level) {
    const int shift = kDigitBits * (levels - 1 - level);
    __syncthreads();   // the histogram of the level before has been read
    for (int b = threadIdx.x; b < kBins; b += kNucleusThreads) histogram[b] = 0;
    __syncthreads();
    for (int e = threadIdx.x; e < count; e += kNucleusThreads) {
      const Entry entry = entries[e];
      if (level > 0 && (entry.place >> (shift + kDigitBits)) != prefix) continue;
      if (entry.weight) atomicAdd(&histogram[(entry.place >> shift) & (kBins - 1)], entry.weight);
    }
    __syncthreads();
    u64 bins[kBinsPerThread], total;
#pragma unroll
    for (int b = 0; b < kBinsPerThread; ++b) bins[b] = histogram[threadIdx.x * kBinsPerThread + b];
    walk_bins<kBinsPerThread>(bins, target, true, small, total);
    prefix = (prefix << kDigitBits) | static_cast<u64>(small->digit);
    target = small->remaining;
  }
  return prefix;
}

// The bin of a value among kValueBins equal parts of [lowest, lowest + kValueBins / per_bin]:
// never falls as the value grows.
__device__ __forceinline__ int value_bin(float v, float lowest, float per_bin) {
  const int bin = __float2int_rz((v - lowest) * per_bin);
  return bin < 0 ? 0 : (bin > kValueBins - 1 ? kValueBins - 1 : bin);
}

// The place of the cut. For a weighted question the target is `fraction` of
// the weight of the tokens that count; otherwise it is `target`.
__device__ u64 nucleus_cut(const Asked& asked, float lowest, float per_bin, u64 target, double fraction,
                           u64* histograms, Entry* own, Entry* all, NucleusSmall* small, int& round) {
  // ---- which bin of values holds the cut
  u64* histogram = histograms + (round & 1) * kBins;
  for (int b = threadIdx.x; b < kValueBins; b += kNucleusThreads) histogram[b] = 0;
  __syncthreads();
  for (int id = asked.begin + threadIdx.x; id < asked.end; id += kNucleusThreads) {
    const float v = asked.values[id];
    if (asked.eligible && asked.order.place(v, id) < asked.eligible) continue;
    const u64 weight = asked.weight(v);
    if (weight) atomicAdd(&histogram[value_bin(v, lowest, per_bin)], weight);
  }
  nucleus_meet();
  ++round;
  constexpr int PER_THREAD = kValueBins / kNucleusThreads;
  u64 bins[PER_THREAD], total;
  gather_bins<PER_THREAD>(histogram, bins);
  if (asked.weighted) {
    // top_p of the kept weight needs the kept weight first: one walk that finds nothing
    walk_bins<PER_THREAD>(bins, 0, false, small, total);
    const double wanted = fraction * static_cast<double>(total);
    target = wanted >= static_cast<double>(total) ? total : static_cast<u64>(wanted);
    if (target < 1) target = 1;   // at least one unit and at most all of it
  }
  walk_bins<PER_THREAD>(bins, target, true, small, total);
  const int chosen = small->digit;
  const u64 inside = small->remaining;   // what the tokens of the chosen bin, from its top, have to weigh
  // ---- the tokens of that bin, from every block into every block
  if (threadIdx.x == 0) small->own_count = 0;
  __syncthreads();
  for (int id = asked.begin + threadIdx.x; id < asked.end; id += kNucleusThreads) {
    const float v = asked.values[id];
    if (value_bin(v, lowest, per_bin) != chosen) continue;
    const u64 place = asked.order.place(v, id);
    if (place < asked.eligible) continue;
    const int slot = atomicAdd(&small->own_count, 1);
    if (slot < kOwnEntries) {
      own[slot].place = place;
      own[slot].weight = asked.weight(v);
    }
  }
  nucleus_meet();
  ++round;   // no histogram was read, but both buffers are free again all the same
  int counts[kNucleusBlocks];
  bool fits = true;
  {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(&small->minimum));
#pragma unroll
    for (uint32_t rank = 0; rank < kNucleusBlocks; ++rank) {
      counts[rank] = static_cast<int>(nucleus_remote(address, rank) >> 32);   // own_count lies behind minimum
      fits = fits && counts[rank] <= kOwnEntries;
    }
  }
  if (!fits) return nucleus_cut_over_the_row(asked, target, histograms, small, round);   // the same for every block
  int offset = 0;
#pragma unroll
  for (uint32_t rank = 0; rank < kNucleusBlocks; ++rank) {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(own));
    for (int e = threadIdx.x; e < counts[rank]; e += kNucleusThreads)
      nucleus_remote_pair(address + e * 16, rank, all[offset + e].place, all[offset + e].weight);
    offset += counts[rank];
  }
  return nucleus_cut_among(all, offset, asked.levels, inside, histograms + (round & 1) * kBins, small);
}

__global__ void __launch_bounds__(kNucleusThreads)
nucleus_mask_kernel(const float* __restrict__ logits, long long row_stride, int vocab, int part, int in_shared,
                    int id_bits, const double* __restrict__ temperature, const double* __restrict__ top_p,
                    const int* __restrict__ top_k, unsigned char* __restrict__ legal, int* status) {
  extern __shared__ __align__(16) unsigned char nucleus_raw[];
  u64* histograms = reinterpret_cast<u64*>(nucleus_raw);                       // [2][kBins]
  Entry* own = reinterpret_cast<Entry*>(histograms + 2 * kBins);               // [kOwnEntries], read by the other blocks
  Entry* all = own + kOwnEntries;                                              // [kAllEntries]
  NucleusSmall* small = reinterpret_cast<NucleusSmall*>(all + kAllEntries);
  float* held = reinterpret_cast<float*>(small + 1);                           // [part] where it fits
  chain_release();
  const int rank = blockIdx.x, r = blockIdx.y, tid = threadIdx.x;
  const int begin = min(vocab, rank * part), end = min(vocab, begin + part);
  unsigned char* out = legal + static_cast<size_t>(r) * vocab;
  int k = top_k[r];
  if (k <= 0 || k >= vocab) k = 0;  // qwen_forward.rs:489: only 0 < top_k < vocab truncates
  const double p = top_p[r];
  const double inv_t = 1.0 / temperature[r];
  chain_wait();
  const float* row = behind_wait(logits) + r * row_stride;
  if (k == 0 && p >= 1.0) {   // the same for all blocks of the cluster: nobody waits for anybody
    for (int id = begin + tid; id < end; id += kNucleusThreads) out[id] = 1;
    return;
  }
  // ---- this block's part of the row, its extremes and whether it is finite
  const float* values = row;
  float local_max = -INFINITY, local_min = INFINITY;
  bool bad = false;
  for (int id = begin + tid; id < end; id += kNucleusThreads) {
    const float v = row[id];
    if (in_shared) held[id - begin] = v;
    bad = bad || !isfinite(v);
    local_max = fmaxf(local_max, v);
    local_min = fminf(local_min, v);
  }
  if (in_shared) values = held - begin;
  local_max = warp_max(local_max);
  local_min = -warp_max(-local_min);
  if (tid == 0) small->bad = 0;
  __syncthreads();
  if (bad) small->bad = 1;
  if ((tid & 31) == 0) { small->warp_maxima[tid >> 5] = local_max; small->warp_minima[tid >> 5] = local_min; }
  __syncthreads();
  if (tid == 0) {
    float block_max = -INFINITY, block_min = INFINITY;
    for (int w = 0; w < kNucleusWarps; ++w) {
      block_max = fmaxf(block_max, small->warp_maxima[w]);
      block_min = fminf(block_min, small->warp_minima[w]);
    }
    small->maximum = block_max;
    small->minimum = block_min;
  }
  nucleus_meet();
  int round = 0;   // cluster barriers so far: picks the histogram buffer
  float row_max = -INFINITY, row_min = INFINITY;
  int any_bad = 0;
  {
    const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(&small->maximum));
    for (uint32_t other = 0; other < kNucleusBlocks; ++other) {
      u64 first, second;   // (maximum, bad), (minimum, own_count)
      nucleus_remote_pair(address, other, first, second);
      row_max = fmaxf(row_max, __uint_as_float(static_cast<uint32_t>(first)));
      any_bad |= static_cast<int>(first >> 32);
      row_min = fminf(row_min, __uint_as_float(static_cast<uint32_t>(second)));
    }
  }
  if (any_bad) {
    if (tid == 0 && rank == 0) atomicOr(status, kStatusNonFinite);
    for (int id = begin + tid; id < end; id += kNucleusThreads) out[id] = 1;
  } else {
    const int pad_bits = (kDigitBits - (32 + id_bits) % kDigitBits) % kDigitBits;
    Asked asked;
    asked.values = values;
    asked.begin = begin;
    asked.end = end;
    asked.order = Order{id_bits, pad_bits};
    asked.levels = (32 + id_bits + pad_bits) / kDigitBits;
    asked.eligible = 0;   // everything counts
    asked.weighted = false;
    asked.maximum = static_cast<double>(row_max);
    asked.inv_t = inv_t;
    asked.scale = static_cast<double>(1ull << (62 - id_bits));
    const float range = row_max - row_min;
    const float per_bin = range > 1e-30f ? static_cast<float>(kValueBins) / range : 0.0f;
    u64 by_count = 0;
    if (k > 0)
      by_count = nucleus_cut(asked, row_min, per_bin, static_cast<u64>(k), 0.0, histograms, own, all, small, round);
    u64 by_mass = 0;
    if (p < 1.0) {
      asked.eligible = by_count;
      asked.weighted = true;
      by_mass = nucleus_cut(asked, row_min, per_bin, 0, p, histograms, own, all, small, round);
    }
    const u64 cut = by_count > by_mass ? by_count : by_mass;
    for (int id = begin + tid; id < end; id += kNucleusThreads) out[id] = asked.order.place(values[id], id) >= cut;
  }
  nucleus_meet();   // nobody leaves while its shared memory is still being read
}

}  // namespace mxb

using namespace mxb;

// Vocabularies up to 2^22 ids (a token's place must fit 55 bits).
MXB_API int mxb_nucleus_mask(const float* logits, long long row_stride, int rows, int vocab,
                             const double* temperature, const double* top_p, const int* top_k,
                             unsigned char* legal, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || vocab > (1 << 22) || rows > 65535) return static_cast<int>(cudaErrorInvalidValue);
  int id_bits = 1;
  while ((1 << id_bits) < vocab) ++id_bits;
  const int part = ((vocab + kNucleusBlocks - 1) / kNucleusBlocks + 3) / 4 * 4;
  const size_t fixed = 2 * kBins * sizeof(u64) + (kOwnEntries + kAllEntries) * sizeof(Entry) + sizeof(NucleusSmall);
  const int in_shared = fixed + static_cast<size_t>(part) * 4 <= static_cast<size_t>(kNucleusSharedLimit) ? 1 : 0;
  const size_t shared = fixed + (in_shared ? static_cast<size_t>(part) * 4 : 0);
  cudaError_t e = cudaFuncSetAttribute(nucleus_mask_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(shared));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_chained_clusters(nucleus_mask_kernel, dim3(kNucleusBlocks, rows),
                                                  dim3(kNucleusThreads), shared, kNucleusBlocks, stream, logits,
                                                  row_stride, vocab, part, in_shared, id_bits, temperature, top_p,
                                                  top_k, legal, status));
}
