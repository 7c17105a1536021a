// The legal set of top-k then top-p sampling, one row per block.
//
// Definition (crates/app/cli/src/qwen_forward.rs:474-549): order the tokens by
// descending logit, lower id first on ties; keep the first top_k; of those,
// keep the shortest prefix whose weight exp((logit - max) / T) reaches top_p
// of the kept weight. The reference sorts on the host; here the k-th value and
// the prefix boundary are found by bisection over the ordered bit pattern of
// the logits (32 passes) and, among equal logits, over the id.
#include "common.cuh"

namespace mxb {

constexpr int kNucleusThreads = 1024;

// Order-preserving map from a finite float to an unsigned key.
__device__ __forceinline__ uint32_t ordered_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

__device__ __forceinline__ long long block_sum_ll(long long v, long long* scratch) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    long long t = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : 0;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
    if (threadIdx.x == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ double block_sum_f64(double v, double* scratch) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    double t = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : 0.0;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) t += __shfl_xor_sync(0xffffffffu, t, offset);
    if (threadIdx.x == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

struct Cut {       // tokens in front of the cut: key > key_cut, or key == key_cut and id <= id_cut
  uint32_t key;
  int id;
  __device__ __forceinline__ bool holds(uint32_t k, int i) const {
    return k > key || (k == key && i <= id);
  }
};

__global__ void __launch_bounds__(kNucleusThreads)
nucleus_mask_kernel(const float* __restrict__ logits, long long row_stride, int vocab,
                    const double* __restrict__ temperature, const double* __restrict__ top_p,
                    const int* __restrict__ top_k, unsigned char* __restrict__ legal, int* status) {
  __shared__ long long s_ll[33];
  __shared__ double s_f64[33];
  __shared__ float s_max[33];
  __shared__ int s_bad;
  const int r = blockIdx.x, tid = threadIdx.x;
  const float* row = logits + r * row_stride;
  unsigned char* out = legal + static_cast<size_t>(r) * vocab;
  int k = top_k[r];
  if (k <= 0 || k >= vocab) k = 0;  // qwen_forward.rs:489: only 0 < top_k < vocab truncates
  const double p = top_p[r];
  if (k == 0 && p >= 1.0) {
    for (int i = tid; i < vocab; i += blockDim.x) out[i] = 1;
    return;
  }
  if (tid == 0) s_bad = 0;
  __syncthreads();
  float local_max = -INFINITY;
  bool bad = false;
  for (int i = tid; i < vocab; i += blockDim.x) {
    const float v = row[i];
    bad = bad || !isfinite(v);
    local_max = fmaxf(local_max, v);
  }
  if (bad) s_bad = 1;
  local_max = warp_max(local_max);
  if ((tid & 31) == 0) s_max[tid >> 5] = local_max;
  __syncthreads();
  if (tid < 32) {
    float v = tid < (blockDim.x >> 5) ? s_max[tid] : -INFINITY;
    v = warp_max(v);
    if (tid == 0) s_max[32] = v;
  }
  __syncthreads();
  if (s_bad) {
    if (tid == 0) atomicOr(status, kStatusNonFinite);
    for (int i = tid; i < vocab; i += blockDim.x) out[i] = 1;
    return;
  }
  const double maximum = static_cast<double>(s_max[32]);
  const double inv_t = 1.0 / temperature[r];

  Cut by_count{0u, 0x7fffffff};  // everything in front by default
  if (k > 0) {
    // The k-th largest key: the largest t with count(key >= t) >= k.
    uint32_t t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t candidate = t | (1u << bit);
      long long count = 0;
      for (int i = tid; i < vocab; i += blockDim.x) count += ordered_key(row[i]) >= candidate;
      if (block_sum_ll(count, s_ll) >= k) t = candidate;
    }
    long long greater = 0;
    for (int i = tid; i < vocab; i += blockDim.x) greater += ordered_key(row[i]) > t;
    greater = block_sum_ll(greater, s_ll);
    const long long need = k - greater;  // equal keys to take, lowest ids first (>= 1)
    int bound = 0;  // the smallest id bound with count(key == t, id <= bound) >= need
    for (int bit = 30; bit >= 0; --bit) {
      // Bisection for the largest id bound that still holds FEWER than need, plus one.
      const int candidate = bound | (1 << bit);
      long long count = 0;
      for (int i = tid; i < vocab; i += blockDim.x) count += ordered_key(row[i]) == t && i < candidate;
      if (block_sum_ll(count, s_ll) < need) bound = candidate;
    }
    by_count = Cut{t, bound};  // ids < bound hold need - 1 equals at most; id == bound completes them
  }

  Cut by_mass{0u, 0x7fffffff};
  if (p < 1.0) {
    double kept = 0.0;
    for (int i = tid; i < vocab; i += blockDim.x) {
      const float v = row[i];
      if (by_count.holds(ordered_key(v), i)) kept += exp((static_cast<double>(v) - maximum) * inv_t);
    }
    kept = block_sum_f64(kept, s_f64);
    const double target = p * kept;
    // The key of the last token of the prefix: the largest t with
    // mass(key >= t) >= target.
    uint32_t t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t candidate = t | (1u << bit);
      double mass = 0.0;
      for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = row[i];
        const uint32_t key = ordered_key(v);
        if (key >= candidate && by_count.holds(key, i)) mass += exp((static_cast<double>(v) - maximum) * inv_t);
      }
      if (block_sum_f64(mass, s_f64) >= target) t = candidate;
    }
    double above = 0.0;
    long long equals = 0;
    for (int i = tid; i < vocab; i += blockDim.x) {
      const float v = row[i];
      const uint32_t key = ordered_key(v);
      if (!by_count.holds(key, i)) continue;
      if (key > t) above += exp((static_cast<double>(v) - maximum) * inv_t);
      equals += key == t;
    }
    above = block_sum_f64(above, s_f64);
    equals = block_sum_ll(equals, s_ll);
    // Equal logits share one weight; take them in id order until the target is reached.
    const uint32_t tbits = (t & 0x80000000u) ? (t & 0x7fffffffu) : ~t;
    const double weight = exp((static_cast<double>(__uint_as_float(tbits)) - maximum) * inv_t);
    long long need = 1;
    double covered = above + weight;
    while (covered < target && need < equals) { covered += weight; ++need; }
    int bound = 0;
    for (int bit = 30; bit >= 0; --bit) {
      const int candidate = bound | (1 << bit);
      long long count = 0;
      for (int i = tid; i < vocab; i += blockDim.x) {
        const uint32_t key = ordered_key(row[i]);
        count += key == t && i < candidate && by_count.holds(key, i);
      }
      if (block_sum_ll(count, s_ll) < need) bound = candidate;
    }
    by_mass = Cut{t, bound};
  }

  for (int i = tid; i < vocab; i += blockDim.x) {
    const uint32_t key = ordered_key(row[i]);
    out[i] = by_count.holds(key, i) && by_mass.holds(key, i);
  }
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_nucleus_mask(const float* logits, long long row_stride, int rows, int vocab,
                             const double* temperature, const double* top_p, const int* top_k,
                             unsigned char* legal, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  nucleus_mask_kernel<<<rows, kNucleusThreads, 0, stream>>>(logits, row_stride, vocab, temperature,
                                                           top_p, top_k, legal, status);
  return static_cast<int>(cudaGetLastError());
}
