// Attention of single decoded tokens over the paged cache, split along the
// keys so that a handful of requests still fills the GPU.
//
// One block takes one request's token, one key/value head and one split of
// kSplitKeys absolute key positions, and serves every query head of that
// key/value head from a single read of K and V. It writes an unnormalised
// partial result (running maximum, sum, accumulator) per (token, head,
// split); a second kernel merges the splits of a head in ascending order.
// Split boundaries sit at multiples of kSplitKeys of the absolute position
// and the merge order is fixed, so a token's result does not depend on what
// else is in the batch. Scores, softmax and accumulators are float32.
//
// Replaces the reference's per-step gather of every row's whole context into
// [rows, kv_heads, longest, head_dim] plus a masked SDPA call
// (crates/models/qwen/src/forward/paged.rs:189-219, :1067-1076, :1216-1232).
#include "tcgen05.cuh"   // TMA tile loads and tensor maps (async_copy.cuh, common.cuh come with it)

namespace mxb {

constexpr int kSplitKeys = 128;
constexpr int kDecodeThreads = 128;
constexpr unsigned kDecodeBlocksAtOnce = 444;   // blocks of the bfloat16 kernels a B200 holds at once: three an SM
constexpr float kDecodeMinusHuge = -1.0e30f;

template <typename T> struct Vec16;  // 16 bytes of T
template <> struct Vec16<float> {
  static constexpr int kElems = 4;
  float4 raw;
  __device__ __forceinline__ void unpack(float* out) const { out[0] = raw.x; out[1] = raw.y; out[2] = raw.z; out[3] = raw.w; }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  uint4 raw;
  __device__ __forceinline__ void unpack(float* out) const {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

__device__ __forceinline__ void decode_copy_async_16(void* dst, const void* src, int src_bytes) {
  const uint32_t address = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(address), "l"(src), "r"(src_bytes));
}

// Partial layout per (token row, head, split): [head_dim] accumulator, then
// the running maximum and the running sum.
//
// The split's keys and values are first brought into shared memory whole,
// with every 16-byte copy of the block in flight at once (keys as one group of
// asynchronous copies, values as a second): a decoded token has no arithmetic
// to hide memory latency behind, so the copies must overlap each other.
template <typename T, int HD, int G>
__global__ void __launch_bounds__(kDecodeThreads)
paged_attention_decode_kernel(const T* __restrict__ q, const T* __restrict__ cache,
                              float* __restrict__ partial, const int* __restrict__ block_tables,
                              int max_pages, const int* __restrict__ row_token,
                              const int* __restrict__ row_request, const int* __restrict__ positions,
                              int heads, int kv_heads, int page_tokens, int num_pages, int max_splits,
                              int window, float scale, int* status) {
  constexpr int E = Vec16<T>::kElems;  // elements per 16-byte piece
  constexpr int LPK = HD / E;          // 16-byte pieces (and lanes) per key row
  constexpr int KPW = 32 / LPK;        // key rows a warp reads at once
  constexpr int ROWS = kDecodeThreads / LPK;
  static_assert(HD % E == 0 && 32 % LPK == 0, "head_dim must split into 16-byte pieces over a warp");
  extern __shared__ __align__(16) unsigned char decode_shared[];
  T* sK = reinterpret_cast<T*>(decode_shared);                  // [kSplitKeys][HD]
  T* sV = sK + kSplitKeys * HD;                                 // [kSplitKeys][HD]
  constexpr size_t kStageBytes = 2 * static_cast<size_t>(kSplitKeys) * HD * sizeof(T);
  constexpr size_t kReduceBytes = static_cast<size_t>(ROWS) * G * (HD + 4) * sizeof(float);
  constexpr size_t kFront = kStageBytes > kReduceBytes ? kStageBytes : kReduceBytes;
  float* s_score = reinterpret_cast<float*>(decode_shared + kFront);  // [G][kSplitKeys]
  float* s_stat = s_score + G * kSplitKeys;                     // [G][2]
  float* s_acc = reinterpret_cast<float*>(decode_shared);       // [ROWS][G][HD + 4], over K and V once they are used up

  const int split = blockIdx.x, kv = blockIdx.y, row = blockIdx.z;
  const int token = row_token[row];
  if (token < 0) return;  // a padding row
  const int pos = positions[token];
  const int group = heads / kv_heads;  // query heads per key/value head, <= G
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int begin = max(split * kSplitKeys, first_key);
  const int end = min((split + 1) * kSplitKeys, pos + 1);
  if (begin >= end) return;  // the merge skips splits outside [first_key, pos]
  const int count = end - begin;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* table = block_tables + static_cast<size_t>(row_request[row]) * max_pages;
  const size_t page_stride = static_cast<size_t>(2) * kv_heads * page_tokens * HD;
  const size_t v_offset = static_cast<size_t>(kv_heads) * page_tokens * HD;
  const T* head_base = cache + static_cast<size_t>(kv) * page_tokens * HD;

  // ---- every copy of the split in flight: keys, then values
  const int piece = tid % LPK;
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    T* dst_base = pass == 0 ? sK : sV;
    for (int kk = tid / LPK; kk < count; kk += ROWS) {
      const int key = begin + kk;
      int page = table[key / page_tokens];
      bool ok = page >= 0 && page < num_pages;
      if (!ok) {
        if (piece == 0 && pass == 0) atomicOr(status, kStatusBadPage);
        page = 0;
      }
      const T* src = head_base + page * page_stride + (pass == 0 ? 0 : v_offset) +
                     static_cast<size_t>(key % page_tokens) * HD + piece * E;
      decode_copy_async_16(dst_base + kk * HD + piece * E, src, ok ? 16 : 0);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  }

  // ---- scores: a group of LPK lanes per key row
  const int sub = lane % LPK, which = lane / LPK;
  float qreg[G][E];
#pragma unroll
  for (int h = 0; h < G; ++h) {
    if (h < group) {
      Vec16<T> v;
      v.raw = *reinterpret_cast<const decltype(v.raw)*>(
          q + (static_cast<size_t>(token) * heads + kv * group + h) * HD + sub * E);
      v.unpack(qreg[h]);
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) qreg[h][e] = 0.0f;
    }
  }
  asm volatile("cp.async.wait_group 1;\n" ::);  // the keys have landed
  __syncthreads();
  for (int base = warp * KPW; base < count; base += (kDecodeThreads / 32) * KPW) {
    const int kk = base + which;
    float dots[G];
#pragma unroll
    for (int h = 0; h < G; ++h) dots[h] = 0.0f;
    if (kk < count) {
      Vec16<T> v;
      v.raw = *reinterpret_cast<const decltype(v.raw)*>(sK + kk * HD + sub * E);
      float kf[E];
      v.unpack(kf);
#pragma unroll
      for (int h = 0; h < G; ++h)
#pragma unroll
        for (int e = 0; e < E; ++e) dots[h] = fmaf(qreg[h][e], kf[e], dots[h]);
    }
#pragma unroll
    for (int h = 0; h < G; ++h) {
#pragma unroll
      for (int offset = LPK / 2; offset > 0; offset >>= 1)
        dots[h] += __shfl_xor_sync(0xffffffffu, dots[h], offset);
      if (sub == 0 && kk < count) s_score[h * kSplitKeys + kk] = dots[h] * scale;
    }
  }
  __syncthreads();

  // ---- softmax statistics of this split, one warp per head
  for (int h = warp; h < group; h += kDecodeThreads / 32) {
    float m = kDecodeMinusHuge;
    for (int kk = lane; kk < count; kk += 32) m = fmaxf(m, s_score[h * kSplitKeys + kk]);
    m = warp_max(m);
    float l = 0.0f;
    for (int kk = lane; kk < count; kk += 32) {
      const float p = expf(s_score[h * kSplitKeys + kk] - m);
      s_score[h * kSplitKeys + kk] = p;
      l += p;
    }
    l = warp_sum(l);
    if (lane == 0) { s_stat[h * 2] = m; s_stat[h * 2 + 1] = l; }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);  // the values have landed
  __syncthreads();

  // ---- P V: LPK threads per value row, ROWS rows at a time
  const int vsub = tid % LPK, vrow = tid / LPK;
  float acc[G][E];
#pragma unroll
  for (int h = 0; h < G; ++h)
#pragma unroll
    for (int e = 0; e < E; ++e) acc[h][e] = 0.0f;
  for (int kk = vrow; kk < count; kk += ROWS) {
    Vec16<T> v;
    v.raw = *reinterpret_cast<const decltype(v.raw)*>(sV + kk * HD + vsub * E);
    float vf[E];
    v.unpack(vf);
#pragma unroll
    for (int h = 0; h < G; ++h) {
      const float p = s_score[h * kSplitKeys + kk];
#pragma unroll
      for (int e = 0; e < E; ++e) acc[h][e] = fmaf(p, vf[e], acc[h][e]);
    }
  }
  __syncthreads();  // s_acc lies over the keys and values: everybody is done reading them
#pragma unroll
  for (int h = 0; h < G; ++h)
#pragma unroll
    for (int e = 0; e < E; ++e) s_acc[(vrow * G + h) * (HD + 4) + vsub * E + e] = acc[h][e];
  __syncthreads();
  // Sum the ROWS partial accumulators in a fixed order and write the partial.
  for (int i = tid; i < group * HD; i += kDecodeThreads) {
    const int h = i / HD, d = i - h * HD;
    float sum = 0.0f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) sum += s_acc[(r * G + h) * (HD + 4) + d];
    const int head = kv * group + h;
    float* dst = partial + ((static_cast<size_t>(row) * heads + head) * max_splits + split) * (HD + 2);
    dst[d] = sum;
    if (d == 0) { dst[HD] = s_stat[h * 2]; dst[HD + 1] = s_stat[h * 2 + 1]; }
  }
}

// ---------------------------------------------------------------------------
// The bfloat16 split on the tensor cores. The scalar kernel above spends more
// issue slots on unpacking, multiply-adds and shuffles than the memory system
// needs time to deliver the keys; here the query heads of one key/value head
// (at most 8) form the rows of a 16-row tensor-core tile, so q k^T and p v
// cost a few hundred instructions per split. Each of the four warps takes 32
// of the split's 128 keys with softmax statistics of its own; the warps'
// results are merged in warp order, then written as one partial.
__device__ __forceinline__ uint32_t decode_smem_address(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void decode_ldmatrix_x4(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void decode_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t address) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(address));
}
__device__ __forceinline__ void decode_mma(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  // Rows 8..15 of the 16-row operand are zero: a1 = a3 = 0.
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float decode_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// Key rows lie in shared memory as they lie in the cache, each followed by 16
// bytes of padding: eight consecutive rows then start in eight different bank
// groups, so ldmatrix meets no conflict, and a row is one bulk copy.
template <int HD> __device__ __forceinline__ uint32_t decode_tile_offset(int row, int chunk) {
  return static_cast<uint32_t>(row * (HD * 2 + 16) + (chunk << 4));
}

template <int HD>
__global__ void __launch_bounds__(kDecodeThreads)
paged_attention_decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ cache,
                                  float* __restrict__ partial, const int* __restrict__ block_tables,
                                  int max_pages, const int* __restrict__ row_token,
                                  const int* __restrict__ row_request, const int* __restrict__ positions,
                                  int heads, int kv_heads, int page_tokens, int num_pages, int max_splits,
                                  int window, float scale, int* status) {
  constexpr int ROW_BYTES = HD * 2;
  constexpr int TILE_BYTES = kSplitKeys * (ROW_BYTES + 16);
  extern __shared__ __align__(128) unsigned char mma_shared[];
  unsigned char* sK = mma_shared;                 // [128] rows of HD values + 16 bytes
  unsigned char* sV = sK + TILE_BYTES;            // the same for the values
  float* s_merge = reinterpret_cast<float*>(mma_shared);  // [4 warps][8 heads][HD + 2], over K once the scores exist
  __shared__ __align__(8) uint64_t barriers[2];   // keys, values

  chain_release();
  // What follows up to chain_wait() reads nothing a kernel of this step writes
  // (the step's integers and the keys and values of earlier positions), so it
  // runs, copies included, while the kernels before this one are still at work.
  const int split = blockIdx.x, kv = blockIdx.y, row = blockIdx.z;
  const int token = row_token[row];
  if (token < 0) return;
  const int pos = positions[token];
  const int group = heads / kv_heads;  // <= 8
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int begin = max(split * kSplitKeys, first_key);
  const int end = min((split + 1) * kSplitKeys, pos + 1);
  if (begin >= end) return;
  const int count = end - begin;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  // ---- one thread per key row: a block-table lookup, then one bulk copy for
  // the row's keys and one for its values (the copy engine moves the bytes;
  // the thread issues two instructions instead of one per 16 bytes).
  if (tid == 0) {
    barrier_init(&barriers[0], kDecodeThreads);
    barrier_init(&barriers[1], kDecodeThreads);
    barrier_init_fence();
  }
  __syncthreads();
  {
    const int* table = block_tables + static_cast<size_t>(row_request[row]) * max_pages;
    const size_t page_stride = static_cast<size_t>(2) * kv_heads * page_tokens * HD;
    const size_t v_offset = static_cast<size_t>(kv_heads) * page_tokens * HD;
    const int kk = tid;  // kSplitKeys == kDecodeThreads
    const int key = begin + kk;
    bool ok = kk < count;
    int page = 0;
    if (ok) {
      page = table[key / page_tokens];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, kStatusBadPage);
        ok = false;
      }
    }
    // The token's own key and value are written by the kernel before this
    // one: that row waits for it; every other row is fetched right away.
    const bool fresh = ok && key == pos;
    const __nv_bfloat16* src = cache + page * page_stride + static_cast<size_t>(kv) * page_tokens * HD +
                               static_cast<size_t>(ok ? key % page_tokens : 0) * HD;
    if (ok && !fresh) {
      barrier_arrive_expect(&barriers[0], ROW_BYTES);
      bulk_copy(sK + decode_tile_offset<HD>(kk, 0), src, ROW_BYTES, &barriers[0]);
      barrier_arrive_expect(&barriers[1], ROW_BYTES);
      bulk_copy(sV + decode_tile_offset<HD>(kk, 0), src + v_offset, ROW_BYTES, &barriers[1]);
    }
    chain_wait();
    if (fresh) {
      barrier_arrive_expect(&barriers[0], ROW_BYTES);
      bulk_copy(sK + decode_tile_offset<HD>(kk, 0), src, ROW_BYTES, &barriers[0]);
      barrier_arrive_expect(&barriers[1], ROW_BYTES);
      bulk_copy(sV + decode_tile_offset<HD>(kk, 0), src + v_offset, ROW_BYTES, &barriers[1]);
    }
    if (!ok) {
      // A row beyond the split's keys: zeros, written by the thread itself.
      uint4* zk = reinterpret_cast<uint4*>(sK + decode_tile_offset<HD>(kk, 0));
      uint4* zv = reinterpret_cast<uint4*>(sV + decode_tile_offset<HD>(kk, 0));
#pragma unroll
      for (int c = 0; c < ROW_BYTES / 16; ++c) zk[c] = zv[c] = make_uint4(0u, 0u, 0u, 0u);
      barrier_arrive(&barriers[0]);
      barrier_arrive(&barriers[1]);
    }
  }

  // ---- the query heads of this key/value head as rows 0..group-1 of the 16-row operand
  uint32_t qa0[HD / 16], qa2[HD / 16];
  {
    // q is written by the kernel ahead of this one
    const __nv_bfloat16* qrow = behind_wait(q) + (static_cast<size_t>(token) * heads + kv * group + (g < group ? g : 0)) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      qa0[ks] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
      qa2[ks] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  const bool keys_landed = barrier_wait(&barriers[0], 0, status);
  __syncthreads();  // also orders the zero rows written by other threads

  // ---- scores of this warp's 32 keys
  const int key_base = warp * 32;
  float sc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
  if (key_base < count) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        uint32_t kf[4];
        const int krow = key_base + nb * 16 + (lane & 7) + (lane >> 4) * 8;
        decode_ldmatrix_x4(kf, decode_smem_address(sK + decode_tile_offset<HD>(krow, ks * 2 + ((lane >> 3) & 1))));
        decode_mma(sc[2 * nb], qa0[ks], qa2[ks], kf[0], kf[1]);
        decode_mma(sc[2 * nb + 1], qa0[ks], qa2[ks], kf[2], kf[3]);
      }
    }
  }
  // Row g of the tile is query head g; this thread holds keys nb * 8 + 2t, 2t + 1.
  const float scale_log2 = scale * 1.4426950408889634f;
  float m_w = -INFINITY;
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int kk = key_base + nb * 8 + 2 * t + j;
      sc[nb][j] = kk < count ? sc[nb][j] * scale_log2 : -INFINITY;
      m_w = fmaxf(m_w, sc[nb][j]);
    }
  }
  m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 1));
  m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 2));
  const float ref = m_w == -INFINITY ? 0.0f : m_w;
  float l_w = 0.0f;
  uint32_t pa0[2], pa2[2];
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    const float p0 = decode_exp2(sc[nb][0] - ref), p1 = decode_exp2(sc[nb][1] - ref);
    l_w += p0 + p1;
    __nv_bfloat162 packed = __floats2bfloat162_rn(p0, p1);
    const uint32_t word = *reinterpret_cast<uint32_t*>(&packed);
    if (nb & 1) pa2[nb >> 1] = word; else pa0[nb >> 1] = word;
  }
  l_w += __shfl_xor_sync(0xffffffffu, l_w, 1);
  l_w += __shfl_xor_sync(0xffffffffu, l_w, 2);

  const bool values_landed = barrier_wait(&barriers[1], 0, status);
  // One decision for the whole block; the status word says why, and both
  // barriers were given their time, so no copy is left in flight.
  if (__syncthreads_or(!keys_landed || !values_landed)) return;

  // ---- o = p v over this warp's 32 keys
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  if (key_base < count) {
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int nb = 0; nb < HD / 16; ++nb) {
        uint32_t vf[4];
        const int vrow = key_base + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        decode_ldmatrix_x4_trans(vf, decode_smem_address(sV + decode_tile_offset<HD>(vrow, nb * 2 + (lane >> 4))));
        decode_mma(o[2 * nb], pa0[ks], pa2[ks], vf[0], vf[1]);
        decode_mma(o[2 * nb + 1], pa0[ks], pa2[ks], vf[2], vf[3]);
      }
    }
  }
  __syncthreads();  // every warp is done with K and V: the merge area lies over K

  // ---- merge the four warps in warp order
  if (g < group) {
    float* mine = s_merge + (warp * 8 + g) * (HD + 2);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      mine[i * 8 + 2 * t] = o[i][0];
      mine[i * 8 + 2 * t + 1] = o[i][1];
    }
    if (t == 0) { mine[HD] = m_w; mine[HD + 1] = l_w; }
  }
  __syncthreads();
  for (int i = tid; i < group * HD; i += kDecodeThreads) {
    const int h = i / HD, d = i - h * HD;
    float m_all = -INFINITY;
#pragma unroll
    for (int wp = 0; wp < 4; ++wp) m_all = fmaxf(m_all, s_merge[(wp * 8 + h) * (HD + 2) + HD]);
    float sum = 0.0f, l_all = 0.0f;
#pragma unroll
    for (int wp = 0; wp < 4; ++wp) {
      const float* theirs = s_merge + (wp * 8 + h) * (HD + 2);
      const float weight = decode_exp2(theirs[HD] - m_all);  // a warp without keys has m = -inf: weight 0
      sum += weight * theirs[d];
      l_all += weight * theirs[HD + 1];
    }
    const int head = kv * group + h;
    float* dst = partial + ((static_cast<size_t>(row) * heads + head) * max_splits + split) * (HD + 2);
    dst[d] = sum;
    if (d == 0) { dst[HD] = m_all * 0.6931471805599453f; dst[HD + 1] = l_all; }  // the merge kernel works in natural units
  }
}

// The same split with the keys and values fetched a page at a time: one TMA
// box of one page x 64 values (128-byte swizzle) instead of one bulk copy per
// 256-byte row. The copy engine takes a request every few tens of cycles
// whatever its size, and 256 requests a block made it, not memory, set the
// pace (clock stamps in the blocks: 4,200 of a block's 9,300 cycles went into
// handing the requests over). A split is always its whole 128 absolute
// positions (a page that holds none of the token's keys is a box beyond the
// cache's last row: zeros); rows read by ldmatrix undo the swizzle.
//   byte offset of 16-byte chunk c of row r:  half c / 8, then r * 128 + ((c % 8) ^ (r % 8)) * 16
template <int HD> __device__ __forceinline__ uint32_t decode_swizzled_offset(int row, int chunk) {
  return static_cast<uint32_t>((chunk >> 3) * (kSplitKeys * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int HD>
__global__ void __launch_bounds__(kDecodeThreads)
paged_attention_decode_tma_kernel(const __grid_constant__ CUtensorMap map_cache, const __nv_bfloat16* __restrict__ q,
                                  float* __restrict__ partial, const int* __restrict__ block_tables,
                                  int max_pages, const int* __restrict__ row_token,
                                  const int* __restrict__ row_request, const int* __restrict__ positions,
                                  int heads, int kv_heads, int page_tokens, int num_pages, int max_splits,
                                  int window, float scale, int* status) {
  constexpr int HALVES = HD / kTmaColumns;                 // 64-value halves of a row
  constexpr int TILE_BYTES = kSplitKeys * HD * 2;
  extern __shared__ unsigned char tma_decode_raw[];
  __shared__ __align__(8) uint64_t barriers[2];   // keys, values
  unsigned char* sK = tma_decode_raw + ((1024 - (shared_address(tma_decode_raw) & 1023)) & 1023);
  unsigned char* sV = sK + TILE_BYTES;
  float* s_merge = reinterpret_cast<float*>(sK);  // [4 warps][8 heads][HD + 2], over K once the scores exist
  static_assert(4 * 8 * (HD + 2) * sizeof(float) <= TILE_BYTES, "the merge area must fit over the keys");

  // A grid that is resident at once lets its successor start right away; one
  // of several rounds only when a block is nearly done: a successor's blocks,
  // resident and waiting, would take the places of this kernel's later rounds.
  const bool release_late = gridDim.x * gridDim.y * gridDim.z > kDecodeBlocksAtOnce;
  if (!release_late) chain_release();
  // What follows up to chain_wait() reads nothing a kernel of this step writes
  // (the step's integers and the pages of earlier positions), so it runs,
  // copies included, while the kernels before this one are still at work.
  const int split = blockIdx.x, kv = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int key0 = split * kSplitKeys;
  // One thread per box: keys or values, page of the split, 64-value half.
  const int pages = kSplitKeys / page_tokens;   // <= 16
  const int boxes = 2 * pages * HALVES;         // <= 64
  const bool fetcher = tid < boxes;
  const int which = tid / (pages * HALVES), slot = (tid / HALVES) % pages, half = tid % HALVES;
  const int page_key = key0 + slot * page_tokens;
  // Two trips to memory before the copies can start, not three: the token and
  // its request's row of the block table first, then the position and,
  // without waiting to learn whether the page holds any of the token's keys,
  // the page.
  const int token = row_token[row];
  const int table_row = row_request[row];
  int page = 0;
  if (fetcher && page_key / page_tokens < max_pages)
    page = block_tables[static_cast<size_t>(table_row) * max_pages + page_key / page_tokens];
  if (token < 0) return;
  const int pos = positions[token];
  const int group = heads / kv_heads;  // <= 8
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  if (key0 > pos || key0 + kSplitKeys <= first_key) return;   // the merge skips splits outside [first_key, pos]
  const int lo = max(first_key - key0, 0), hi = min(pos - key0, kSplitKeys - 1);   // the split's rows that count

  if (tid == 0) {
    barrier_init(&barriers[0], 1);
    barrier_init(&barriers[1], 1);
    barrier_init_fence();
    barrier_arrive_expect(&barriers[0], TILE_BYTES);   // every box is fetched, whatever it holds
    barrier_arrive_expect(&barriers[1], TILE_BYTES);
  }
  __syncthreads();
  // The page that holds the token's own position is written by the kernel
  // ahead of this one: it waits; every other page is fetched right away. A
  // page that holds none of the token's keys is not wanted: its box starts
  // beyond the cache's last row, where the copy engine writes zeros.
  const bool fresh = fetcher && pos >= page_key && pos < page_key + page_tokens;
  bool wanted = fetcher && page_key <= pos && page_key + page_tokens > first_key;
  if (wanted && (page < 0 || page >= num_pages)) {
    atomicOr(status, kStatusBadPage);
    wanted = false;
  }
  unsigned char* dst = (which ? sV : sK) + half * (kSplitKeys * 128) + slot * page_tokens * 128;
  const int box_row = wanted ? ((page * 2 + which) * kv_heads + kv) * page_tokens
                             : num_pages * 2 * kv_heads * page_tokens;
  if (fetcher && !fresh) tma_load_2d(dst, &map_cache, half * kTmaColumns, box_row, &barriers[which]);
  chain_wait();
  if (fresh) tma_load_2d(dst, &map_cache, half * kTmaColumns, box_row, &barriers[which]);

  // ---- the query heads of this key/value head as rows 0..group-1 of the 16-row operand
  uint32_t qa0[HD / 16], qa2[HD / 16];
  {
    // q is written by the kernel ahead of this one
    const __nv_bfloat16* qrow = behind_wait(q) + (static_cast<size_t>(token) * heads + kv * group + (g < group ? g : 0)) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      qa0[ks] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
      qa2[ks] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  const bool keys_landed = barrier_wait(&barriers[0], 0, status);

  // ---- scores of this warp's 32 keys
  const int key_base = warp * 32;
  const bool has_keys = key_base <= hi && key_base + 31 >= lo;
  float sc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
  if (has_keys) {
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        uint32_t kf[4];
        const int krow = key_base + nb * 16 + (lane & 7) + (lane >> 4) * 8;
        decode_ldmatrix_x4(kf, decode_smem_address(sK + decode_swizzled_offset<HD>(krow, ks * 2 + ((lane >> 3) & 1))));
        decode_mma(sc[2 * nb], qa0[ks], qa2[ks], kf[0], kf[1]);
        decode_mma(sc[2 * nb + 1], qa0[ks], qa2[ks], kf[2], kf[3]);
      }
    }
  }
  // Row g of the tile is query head g; this thread holds keys nb * 8 + 2t, 2t + 1.
  const float scale_log2 = scale * 1.4426950408889634f;
  float m_w = -INFINITY;
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int kk = key_base + nb * 8 + 2 * t + j;
      sc[nb][j] = kk >= lo && kk <= hi ? sc[nb][j] * scale_log2 : -INFINITY;
      m_w = fmaxf(m_w, sc[nb][j]);
    }
  }
  m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 1));
  m_w = fmaxf(m_w, __shfl_xor_sync(0xffffffffu, m_w, 2));
  const float ref = m_w == -INFINITY ? 0.0f : m_w;
  float l_w = 0.0f;
  uint32_t pa0[2], pa2[2];
#pragma unroll
  for (int nb = 0; nb < 4; ++nb) {
    const float p0 = decode_exp2(sc[nb][0] - ref), p1 = decode_exp2(sc[nb][1] - ref);
    l_w += p0 + p1;
    __nv_bfloat162 packed = __floats2bfloat162_rn(p0, p1);
    const uint32_t word = *reinterpret_cast<uint32_t*>(&packed);
    if (nb & 1) pa2[nb >> 1] = word; else pa0[nb >> 1] = word;
  }
  l_w += __shfl_xor_sync(0xffffffffu, l_w, 1);
  l_w += __shfl_xor_sync(0xffffffffu, l_w, 2);

  const bool values_landed = barrier_wait(&barriers[1], 0, status);
  // One decision for the whole block; the status word says why, and both
  // barriers were given their time, so no copy is left in flight.
  if (__syncthreads_or(!keys_landed || !values_landed)) return;

  // A masked key has weight 0, but 0 x NaN is NaN: value rows outside the
  // token's keys (the rest of the last page, whatever an earlier owner of the
  // page left there) are zeroed, so that nothing is asked
  // of what the cache holds beyond a request's own positions. A warp reads
  // only its own 32 rows, and only a split's first and last warps have any.
  if (has_keys && (key_base < lo || key_base + 31 > hi)) {
    for (int i = lane; i < 32 * (HD / 8); i += 32) {
      const int vrow = key_base + i / (HD / 8);
      if (vrow < lo || vrow > hi)
        *reinterpret_cast<uint4*>(sV + decode_swizzled_offset<HD>(vrow, i % (HD / 8))) = make_uint4(0u, 0u, 0u, 0u);
    }
    __syncwarp();
  }

  // ---- o = p v over this warp's 32 keys
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
  if (has_keys) {
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int nb = 0; nb < HD / 16; ++nb) {
        uint32_t vf[4];
        const int vrow = key_base + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        decode_ldmatrix_x4_trans(vf, decode_smem_address(sV + decode_swizzled_offset<HD>(vrow, nb * 2 + (lane >> 4))));
        decode_mma(o[2 * nb], pa0[ks], pa2[ks], vf[0], vf[1]);
        decode_mma(o[2 * nb + 1], pa0[ks], pa2[ks], vf[2], vf[3]);
      }
    }
  }
  __syncthreads();  // every warp is done with K and V: the merge area lies over K

  if (release_late) chain_release();
  // ---- merge the four warps in warp order
  if (g < group) {
    float* mine = s_merge + (warp * 8 + g) * (HD + 2);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      mine[i * 8 + 2 * t] = o[i][0];
      mine[i * 8 + 2 * t + 1] = o[i][1];
    }
    if (t == 0) { mine[HD] = m_w; mine[HD + 1] = l_w; }
  }
  __syncthreads();
  for (int i = tid; i < group * HD; i += kDecodeThreads) {
    const int h = i / HD, d = i - h * HD;
    float m_all = -INFINITY;
#pragma unroll
    for (int wp = 0; wp < 4; ++wp) m_all = fmaxf(m_all, s_merge[(wp * 8 + h) * (HD + 2) + HD]);
    float sum = 0.0f, l_all = 0.0f;
#pragma unroll
    for (int wp = 0; wp < 4; ++wp) {
      const float* theirs = s_merge + (wp * 8 + h) * (HD + 2);
      const float weight = decode_exp2(theirs[HD] - m_all);  // a warp without keys has m = -inf: weight 0
      sum += weight * theirs[d];
      l_all += weight * theirs[HD + 1];
    }
    const int head = kv * group + h;
    float* dst_partial = partial + ((static_cast<size_t>(row) * heads + head) * max_splits + split) * (HD + 2);
    dst_partial[d] = sum;
    if (d == 0) { dst_partial[HD] = m_all * 0.6931471805599453f; dst_partial[HD + 1] = l_all; }  // the merge kernel works in natural units
  }
}

// ---------------------------------------------------------------------------
// The same attention for steps whose (token, key/value head) pairs are few
// enough that all their blocks can be resident at once but whose tiles are
// too many for that: a pair gets `slots` blocks, and block s takes the 128-key
// tiles first + s, first + s + slots, ... of the token's keys one after
// another, with a running maximum, sum and accumulator per warp. The next
// tile's keys are fetched while this tile's values are still being used, its
// values while the next scores are taken, so two tiles' copies overlap in the
// 64 KB a block holds anyway. Every block is resident from the start, so every
// block's first tile is fetched before the wait for the kernel ahead, and no
// block waits for a slot on an SM behind a whole round of others. A block
// leaves one partial result (slot s of the pair); the merge kernel puts the
// slots together in slot order. Which block takes which tile depends on the
// token's position and on `slots` alone.
template <int HD>
__global__ void __launch_bounds__(kDecodeThreads)
paged_attention_decode_resident_kernel(const __grid_constant__ CUtensorMap map_cache, const __nv_bfloat16* __restrict__ q,
                                       float* __restrict__ partial, const int* __restrict__ block_tables,
                                       int max_pages, const int* __restrict__ row_token,
                                       const int* __restrict__ row_request, const int* __restrict__ positions,
                                       int heads, int kv_heads, int page_tokens, int num_pages, int max_splits,
                                       int window, float scale, int* status) {
  constexpr int HALVES = HD / kTmaColumns;                 // 64-value halves of a row
  constexpr int TILE_BYTES = kSplitKeys * HD * 2;
  extern __shared__ unsigned char tma_decode_raw[];
  __shared__ __align__(8) uint64_t barriers[2];   // keys, values
  unsigned char* sK = tma_decode_raw + ((1024 - (shared_address(tma_decode_raw) & 1023)) & 1023);
  unsigned char* sV = sK + TILE_BYTES;
  float* s_merge = reinterpret_cast<float*>(sK);           // [4 warps][8 heads][HD + 2], over K once the scores exist
  static_assert(4 * 8 * (HD + 2) * sizeof(float) <= TILE_BYTES, "the merge area must fit over the keys");

  const bool release_late = gridDim.x * gridDim.y * gridDim.z > kDecodeBlocksAtOnce;   // as in the kernel above
  if (!release_late) chain_release();
  // What follows up to chain_wait() reads nothing a kernel of this step writes.
  const int rank = blockIdx.x, slots = gridDim.x, kv = blockIdx.y, row = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  // One thread per box: keys or values, page of the tile, 64-value half.
  const int pages = kSplitKeys / page_tokens;   // <= 16
  const int boxes = 2 * pages * HALVES;         // <= 64
  const bool fetcher = tid < boxes;
  const int which = tid / (pages * HALVES), slot = (tid / HALVES) % pages, half = tid % HALVES;
  const int token = row_token[row];
  const int table_row = row_request[row];
  const int* table = block_tables + static_cast<size_t>(table_row) * max_pages;
  // The page of this block's first tile is asked for together with the
  // position, on the guess that no window has moved the first tile.
  int page = 0;
  if (fetcher && rank * pages + slot < max_pages) page = table[rank * pages + slot];
  if (token < 0) return;   // a padding row
  const int pos = positions[token];
  const int group = heads / kv_heads;  // <= 8
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_tile = first_key / kSplitKeys, last_tile = pos / kSplitKeys;
  int tile = first_tile + rank;
  if (first_tile > 0) {
    page = 0;
    if (fetcher && tile * pages + slot < max_pages) page = table[tile * pages + slot];
  }

  if (tid == 0) {
    barrier_init(&barriers[0], 1);
    barrier_init(&barriers[1], 1);
    barrier_init_fence();
    if (tile <= last_tile) {
      barrier_arrive_expect(&barriers[0], TILE_BYTES);   // every box is fetched, whatever it holds
      barrier_arrive_expect(&barriers[1], TILE_BYTES);
    }
  }
  __syncthreads();
  unsigned char* dst = (which ? sV : sK) + half * (kSplitKeys * 128) + slot * page_tokens * 128;
  // The box of page `page_id` of tile `of_tile` for this thread: beyond the
  // cache's last row (zeros) when the page holds none of the token's keys.
  auto box_row_of = [&](int of_tile, int page_id) {
    const int page_key = of_tile * kSplitKeys + slot * page_tokens;
    bool wanted = page_key <= pos && page_key + page_tokens > first_key;
    if (wanted && (page_id < 0 || page_id >= num_pages)) {
      atomicOr(status, kStatusBadPage);
      wanted = false;
    }
    return wanted ? ((page_id * 2 + which) * kv_heads + kv) * page_tokens : num_pages * 2 * kv_heads * page_tokens;
  };
  // The page that holds the token's own position is written by the kernel
  // ahead of this one: it waits; every other page of the first tile is
  // fetched right away.
  bool fresh = false;
  if (fetcher && tile <= last_tile) {
    const int page_key = tile * kSplitKeys + slot * page_tokens;
    fresh = pos >= page_key && pos < page_key + page_tokens;
    if (!fresh) tma_load_2d(dst, &map_cache, half * kTmaColumns, box_row_of(tile, page), &barriers[which]);
  }
  chain_wait();
  if (fresh) tma_load_2d(dst, &map_cache, half * kTmaColumns, box_row_of(tile, page), &barriers[which]);

  // ---- the query heads of this key/value head as rows 0..group-1 of the 16-row operand
  uint32_t qa0[HD / 16], qa2[HD / 16];
  {
    // q is written by the kernel ahead of this one
    const __nv_bfloat16* qrow = behind_wait(q) + (static_cast<size_t>(token) * heads + kv * group + (g < group ? g : 0)) * HD;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks) {
      qa0[ks] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t) : 0u;
      qa2[ks] = g < group ? *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t) : 0u;
    }
  }
  const float scale_log2 = scale * 1.4426950408889634f;
  const int key_base = warp * 32;
  float m_run = -INFINITY, l_run = 0.0f;   // of this warp's keys of all tiles so far, row g
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;

  if (tile > last_tile) return;   // more slots than tiles: the merge skips this one
  for (uint32_t turn = 0; tile <= last_tile; tile += slots, ++turn) {
    const uint32_t parity = turn & 1;
    const int next = tile + slots;
    int next_page = 0;   // asked for now, needed when this tile's keys are used up
    if (fetcher && next <= last_tile && next * pages + slot < max_pages) next_page = table[next * pages + slot];
    const int key0 = tile * kSplitKeys;
    const int lo = max(first_key - key0, 0), hi = min(pos - key0, kSplitKeys - 1);   // the tile's rows that count
    const bool has_keys = key_base <= hi && key_base + 31 >= lo;
    const bool keys_landed = barrier_wait(&barriers[0], parity, status);

    // ---- scores of this warp's 32 keys
    float sc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.0f;
    if (has_keys) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          uint32_t kf[4];
          const int krow = key_base + nb * 16 + (lane & 7) + (lane >> 4) * 8;
          decode_ldmatrix_x4(kf, decode_smem_address(sK + decode_swizzled_offset<HD>(krow, ks * 2 + ((lane >> 3) & 1))));
          decode_mma(sc[2 * nb], qa0[ks], qa2[ks], kf[0], kf[1]);
          decode_mma(sc[2 * nb + 1], qa0[ks], qa2[ks], kf[2], kf[3]);
        }
      }
    }
    // Row g of the tile is query head g; this thread holds keys nb * 8 + 2t, 2t + 1.
    float m_t = -INFINITY;
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kk = key_base + nb * 8 + 2 * t + j;
        sc[nb][j] = kk >= lo && kk <= hi ? sc[nb][j] * scale_log2 : -INFINITY;
        m_t = fmaxf(m_t, sc[nb][j]);
      }
    }
    m_t = fmaxf(m_t, __shfl_xor_sync(0xffffffffu, m_t, 1));
    m_t = fmaxf(m_t, __shfl_xor_sync(0xffffffffu, m_t, 2));
    const float m_new = fmaxf(m_run, m_t);
    const float ref = m_new == -INFINITY ? 0.0f : m_new;
    const float carry = decode_exp2(m_run - ref);   // what earlier tiles gathered, on the new maximum (0 if nothing yet)
    float l_t = 0.0f;
    uint32_t pa0[2], pa2[2];
#pragma unroll
    for (int nb = 0; nb < 4; ++nb) {
      const float p0 = decode_exp2(sc[nb][0] - ref), p1 = decode_exp2(sc[nb][1] - ref);
      l_t += p0 + p1;
      __nv_bfloat162 packed = __floats2bfloat162_rn(p0, p1);
      const uint32_t word = *reinterpret_cast<uint32_t*>(&packed);
      if (nb & 1) pa2[nb >> 1] = word; else pa0[nb >> 1] = word;
    }
    l_t += __shfl_xor_sync(0xffffffffu, l_t, 1);
    l_t += __shfl_xor_sync(0xffffffffu, l_t, 2);
    l_run = l_run * carry + l_t;
    m_run = m_new;

    // Every warp is done with the keys: the next tile's may come. One
    // decision for the whole block if a wait ran out (the status word says so).
    if (__syncthreads_or(!keys_landed)) break;
    if (next <= last_tile) {
      if (tid == 0) barrier_arrive_expect(&barriers[0], TILE_BYTES);
      if (fetcher && which == 0) tma_load_2d(dst, &map_cache, half * kTmaColumns, box_row_of(next, next_page), &barriers[0]);
    }
    const bool values_landed = barrier_wait(&barriers[1], parity, status);

    // A masked key has weight 0, but 0 x NaN is NaN: value rows outside the
    // token's keys (the rest of the last page, whatever an earlier owner of
    // the page left there) are zeroed. A warp reads only its own 32 rows.
    if (has_keys && (key_base < lo || key_base + 31 > hi)) {
      for (int i = lane; i < 32 * (HD / 8); i += 32) {
        const int vrow = key_base + i / (HD / 8);
        if (vrow < lo || vrow > hi)
          *reinterpret_cast<uint4*>(sV + decode_swizzled_offset<HD>(vrow, i % (HD / 8))) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncwarp();
    }

    // ---- o = o * carry + p v over this warp's 32 keys
    if (turn > 0) {
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) { o[i][0] *= carry; o[i][1] *= carry; }
    }
    if (has_keys) {
#pragma unroll
      for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
        for (int nb = 0; nb < HD / 16; ++nb) {
          uint32_t vf[4];
          const int vrow = key_base + ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          decode_ldmatrix_x4_trans(vf, decode_smem_address(sV + decode_swizzled_offset<HD>(vrow, nb * 2 + (lane >> 4))));
          decode_mma(o[2 * nb], pa0[ks], pa2[ks], vf[0], vf[1]);
          decode_mma(o[2 * nb + 1], pa0[ks], pa2[ks], vf[2], vf[3]);
        }
      }
    }
    if (__syncthreads_or(!values_landed)) break;   // every warp is done with the values
    if (next <= last_tile) {
      if (tid == 0) barrier_arrive_expect(&barriers[1], TILE_BYTES);
      if (fetcher && which == 1) tma_load_2d(dst, &map_cache, half * kTmaColumns, box_row_of(next, next_page), &barriers[1]);
    }
  }

  if (release_late) chain_release();
  // ---- the four warps in warp order: this block's partial result (the area lies over K, which is used up)
  if (g < group) {
    float* mine = s_merge + (warp * 8 + g) * (HD + 2);
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      mine[i * 8 + 2 * t] = o[i][0];
      mine[i * 8 + 2 * t + 1] = o[i][1];
    }
    if (t == 0) { mine[HD] = m_run; mine[HD + 1] = l_run; }
  }
  __syncthreads();
  for (int i = tid; i < group * HD; i += kDecodeThreads) {
    const int h = i / HD, d = i - h * HD;
    float m_all = -INFINITY;
#pragma unroll
    for (int wp = 0; wp < 4; ++wp) m_all = fmaxf(m_all, s_merge[(wp * 8 + h) * (HD + 2) + HD]);
    float sum = 0.0f, l_all = 0.0f;
#pragma unroll
    for (int wp = 0; wp < 4; ++wp) {
      const float* theirs = s_merge + (wp * 8 + h) * (HD + 2);
      const float weight = decode_exp2(theirs[HD] - m_all);  // a warp without keys has m = -inf: weight 0
      sum += weight * theirs[d];
      l_all += weight * theirs[HD + 1];
    }
    const int head = kv * group + h;
    // the blocks of a pair lie side by side: gridDim.x partial results a pair, not max_splits
    float* dst_partial = partial + ((static_cast<size_t>(row) * heads + head) * gridDim.x + rank) * (HD + 2);
    dst_partial[d] = sum;
    if (d == 0) { dst_partial[HD] = m_all * 0.6931471805599453f; dst_partial[HD + 1] = l_all; }  // the merge kernel works in natural units
  }
}

// out[token, head, :] = sum_s exp(m_s - M) acc_s / sum_s exp(m_s - M) l_s over
// the splits that hold keys of this token, in ascending order. One block per
// (token, head), one thread per value of the head. A thread fetches the
// maxima, the sums and its own value of up to kMergeSplits splits in one go
// (all loads in flight together: one trip to memory instead of one for the
// maxima, one for the weights and one for the values) and finds the weights
// itself; longer contexts take further rounds with the running maximum
// carried along.
constexpr int kMergeSplits = 32;  // splits per round: 4,096 keys

template <typename T>
__global__ void __launch_bounds__(256)
paged_attention_merge_kernel(const float* __restrict__ partial, T* __restrict__ out,
                             const int* __restrict__ row_token, const int* __restrict__ positions,
                             int rows, int heads, int head_dim, int max_splits, int window, int slots,
                             int* status) {
  chain_release();
  const int row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int token = row_token[row];  // the step's integers are not written by any kernel of the step
  if (token < 0 || d >= head_dim) return;
  const int pos = positions[token];
  const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
  const int first_split = first_key / kSplitKeys, last_split = pos / kSplitKeys;
  if (last_split >= max_splits) {
    // The caller's bound on the contexts does not cover this row: its partial
    // results lie outside what the scratch was sized for. The row is left as it is.
    if (d == 0) atomicOr(status, kStatusBadSlot);
    return;
  }
  // One partial result per split of 128 keys, or (slots > 0) per block of the
  // resident kernel: slot s gathered the tiles first + s, first + s + slots, ...
  const int splits = slots > 0 ? min(slots, last_split - first_split + 1) : last_split - first_split + 1;
  const int stride = head_dim + 2;
  const float* base = partial + (slots > 0 ? (static_cast<size_t>(row) * heads + head) * slots
                                            : (static_cast<size_t>(row) * heads + head) * max_splits + first_split) * stride;
  chain_wait();
  base = behind_wait(base);  // the partial results are written by the kernel ahead of this one
  float m = kDecodeMinusHuge, acc = 0.0f, l = 0.0f;
  for (int chunk = 0; chunk < splits; chunk += kMergeSplits) {
    float ms[kMergeSplits], ls[kMergeSplits], values[kMergeSplits];
#pragma unroll
    for (int j = 0; j < kMergeSplits; ++j) {
      const bool live = chunk + j < splits;
      const float* p = base + static_cast<size_t>(live ? chunk + j : 0) * stride;
      ms[j] = live ? p[head_dim] : kDecodeMinusHuge;
      ls[j] = live ? p[head_dim + 1] : 0.0f;
      values[j] = live ? p[d] : 0.0f;
    }
    float round_max = m;
#pragma unroll
    for (int j = 0; j < kMergeSplits; ++j) round_max = fmaxf(round_max, ms[j]);
    const float carry = expf(m - round_max);  // what earlier rounds gathered, on the new maximum
    acc *= carry;
    l *= carry;
#pragma unroll
    for (int j = 0; j < kMergeSplits; ++j) {
      const float weight = expf(ms[j] - round_max);
      acc = fmaf(weight, values[j], acc);
      l = fmaf(weight, ls[j], l);
    }
    m = round_max;
  }
  out[(static_cast<size_t>(token) * heads + head) * head_dim + d] = from_float<T>(acc / l);
}

}  // namespace mxb
#include "attention_decode_project.cuh"
namespace mxb {

// What follows the attention kernel of a decode step: the merge of the partial
// results into `out`, or (project.w given) the kernel that merges and
// multiplies by the output projection at once.
struct DecodeProject {
  const __nv_bfloat16* w = nullptr;  // W_o [hidden, heads * head_dim], rows ldw values apart
  long long ldw = 0;
  int hidden = 0, tokens = 0;
  float* summands = nullptr;         // [heads, tokens, hidden]
};

template <typename T, int HD, int G>
static int launch_decode(const void* q, const void* cache, void* out, float* partial,
                         const int* block_tables, int max_pages, const int* row_token,
                         const int* row_request, const int* positions, int rows, int heads,
                         int kv_heads, int page_tokens, int num_pages, int max_splits, int window,
                         float scale, int* status, cudaStream_t stream) {
  dim3 grid(max_splits, kv_heads, rows);
  constexpr int kElems = Vec16<T>::kElems;
  constexpr size_t kStage = 2 * static_cast<size_t>(kSplitKeys) * HD * sizeof(T);       // keys and values
  constexpr size_t kReduce = static_cast<size_t>(kDecodeThreads / (HD / kElems)) * G * (HD + 4) * sizeof(float);
  const size_t shared = (kStage > kReduce ? kStage : kReduce) +
                        (static_cast<size_t>(G) * kSplitKeys + G * 2) * sizeof(float);
  auto kernel = paged_attention_decode_kernel<T, HD, G>;
  if (shared > 48 * 1024) {
    cudaError_t attribute = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    if (attribute != cudaSuccess) return static_cast<int>(attribute);
  }
  kernel<<<grid, kDecodeThreads, shared, stream>>>(
      static_cast<const T*>(q), static_cast<const T*>(cache), partial, block_tables, max_pages,
      row_token, row_request, positions, heads, kv_heads, page_tokens, num_pages, max_splits, window,
      scale, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(launch_chained(paged_attention_merge_kernel<T>, dim3(rows, heads), dim3(HD <= 64 ? 64 : (HD <= 128 ? 128 : 256)), 0,
                                         stream, static_cast<const float*>(partial), static_cast<T*>(out),
                                         row_token, positions, rows, heads, HD, max_splits, window, 0, status));
}

static int decode_resident_blocks = 444;   // blocks of the decode attention that fit the GPU at once (3 an SM); 0: always one block per tile
static int decode_many_blocks = 2048;      // blocks of a step with more (token, key/value head) pairs than that

template <int HD>
static int launch_decode_mma(const void* q, const void* cache, void* out, float* partial,
                             const int* block_tables, int max_pages, const int* row_token,
                             const int* row_request, const int* positions, int rows, int heads,
                             int kv_heads, int page_tokens, int num_pages, int max_splits, int window,
                             float scale, int* status, cudaStream_t stream, DecodeProject project = DecodeProject()) {
  static_assert(kSplitKeys == kDecodeThreads, "one thread per key row of a split");
  auto finish = [&](int slots) -> int {
    if (project.w != nullptr)
      return static_cast<int>(launch_merge_project<HD>(partial, project.w, project.ldw, project.summands, row_token,
                                                       positions, rows, project.tokens, heads, project.hidden,
                                                       max_splits, window, slots, kSplitKeys, kDecodeMinusHuge, status,
                                                       stream));
    return static_cast<int>(launch_chained(paged_attention_merge_kernel<__nv_bfloat16>, dim3(rows, heads),
                                           dim3(HD <= 64 ? 64 : (HD <= 128 ? 128 : 256)), 0, stream,
                                           static_cast<const float*>(partial), static_cast<__nv_bfloat16*>(out),
                                           row_token, positions, rows, heads, HD, max_splits, window, slots, status));
  };
  static_assert(4 * 8 * (HD + 2) * sizeof(float) <= kSplitKeys * HD * 2, "the merge area must fit over the keys");
  dim3 grid(max_splits, kv_heads, rows);
  cudaError_t e;
  const long long cache_rows = static_cast<long long>(num_pages) * 2 * kv_heads * page_tokens;
  CUtensorMap map_cache;
  // Pages of 8, 16, ... 128 tokens fill whole 8-row groups of the swizzled
  // tile and divide a split: one TMA box per page and 64-value half. Other
  // page sizes keep the kernel with one bulk copy per row.
  if (page_tokens >= 8 && page_tokens <= kSplitKeys && kSplitKeys % page_tokens == 0 && cache_rows <= 0x7fffffffLL &&
      (reinterpret_cast<uintptr_t>(cache) & 15) == 0 &&
      make_map(&map_cache, cache, static_cast<int>(cache_rows), HD, HD, page_tokens)) {
    const int shared = 2 * kSplitKeys * HD * 2 + 1024;   // keys and values, and room to align them to 1024 bytes
    // A block that walks over several tiles keeps the copy engine busy
    // without a new block's start-up per tile, so a pair of (token, key/value
    // head) gets as few blocks as still fill the GPU: as many as keep the
    // whole grid resident at once when the pairs are few, else a few rounds'
    // worth. Where that would leave a block fewer than two tiles (few pairs,
    // short contexts) one block per tile is as good and simpler.
    const int pairs = rows * kv_heads;
    int slots = 0;
    if (decode_resident_blocks > 0 && pairs > 0) {
      const int target = pairs <= decode_resident_blocks ? decode_resident_blocks : decode_many_blocks;
      slots = target / pairs > 0 ? target / pairs : 1;
    }
    if (slots > 0 && 2 * slots <= max_splits) {
      auto kernel = paged_attention_decode_resident_kernel<HD>;
      cudaError_t attribute = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
      if (attribute != cudaSuccess) return static_cast<int>(attribute);
      e = launch_chained(kernel, dim3(slots, kv_heads, rows), dim3(kDecodeThreads), shared, stream, map_cache,
                         static_cast<const __nv_bfloat16*>(q), partial, block_tables, max_pages, row_token, row_request,
                         positions, heads, kv_heads, page_tokens, num_pages, max_splits, window, scale, status);
      if (e != cudaSuccess) return static_cast<int>(e);
      return finish(slots);
    }
    auto kernel = paged_attention_decode_tma_kernel<HD>;
    cudaError_t attribute = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (attribute != cudaSuccess) return static_cast<int>(attribute);
    e = launch_chained(kernel, grid, dim3(kDecodeThreads), shared, stream, map_cache,
                       static_cast<const __nv_bfloat16*>(q), partial, block_tables, max_pages, row_token, row_request,
                       positions, heads, kv_heads, page_tokens, num_pages, max_splits, window, scale, status);
  } else {
    const int shared = 2 * kSplitKeys * (HD * 2 + 16);
    auto kernel = paged_attention_decode_mma_kernel<HD>;
    cudaError_t attribute = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (attribute != cudaSuccess) return static_cast<int>(attribute);
    e = launch_chained(kernel, grid, dim3(kDecodeThreads), shared, stream,
                       static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(cache),
                       partial, block_tables, max_pages, row_token, row_request, positions, heads,
                       kv_heads, page_tokens, num_pages, max_splits, window, scale, status);
  }
  if (e != cudaSuccess) return static_cast<int>(e);
  return finish(0);
}

}  // namespace mxb

using namespace mxb;

// Whether the split kernel takes this shape (else the caller uses the general
// tile kernel): head_dim 64 or 128 (and 256 in bfloat16), up to 8 query heads
// per key/value head.
MXB_API int mxb_paged_attention_decode_supported(int head_dim, int heads, int kv_heads, int dtype) {
  if (kv_heads <= 0 || heads % kv_heads != 0 || heads / kv_heads > 8) return 0;
  if (dtype != kF32 && dtype != kBF16) return 0;
  return head_dim == 64 || head_dim == 128 || (head_dim == 256 && dtype == kBF16) ? 1 : 0;
}

MXB_API int mxb_paged_attention_split_keys() { return kSplitKeys; }

// How many blocks of the bfloat16 decode attention the GPU holds at once (3
// an SM with their 64 KB of keys and values), and how many blocks a step with
// more (token, key/value head) pairs than that is cut into. 0: one block per
// tile always.
MXB_API int mxb_set_decode_resident_blocks(int blocks, int many) {
  if (blocks < 0 || many < blocks) return static_cast<int>(cudaErrorInvalidValue);
  decode_resident_blocks = blocks;
  decode_many_blocks = many;
  return 0;
}

// partial: float32 scratch of rows * heads * max_splits * (head_dim + 2) values.
// rows of row_token that are negative are padding. max_splits must cover the
// longest context: ceil(longest / 128).
MXB_API int mxb_paged_attention_decode(const void* q, const void* cache, void* out, float* partial,
                                       const int* block_tables, int max_pages, const int* row_token,
                                       const int* row_request, const int* positions, int rows,
                                       int heads, int kv_heads, int head_dim, int page_tokens,
                                       int num_pages, int max_splits, int window, float scale,
                                       int dtype, int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (!mxb_paged_attention_decode_supported(head_dim, heads, kv_heads, dtype) || max_splits <= 0)
    return static_cast<int>(cudaErrorInvalidValue);
  const int group = heads / kv_heads;
#define ARGS q, cache, out, partial, block_tables, max_pages, row_token, row_request, positions, rows, \
             heads, kv_heads, page_tokens, num_pages, max_splits, window, scale, status, stream
#define BY_GROUP(T, HD)                                        \
  if (group == 1) return launch_decode<T, HD, 1>(ARGS);        \
  if (group == 2) return launch_decode<T, HD, 2>(ARGS);        \
  if (group <= 4) return launch_decode<T, HD, 4>(ARGS);        \
  return launch_decode<T, HD, 8>(ARGS);
  if (dtype == kBF16 && (head_dim == 64 || head_dim == 128)) {
    return head_dim == 64 ? launch_decode_mma<64>(ARGS) : launch_decode_mma<128>(ARGS);
  }
  if (dtype == kBF16) {
    if (head_dim == 256) { BY_GROUP(__nv_bfloat16, 256) }
  } else {
    if (head_dim == 64) { BY_GROUP(float, 64) }
    if (head_dim == 128) { BY_GROUP(float, 128) }
  }
#undef BY_GROUP
#undef ARGS
  return static_cast<int>(cudaErrorInvalidValue);
}

// Whether mxb_paged_attention_decode_project takes this shape.
MXB_API int mxb_paged_attention_decode_project_supported(int head_dim, int heads, int kv_heads, int dtype, int tokens,
                                                        const void* w, long long ldw) {
  return dtype == kBF16 && mxb_paged_attention_decode_supported(head_dim, heads, kv_heads, dtype) &&
                 decode_project_takes(head_dim, tokens, w, ldw) ? 1 : 0;
}

// The decode attention followed at once by the output projection (bfloat16):
// summands[h, token, :] = (attention output of head h) * W_o[:, h * head_dim ...]^T
// in float32, [heads, tokens, hidden]; their sum over h is the projected
// output. Tokens that no row names give zeros. w: [hidden, heads * head_dim].
MXB_API int mxb_paged_attention_decode_project(const void* q, const void* cache, float* partial,
                                               const int* block_tables, int max_pages, const int* row_token,
                                               const int* row_request, const int* positions, int rows, int tokens,
                                               int heads, int kv_heads, int head_dim, int page_tokens, int num_pages,
                                               int max_splits, int window, float scale, const void* w, long long ldw,
                                               int hidden, float* summands, int* status, cudaStream_t stream) {
  if (rows <= 0 || hidden <= 0 || max_splits <= 0) return static_cast<int>(cudaErrorInvalidValue);
  if (!mxb_paged_attention_decode_project_supported(head_dim, heads, kv_heads, kBF16, tokens, w, ldw))
    return static_cast<int>(cudaErrorInvalidValue);
  DecodeProject project;
  project.w = static_cast<const __nv_bfloat16*>(w);
  project.ldw = ldw;
  project.hidden = hidden;
  project.tokens = tokens;
  project.summands = summands;
  void* out = nullptr;
#define ARGS q, cache, out, partial, block_tables, max_pages, row_token, row_request, positions, rows, \
             heads, kv_heads, page_tokens, num_pages, max_splits, window, scale, status, stream, project
  return head_dim == 64 ? launch_decode_mma<64>(ARGS) : launch_decode_mma<128>(ARGS);
#undef ARGS
}

// ---------------------------------------------------------------------------
// The same attention for callers that cannot allocate: see
// attention_decode_noalloc.h. The partial results live in a fixed array
// inside the library instead of a buffer from the caller.
#include <cstdio>
#include <mutex>

#include "attention_decode_noalloc.h"

namespace mxb {

// Device memory of every GPU that loads this library, until the process ends.
static __device__ __align__(256) unsigned char noalloc_scratch[MXB_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static float* noalloc_address[kMaxDevices];  // the array's device address, per device
static std::mutex noalloc_mutex;

// In host code `noalloc_scratch` is only a handle of the symbol, not memory a
// kernel may touch; the address kernels can use comes from the runtime, once
// per device, with that device current.
static cudaError_t noalloc_scratch_address(float** address) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return e;
  if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> guard(noalloc_mutex);
  if (noalloc_address[device] == nullptr) {
    void* found = nullptr;
    e = cudaGetSymbolAddress(&found, noalloc_scratch);
    if (e != cudaSuccess) return e;
    noalloc_address[device] = static_cast<float*>(found);
  }
  *address = noalloc_address[device];
  return cudaSuccess;
}

}  // namespace mxb

MXB_API int mxb_paged_attention_decode_noalloc(const void* q, const void* cache, void* out,
                                               const int* block_tables, int max_pages,
                                               const int* row_token, const int* row_request,
                                               const int* positions, int rows, int heads, int kv_heads,
                                               int head_dim, int page_tokens, int num_pages,
                                               int longest_context, int window, float scale, int dtype,
                                               int* status, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (longest_context <= 0 || heads <= 0 || head_dim <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const int splits = (longest_context + kSplitKeys - 1) / kSplitKeys;
  const unsigned long long need = static_cast<unsigned long long>(rows) * heads * splits *
                                  (head_dim + 2) * sizeof(float);
  if (need > MXB_NOALLOC_SCRATCH_BYTES) {
    std::fprintf(stderr,
                 "mxb_paged_attention_decode_noalloc: %d rows x %d heads x %d splits x (%d + 2) floats "
                 "= %llu bytes of scratch, the built-in array holds %u; use fewer rows per call or "
                 "mxb_paged_attention_decode with a buffer of your own\n",
                 rows, heads, splits, head_dim, need, MXB_NOALLOC_SCRATCH_BYTES);
    return static_cast<int>(cudaErrorInvalidValue);
  }
  float* scratch = nullptr;
  const cudaError_t e = noalloc_scratch_address(&scratch);
  if (e != cudaSuccess) return static_cast<int>(e);
  return mxb_paged_attention_decode(q, cache, out, scratch, block_tables, max_pages, row_token,
                                    row_request, positions, rows, heads, kv_heads, head_dim, page_tokens,
                                    num_pages, splits, window, scale, dtype, status, stream);
}

MXB_TIMELINE_EXPORT(mxb_timeline_attention)
