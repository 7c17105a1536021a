// Causal grouped-query attention for prompt portions in bfloat16 on the
// fifth-generation tensor cores, over the paged cache (which already holds
// this step's own keys and values).
//
// One block takes up to 128 consecutive query tokens of one request and one
// query head and walks the request's keys in tiles of 128 absolute positions.
//   warp 0, 18  fetch: warp 0 the query tile once and the keys, warp 18 the
//               values, for every key tile the pages the block table names as
//               TMA boxes of one page x 64 values with the 128-byte swizzle
//               (so a tile of K is a K-major operand and a tile of V an
//               MN-major one, as they lie in the cache);
//   warp 1      owns tensor memory and issues the MMAs: S = Q K^T into one of
//               two score buffers, and O_tile = P V into one of two output
//               buffers, with P read from tensor memory where the softmax
//               warps left it (over the scores it came from);
//   warps 2..17 four threads per query row, each with a quarter of the tile's
//               keys and a quarter of the head's values: mask, running maximum
//               (the four exchange their maxima once per tile) and sum in float32,
//               P = exp2(...) back to tensor memory as bfloat16, and the
//               row's output accumulator in registers: acc = acc * alpha +
//               O_tile, read back with tcgen05.ld.
// The MMAs of tile j + 1's scores run while the softmax of tile j does, and
// the accumulation of tile j - 1 while P_j V_j runs.
//
// Key tiles start at multiples of 128 of the absolute position and a row's
// arithmetic does not depend on the other rows of its tile, so a position's
// result is the same however the prompt was cut.
//
// Replaces the reference's gather of the whole context plus
// fast::scaled_dot_product_attention with a causal mask aligned to the last
// key (crates/models/qwen/src/forward/paged.rs:1143-1148, :1176-1184;
// crates/models/qwen/src/forward.rs:1967-1989).
//
// Every wait on a barrier is bounded: if one runs out, the status word gets a
// bit, the block stops issuing work, frees its tensor memory and leaves.
#include "tcgen05.cuh"

namespace mxb {

constexpr int kFaRows = 128;     // query rows of a block
constexpr int kFaKeys = 128;     // keys of a tile
constexpr int kFaParts = 4;      // threads per query row
constexpr int kFaSoftmaxThreads = kFaParts * kFaRows;
constexpr int kFaThreads = 64 + kFaSoftmaxThreads + 32;   // fetch (keys), MMA, softmax, fetch (values)
constexpr int kFaValueWarp = kFaThreads / 32 - 1;
constexpr int kFaTmemColumns = 512;
constexpr int kFaHalfBytes = 128 * kTmaColumns * 2;  // a [128 x 64] bfloat16 operand block: 16 KiB

template <int HD> struct FaConfig {
  static constexpr int kHalves = HD / kTmaColumns;
  static constexpr int kTileBytes = kHalves * kFaHalfBytes;    // Q, a K stage or a V stage
  static constexpr int kKeyStages = HD == 64 ? 4 : 3;          // at most; one block per SM either way
  static constexpr int kValueStages = HD == 64 ? 4 : 2;
  static constexpr int kSmallBytes = 512 + 2 * kFaParts * kFaRows * 4;  // barriers and the exchange of maxima, after the tiles
  // Wanted: the tiles of every stage, the small area and room to align to 1024 bytes.
  static constexpr int kSharedBytes = (1 + kKeyStages + kValueStages) * kTileBytes + kSmallBytes + 1024;
  static constexpr int kScoreColumns = kFaKeys;                // two buffers of 128 columns
  static constexpr int kOutputBase = 2 * kFaKeys;              // then two buffers of HD columns
};

__device__ __forceinline__ float fa_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t fa_pack(float lo, float hi) {
  __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&pair);
}

template <int HD>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_cache,
                             __nv_bfloat16* __restrict__ out, const int* __restrict__ block_tables, int max_pages,
                             const int* __restrict__ tile_request, const int* __restrict__ tile_start,
                             const int* __restrict__ tile_length, const int* __restrict__ positions, int heads,
                             int kv_heads, int page_tokens, int num_pages, int window, float scale,
                             int shared_bytes, float* __restrict__ partial, int* status) {
  using Config = FaConfig<HD>;
  constexpr int MAX_STAGES = Config::kKeyStages;
  constexpr int HALVES = Config::kHalves;
  // All shared memory is dynamic: the block gets `shared_bytes` (up to the
  // device's limit) and uses as many key stages as fit behind the 1024-byte
  // boundary the swizzled tiles need.
  extern __shared__ unsigned char fa_shared_raw[];
  const int slack = (1024 - (shared_address(fa_shared_raw) & 1023)) & 1023;
  const int VS = Config::kValueStages;
  const int fitting = (shared_bytes - slack - Config::kSmallBytes) / Config::kTileBytes - 1 - VS;
  const int KS = fitting < MAX_STAGES ? fitting : MAX_STAGES;
  if (KS < 1) {  // the launcher asks for more than that
    if (threadIdx.x == 0) atomicOr(status, kStatusWaitTimeout);
    return;
  }
  unsigned char* q_tile = fa_shared_raw + slack;
  unsigned char* k_tiles = q_tile + Config::kTileBytes;
  unsigned char* v_tiles = k_tiles + KS * Config::kTileBytes;
  unsigned char* small = v_tiles + VS * Config::kTileBytes;
  uint64_t* q_full = reinterpret_cast<uint64_t*>(small);
  uint64_t* k_full = q_full + 1;
  uint64_t* k_empty = k_full + MAX_STAGES;
  uint64_t* v_full = k_empty + MAX_STAGES;
  uint64_t* v_empty = v_full + MAX_STAGES;
  uint64_t* s_full = v_empty + MAX_STAGES;
  uint64_t* p_full = s_full + 2;
  uint64_t* o_full = p_full + 2;
  uint64_t* row_ready = o_full + 2;  // [4]: the softmax warps of a lane group meet here
  uint64_t* v_tail = row_ready + 4;   // the values of a request's last page land here first
  uint32_t& tmem_base_slot = *reinterpret_cast<uint32_t*>(v_tail + 1);
  volatile int& failed = *reinterpret_cast<volatile int*>(&tmem_base_slot + 1);
  // [tile parity][part][row]: the threads of a row exchange maxima (and, at the end, sums)
  float (*row_max)[kFaParts][kFaRows] = reinterpret_cast<float (*)[kFaParts][kFaRows]>(small + 512);
  static_assert((1 + 4 * MAX_STAGES + 8 + 4 + 1) * 8 + 8 <= 512, "the barriers do not fit their area");

  const int head = blockIdx.x, tile = blockIdx.y;  // heads of one tile run side by side and share its keys in L2
  const int kv = head / (heads / kv_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = tile_start[tile], n = tile_length[tile];
  const int pos0 = positions[t0];
  const int last_pos = pos0 + n - 1;
  const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
  // The key tiles of this query tile. With gridDim.z > 1 they are shared out
  // among that many blocks (a portion of a prompt behind a long context is few
  // query tiles with many key tiles each: this way it still fills the GPU);
  // each block then leaves its unnormalised output, maximum and sum in
  // `partial` and a second kernel puts them together. A block's share may be empty.
  const int all_begin = first_key / kFaKeys, all_end = last_pos / kFaKeys;   // all_end holds the tile's last position
  const int all_tiles = all_end - all_begin + 1;
  const int shares = gridDim.z, share = blockIdx.z;
  const int tile_begin = all_begin + static_cast<int>(static_cast<long long>(share) * all_tiles / shares);
  const int key_tiles = all_begin + static_cast<int>(static_cast<long long>(share + 1) * all_tiles / shares) - tile_begin;

  if (threadIdx.x == 0) {
    barrier_init(q_full, 1);
    for (int s = 0; s < MAX_STAGES; ++s) {
      barrier_init(&k_full[s], 1);
      barrier_init(&k_empty[s], 1);
      barrier_init(&v_full[s], 1);
      barrier_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(&s_full[b], 1);
      barrier_init(&p_full[b], kFaSoftmaxThreads);   // every softmax thread arrives
      barrier_init(&o_full[b], 1);
    }
    for (int g = 0; g < 4; ++g) barrier_init(&row_ready[g], kFaParts * 32);
    barrier_init(v_tail, 1);
    barrier_init_fence();
    failed = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(shared_address(&tmem_base_slot)), "r"(kFaTmemColumns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0 || warp == kFaValueWarp) {
    // ---- fetch: warp 0 the query tile and the keys, the last warp the values
    // of every key tile, page by page. A warp's 32 TMA requests of one tile go
    // out one after the other (some 37 cycles each: with keys and values on
    // one warp the fetch paced the whole block), so keys and values have a
    // warp each; the page of the next tile is looked up a tile ahead.
    const bool values = warp == kFaValueWarp;
    const int stages = values ? VS : KS;
    uint64_t* full = values ? v_full : k_full;
    uint64_t* empty = values ? v_empty : k_empty;
    unsigned char* tiles = values ? v_tiles : k_tiles;
    const int* table = block_tables + static_cast<size_t>(tile_request[tile]) * max_pages;
    if (!values && lane == 0) {
      barrier_arrive_expect(q_full, Config::kTileBytes);
      for (int half = 0; half < HALVES; ++half)
        tma_load_2d(q_tile + half * kFaHalfBytes, &map_q, head * HD + half * kTmaColumns, t0, q_full);
    }
    const int pages_per_tile = kFaKeys / page_tokens;
    const int copies = pages_per_tile * HALVES;  // every page, every 64-value half
    const int slot = lane / HALVES, half = lane % HALVES;  // copies <= 32: one per lane
    const uint32_t offset = half * kFaHalfBytes + slot * page_tokens * (kTmaColumns * 2);
    // Pages no row of the tile can see are not looked up: their box starts
    // beyond the cache's last row, where the copy engine writes zeros. A
    // masked key has weight 0, but 0 x NaN is NaN, so nothing is asked of what
    // the cache holds beyond the request's own positions: the rows of its last
    // page behind the tile's last position are zeroed here before the MMA
    // warp may read the values (the keys' scores are replaced, not weighted).
    constexpr int kNoPage = -0x40000000;
    const int beyond_cache = num_pages * 2 * kv_heads * page_tokens;
    auto page_of = [&](int i) {
      const int page_key = (tile_begin + i) * kFaKeys + slot * page_tokens;
      if (i < key_tiles && lane < copies && page_key <= last_pos && page_key + page_tokens > first_key &&
          page_key / page_tokens < max_pages)
        return table[page_key / page_tokens];
      return kNoPage;
    };
    int page = page_of(0);
    for (int i = 0; i < key_tiles && !failed; ++i) {
      const int stage = i % stages;
      const int upcoming = page_of(i + 1);   // in flight while this tile's requests go out
      if (page != kNoPage && (page < 0 || page >= num_pages)) {
        atomicOr(status, kStatusBadPage);
        page = kNoPage;
      }
      const int box_row = page == kNoPage ? beyond_cache
                                          : ((page * 2 + (values ? 1 : 0)) * kv_heads + kv) * page_tokens;
      // rows [zero_from, zero_to) of the tile: the last page's rows behind the last position
      const int zero_from = last_pos + 1 - (tile_begin + i) * kFaKeys;
      const int zero_to = (last_pos / page_tokens + 1) * page_tokens - (tile_begin + i) * kFaKeys;
      const bool tail = values && tile_begin + i == all_end && zero_from < zero_to;
      uint64_t* landing = tail ? v_tail : &full[stage];
      // K as soon as the scores that read this stage last are done, V when the P V product is.
      if (!barrier_wait(&empty[stage], ((i / stages) & 1) ^ 1, status)) { failed = 1; break; }
      if (lane == 0) barrier_arrive_expect(landing, Config::kTileBytes);
      __syncwarp();
      unsigned char* stage_tile = tiles + stage * Config::kTileBytes;
      if (lane < copies)
        tma_load_2d(stage_tile + offset, &map_cache, half * kTmaColumns, box_row, landing);
      if (tail) {
        if (!barrier_wait(v_tail, 0, status)) { failed = 1; break; }
        // a key's 64 values of one half are 128 bytes, swizzled among themselves
        for (int c = lane; c < (zero_to - zero_from) * HALVES * 8; c += 32)
          *reinterpret_cast<uint4*>(stage_tile + ((c >> 3) % HALVES) * kFaHalfBytes +
                                    (zero_from + c / (HALVES * 8)) * (kTmaColumns * 2) + (c & 7) * 16) =
              make_uint4(0u, 0u, 0u, 0u);
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // before the tensor core reads them
        __syncwarp();
        if (lane == 0) barrier_arrive(&full[stage]);
      }
      page = upcoming;
    }
  } else if (warp == 1) {
    // ---- one thread issues every MMA
    if (lane == 0) {
      constexpr uint32_t idesc_s = tc_instruction_descriptor(kFaRows, kFaKeys);
      constexpr uint32_t idesc_o = tc_instruction_descriptor_b_mn(kFaRows, HD);
      // This one thread is the block's pacemaker: what it does per key tile
      // (three waits, sixteen MMAs, four commits) is kept short. The
      // descriptors of the operands are made once; a stage or a step along k
      // only adds to their address field (16-byte units, no carry: shared
      // memory ends below 256 KiB).
      const uint64_t q_desc = tc_smem_descriptor(shared_address(q_tile));
      const uint64_t k_desc = tc_smem_descriptor(shared_address(k_tiles));
      const uint64_t v_desc = tc_smem_descriptor_mn(shared_address(v_tiles), kFaHalfBytes);
      bool ok = barrier_wait(q_full, 0, status);
      auto scores = [&](int i) {  // S_i = Q K_i^T
        const int stage = i % KS;
        if (!barrier_wait(&k_full[stage], (i / KS) & 1, status)) return false;
        tc_fence_after_sync();
        const uint64_t k_stage = k_desc + static_cast<uint64_t>(stage) * (Config::kTileBytes >> 4);
        const uint32_t tmem_s = tmem_base + (i & 1) * Config::kScoreColumns;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint64_t offset = ((kk / 4) * kFaHalfBytes + (kk % 4) * 32) >> 4;
          tc_mma(tmem_s, q_desc + offset, k_stage + offset, idesc_s, kk > 0 ? 1u : 0u);
        }
        tc_commit(&k_empty[stage]);
        tc_commit(&s_full[i & 1]);
        return true;
      };
      auto outputs = [&](int i) {  // O_tile_i = P_i V_i
        const int stage = i % VS, buffer = i & 1;
        if (!barrier_wait(&v_full[stage], (i / VS) & 1, status)) return false;
        // The output buffer is free: every softmax thread took tile i - 2 out of
        // it before it arrived for P of tile i - 1, let alone of tile i.
        if (!barrier_wait(&p_full[buffer], (i >> 1) & 1, status)) return false;
        tc_fence_after_sync();
        const uint64_t v_stage = v_desc + static_cast<uint64_t>(stage) * (Config::kTileBytes >> 4);
        const uint32_t tmem_p = tmem_base + buffer * Config::kScoreColumns;
        const uint32_t tmem_o = tmem_base + Config::kOutputBase + buffer * HD;
#pragma unroll
        for (int kk = 0; kk < kFaKeys / 16; ++kk) {  // 16 keys per instruction: two 8-row groups of V, 8 columns of P
          // P of the keys' quarter q lies over the first half of that quarter's score columns.
          tc_mma_ts(tmem_o, tmem_p + (kk / 2) * (kFaKeys / kFaParts) + (kk % 2) * 8, v_stage + kk * (2048 >> 4),
                    idesc_o, kk > 0 ? 1u : 0u);
        }
        tc_commit(&v_empty[stage]);
        tc_commit(&o_full[buffer]);
        return true;
      };
      ok = ok && (key_tiles == 0 || scores(0));
      for (int i = 0; i < key_tiles && ok && !failed; ++i) {
        if (i + 1 < key_tiles) ok = scores(i + 1);
        ok = ok && outputs(i);
      }
      if (!ok) failed = 1;
    }
  } else {
    // ---- softmax and accumulation: four threads per query row. Warps w,
    // w + 4, w + 8 and w + 12 reach the same 32 lanes of tensor memory; each
    // takes 32 keys of a tile and HD / 4 values of the output.
    constexpr int PART_KEYS = kFaKeys / kFaParts, PART_HD = HD / kFaParts;
    static_assert(PART_KEYS == 32 && (PART_HD == 16 || PART_HD == 32), "the tensor-memory loads below take 16 or 32 columns");
    const int lane_base = (warp & 3) * 32;
    const int part = (warp - 2) >> 2;
    const int row = lane_base + lane;
    const bool valid = row < n;
    const int pos = pos0 + row;
    const int key_hi = valid ? pos : -1;                                   // last key this row sees
    const int key_lo = window > 0 ? max(0, pos - window + 1) : 0;          // first key this row sees
    const float scale_log2 = scale * 1.4426950408889634f;
    const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
    uint64_t* meet = &row_ready[warp & 3];
    float acc[PART_HD];
#pragma unroll
    for (int i = 0; i < PART_HD; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f, alpha_pending = 0.0f;
    bool ok = true;

    auto accumulate = [&](int i, float alpha) {  // acc = acc * alpha + O_tile_i
      const int buffer = i & 1;
      if (!barrier_wait(&o_full[buffer], (i >> 1) & 1, status)) return false;
      tc_fence_after_sync();
      uint32_t o[PART_HD];
      tc_load(tmem_lane + Config::kOutputBase + buffer * HD + part * PART_HD, o);
      tc_fence_before_sync();   // the MMA thread reuses the buffer only behind this thread's next arrival for P
#pragma unroll
      for (int j = 0; j < PART_HD; ++j) acc[j] = fmaf(acc[j], alpha, __uint_as_float(o[j]));
      return true;
    };

    for (int i = 0; i < key_tiles; ++i) {
      const int buffer = i & 1;
      const int key0 = (tile_begin + i) * kFaKeys + part * PART_KEYS;  // first key of this thread's share
      if (!barrier_wait(&s_full[buffer], (i >> 1) & 1, status) || failed) { ok = false; break; }
      tc_fence_after_sync();
      const uint32_t tmem_s = tmem_lane + buffer * Config::kScoreColumns + part * PART_KEYS;
      const bool all_seen = key0 >= key_lo && key0 + PART_KEYS - 1 <= key_hi;
      uint32_t raw[PART_KEYS];
      tc_load_32(tmem_s, raw);
      float s[PART_KEYS];
      if (all_seen) {
#pragma unroll
        for (int j = 0; j < PART_KEYS; ++j) s[j] = __uint_as_float(raw[j]);
      } else {
#pragma unroll
        for (int j = 0; j < PART_KEYS; ++j)
          s[j] = key0 + j >= key_lo && key0 + j <= key_hi ? __uint_as_float(raw[j]) : -INFINITY;
      }
      // Running maximum, already multiplied by scale * log2(e) (scale > 0 keeps the order).
      float max4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < PART_KEYS; ++j) max4[j & 3] = fmaxf(max4[j & 3], s[j]);
      row_max[buffer][part][row] = fmaxf(fmaxf(max4[0], max4[1]), fmaxf(max4[2], max4[3]));
      barrier_arrive(meet);
      if (!barrier_wait(meet, i & 1, status)) { ok = false; break; }
      const float tile_max = fmaxf(fmaxf(row_max[buffer][0][row], row_max[buffer][1][row]),
                                   fmaxf(row_max[buffer][2][row], row_max[buffer][3][row]));
      const float m_new = fmaxf(m, tile_max * scale_log2);
      // A row that has seen no key yet keeps a finite reference so that no inf - inf appears.
      const float ref = m_new == -INFINITY ? 0.0f : m_new;
      const float alpha = fa_exp2(m - ref);
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      uint32_t packed[PART_KEYS / 2];
#pragma unroll
      for (int j = 0; j < PART_KEYS; j += 2) {
        // A masked score is -inf here and gives exactly 0.
        const float p0 = fa_exp2(fmaf(s[j], scale_log2, -ref));
        const float p1 = fa_exp2(fmaf(s[j + 1], scale_log2, -ref));
        sum4[(j >> 1) & 3] += p0 + p1;
        packed[j >> 1] = fa_pack(p0, p1);
      }
      // P lies over the scores it came from: columns only this thread reads.
      tc_store_16(tmem_s, packed);
      tc_store_wait();
      tc_fence_before_sync();
      barrier_arrive(&p_full[buffer]);
      l = fmaf(l, alpha, (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]));
      m = m_new;
      if (i > 0 && !accumulate(i - 1, alpha_pending)) { ok = false; break; }
      alpha_pending = alpha;
    }
    if (ok && !failed && key_tiles > 0) ok = accumulate(key_tiles - 1, alpha_pending);
    if (!ok) failed = 1;
    // The row's sum: this thread's keys plus its partners' (all scaled to the
    // same final maximum). The buffer of this parity was last read two
    // exchanges ago.
    row_max[key_tiles & 1][part][row] = l;
    barrier_arrive(meet);
    if (ok && !barrier_wait(meet, key_tiles & 1, status)) ok = false;
    l = (row_max[key_tiles & 1][0][row] + row_max[key_tiles & 1][1][row]) +
        (row_max[key_tiles & 1][2][row] + row_max[key_tiles & 1][3][row]);
    if (!ok) failed = 1;
    if (ok && valid && partial != nullptr) {
      // [token][head][share][HD values, maximum (in units of log 2), sum]
      float* dst = partial + ((static_cast<size_t>(t0 + row) * heads + head) * shares + share) * (HD + 2);
#pragma unroll
      for (int c = 0; c < PART_HD; c += 4)
        *reinterpret_cast<float2*>(dst + part * PART_HD + c) = make_float2(acc[c], acc[c + 1]),
        *reinterpret_cast<float2*>(dst + part * PART_HD + c + 2) = make_float2(acc[c + 2], acc[c + 3]);
      if (part == 0) { dst[HD] = m; dst[HD + 1] = l; }
    } else if (ok && valid) {
      const float inv = 1.0f / l;
      __nv_bfloat16* dst = out + (static_cast<size_t>(t0 + row) * heads + head) * HD + part * PART_HD;
#pragma unroll
      for (int c = 0; c < PART_HD; c += 8) {
        *reinterpret_cast<uint4*>(dst + c) =
            make_uint4(fa_pack(acc[c] * inv, acc[c + 1] * inv), fa_pack(acc[c + 2] * inv, acc[c + 3] * inv),
                       fa_pack(acc[c + 4] * inv, acc[c + 5] * inv), fa_pack(acc[c + 6] * inv, acc[c + 7] * inv));
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (failed && threadIdx.x == 0) {
    // A wait ran out somewhere. Give loads that may still be in flight a
    // millisecond before the block's shared memory goes back.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kFaTmemColumns) : "memory");
  }
}

// out[token, head, :] from the shares' unnormalised outputs, maxima and sums:
// a block per (head, query tile, group of rows), one thread per value of the
// head; a block takes every kMergeGroups-th row of the tile, so that the
// trips to memory of many rows are under way at once.
constexpr int kMergeGroups = 32;
constexpr int kMergeShares = 8;   // at most

template <int HD>
__global__ void __launch_bounds__(HD)
flash_prefill_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out,
                           const int* __restrict__ tile_start, const int* __restrict__ tile_length, int heads,
                           int shares) {
  const int head = blockIdx.x, tile = blockIdx.y, d = threadIdx.x;
  const int t0 = tile_start[tile], n = tile_length[tile];
  for (int row = blockIdx.z; row < n; row += kMergeGroups) {
    const float* base = partial + (static_cast<size_t>(t0 + row) * heads + head) * shares * (HD + 2);
    float maxima[kMergeShares], sums[kMergeShares], values[kMergeShares];
#pragma unroll
    for (int s = 0; s < kMergeShares; ++s) {   // every load first, then the arithmetic
      const bool live = s < shares;
      maxima[s] = live ? base[s * (HD + 2) + HD] : -INFINITY;
      sums[s] = live ? base[s * (HD + 2) + HD + 1] : 0.0f;
      values[s] = live ? base[s * (HD + 2) + d] : 0.0f;
    }
    float highest = -INFINITY;
#pragma unroll
    for (int s = 0; s < kMergeShares; ++s) highest = fmaxf(highest, maxima[s]);
    float value = 0.0f, sum = 0.0f;
#pragma unroll
    for (int s = 0; s < kMergeShares; ++s) {   // a share without keys of this row has maximum -inf and weight 0
      const float weight = fa_exp2(maxima[s] - highest);
      value = fmaf(weight, values[s], value);
      sum = fmaf(weight, sums[s], sum);
    }
    out[(static_cast<size_t>(t0 + row) * heads + head) * HD + d] = __float2bfloat16_rn(value / sum);
  }
}

template <int HD>
static int launch_flash_tc(const void* q, const void* cache, void* out, const int* block_tables, int max_pages,
                           const int* tile_request, const int* tile_start, const int* tile_length,
                           const int* positions, int tokens, int tiles, int heads, int kv_heads, int page_tokens,
                           int num_pages, int window, float scale, int key_shares, float* partial, int* status,
                           cudaStream_t stream) {
  using Config = FaConfig<HD>;
  CUtensorMap map_q, map_cache;
  // q as [tokens, heads * HD]; the cache as [pages * 2 * kv_heads * page_tokens, HD].
  const long long cache_rows = static_cast<long long>(num_pages) * 2 * kv_heads * page_tokens;
  if (cache_rows > 0x7fffffffLL) return static_cast<int>(cudaErrorInvalidValue);
  if (!make_map(&map_q, q, tokens, heads * HD, static_cast<long long>(heads) * HD, kFaRows) ||
      !make_map(&map_cache, cache, static_cast<int>(cache_rows), HD, HD, page_tokens))
    return static_cast<int>(cudaErrorInvalidValue);
  auto kernel = flash_prefill_tcgen05_kernel<HD>;
  static int shared_limit = 0;
  if (shared_limit == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&shared_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, device);
  }
  const int shared_bytes = Config::kSharedBytes < shared_limit ? Config::kSharedBytes : shared_limit;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  const bool shared_out = key_shares > 1;
  dim3 grid(heads, tiles, shared_out ? key_shares : 1);
  kernel<<<grid, kFaThreads, shared_bytes, stream>>>(
      map_q, map_cache, static_cast<__nv_bfloat16*>(out), block_tables, max_pages, tile_request, tile_start,
      tile_length, positions, heads, kv_heads, page_tokens, num_pages, window, scale, shared_bytes,
      shared_out ? partial : nullptr, status);
  e = cudaGetLastError();
  if (e != cudaSuccess || !shared_out) return static_cast<int>(e);
  flash_prefill_merge_kernel<HD><<<dim3(heads, tiles, kMergeGroups), HD, 0, stream>>>(
      partial, static_cast<__nv_bfloat16*>(out), tile_start, tile_length, heads, key_shares);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mxb

using namespace mxb;

// bfloat16, head_dim 64 or 128, pages of 8, 16, 32, 64 or 128 tokens (a page
// must fill whole 8-row groups of the swizzled tile and divide a key tile).
MXB_API int mxb_flash_prefill_tcgen05_supported(int head_dim, int heads, int kv_heads, int page_tokens, int dtype) {
  if (kv_heads <= 0 || heads % kv_heads != 0 || dtype != kBF16) return 0;
  if (head_dim != 64 && head_dim != 128) return 0;
  if (page_tokens < 8 || page_tokens > kFaKeys || kFaKeys % page_tokens != 0) return 0;
  return 1;
}

MXB_API int mxb_flash_prefill_tcgen05_tile() { return kFaRows; }

// Query tiles of up to 128 tokens each; q and out are [tokens, heads, head_dim].
// key_shares > 1: that many blocks share a query tile's keys; partial is
// float32 scratch of tokens * heads * key_shares * (head_dim + 2) values.
MXB_API int mxb_flash_prefill_tcgen05(const void* q, const void* cache, void* out, const int* block_tables,
                                      int max_pages, const int* tile_request, const int* tile_start,
                                      const int* tile_length, const int* positions, int tokens, int tiles,
                                      int heads, int kv_heads, int head_dim, int page_tokens, int num_pages,
                                      int window, float scale, int dtype, int key_shares, float* partial,
                                      int* status, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (key_shares < 1 || key_shares > kMergeShares || (key_shares > 1 && partial == nullptr))
    return static_cast<int>(cudaErrorInvalidValue);
  if (!mxb_flash_prefill_tcgen05_supported(head_dim, heads, kv_heads, page_tokens, dtype))
    return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(cache) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return static_cast<int>(cudaErrorInvalidValue);
  if (head_dim == 64)
    return launch_flash_tc<64>(q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length,
                               positions, tokens, tiles, heads, kv_heads, page_tokens, num_pages, window, scale,
                               key_shares, partial, status, stream);
  return launch_flash_tc<128>(q, cache, out, block_tables, max_pages, tile_request, tile_start, tile_length,
                              positions, tokens, tiles, heads, kv_heads, page_tokens, num_pages, window, scale,
                              key_shares, partial, status, stream);
}
