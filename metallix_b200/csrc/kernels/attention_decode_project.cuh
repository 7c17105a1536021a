// The end of a decode step's attention and the output projection in one
// kernel: the partial results of the splits are put together (as the merge
// kernel does, value for value) and multiplied by W_o at once, head by head.
//
// Block (c, h) takes head h and 128 columns of the output: its slice of W_o,
// [128 rows, head_dim values] of 32 KB, is on its way (one bulk copy per row)
// before the block waits for the attention kernel. Behind the wait a warp per
// token merges the head's partial results into a [tokens, head_dim] tile of
// bfloat16 in shared memory; eight warps multiply it by the slice
// (mma.sync m16n8k16, W as the 16-row operand) and the block writes
// summands[h, token, 128 columns] in float32. The sum over the heads, which is
// the sum over k of the projection, is taken in the order of the heads by the
// residual-sum-and-norm kernel that follows, which has to read a row anyway:
// one kernel and one hand-over less per layer than merge, projection, sum.
// The reference projects the concatenated heads with one matrix product
// (crates/models/qwen/src/forward.rs:1871-1876); the sum is the same.
#pragma once

#include "async_copy.cuh"
#include "common.cuh"

namespace mxb {

constexpr int kProjectColumns = 128;  // output columns (rows of W_o) per block
constexpr int kProjectThreads = 256;

// MB: blocks of eight tokens (tokens <= 8 * MB). split_keys: keys per split.
template <int HD, int MB>
__global__ void __launch_bounds__(kProjectThreads)
decode_merge_project_kernel(const float* __restrict__ partial, const __nv_bfloat16* __restrict__ w, long long ldw,
                            float* __restrict__ summands, const int* __restrict__ row_token,
                            const int* __restrict__ positions, int rows, int tokens, int heads, int hidden,
                            int max_splits, int window, int slots, int split_keys, float minus_huge, int* status) {
  constexpr int PITCH = HD * 2 + 16;  // bytes per row of a tile: rows a warp reads together fall on all banks
  constexpr int X_ROWS = MB * 8;
  extern __shared__ __align__(128) unsigned char project_shared[];
  unsigned char* s_w = project_shared;                                   // [128 columns][PITCH]
  unsigned char* s_x = s_w + kProjectColumns * PITCH;                    // [X_ROWS][PITCH]
  float (*s_out)[kProjectColumns + 1] = reinterpret_cast<float (*)[kProjectColumns + 1]>(s_x + X_ROWS * PITCH);
  __shared__ __align__(8) uint64_t barrier;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.y, n0 = blockIdx.x * kProjectColumns;

  chain_release();
  if (tid == 0) {
    barrier_init(&barrier, kProjectColumns);
    barrier_init_fence();
  }
  for (int i = tid; i < X_ROWS * PITCH / 4; i += kProjectThreads) reinterpret_cast<uint32_t*>(s_x)[i] = 0u;
  __syncthreads();
  if (tid < kProjectColumns) {
    if (n0 + tid < hidden) {
      barrier_arrive_expect(&barrier, HD * 2);
      bulk_copy(s_w + tid * PITCH, w + static_cast<long long>(n0 + tid) * ldw + head * HD, HD * 2, &barrier);
    } else {
      barrier_arrive(&barrier);  // a row past the matrix: its results are not stored
    }
  }
  // The step's integers are written by no kernel of the step: a warp's tokens
  // (one, or two with more than eight rows) and their splits are known before
  // the wait for the attention kernel.
  constexpr int TURNS = MB;             // rows warp, warp + 8
  constexpr int kChunk = 32;            // splits put together at once, as in the merge kernel
  const int stride = HD + 2;
  int turn_token[TURNS], turn_splits[TURNS];
  size_t turn_base[TURNS];
#pragma unroll
  for (int turn = 0; turn < TURNS; ++turn) {
    const int row = warp + turn * (kProjectThreads / 32);
    turn_token[turn] = -1;
    turn_splits[turn] = 0;
    turn_base[turn] = 0;
    if (row >= rows) continue;
    const int token = row_token[row];
    if (token < 0 || token >= X_ROWS) continue;
    const int pos = positions[token];
    const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
    const int first_split = first_key / split_keys, last_split = pos / split_keys;
    if (last_split >= max_splits) {
      if (lane == 0) atomicOr(status, kStatusBadSlot);
      continue;
    }
    turn_token[turn] = token;
    turn_splits[turn] = slots > 0 ? min(slots, last_split - first_split + 1) : last_split - first_split + 1;
    turn_base[turn] = (slots > 0 ? (static_cast<size_t>(row) * heads + head) * slots
                                 : (static_cast<size_t>(row) * heads + head) * max_splits + first_split) * stride;
  }
  chain_wait();
  partial = behind_wait(partial);  // written by the attention kernel ahead of this one

  // ---- merge: the same sums in the same order as paged_attention_merge_kernel
#pragma unroll
  for (int turn = 0; turn < TURNS; ++turn) {
    const int token = turn_token[turn], splits = turn_splits[turn];
    if (token < 0) continue;
    const float* base = partial + turn_base[turn];
    float m = minus_huge, l = 0.0f;
    float2 acc[HD / 64];
#pragma unroll
    for (int h = 0; h < HD / 64; ++h) acc[h] = make_float2(0.0f, 0.0f);
    for (int chunk = 0; chunk < splits; chunk += kChunk) {
      const int live = min(kChunk, splits - chunk);
      float mine = minus_huge, mine_sum = 0.0f;
      if (lane < live) {
        const float2 stats = *reinterpret_cast<const float2*>(base + static_cast<size_t>(chunk + lane) * stride + HD);
        mine = stats.x;
        mine_sum = stats.y;
      }
      constexpr int kBatch = 8;
      float2 values[kBatch][HD / 64], ahead[kBatch][HD / 64];
      auto fetch = [&](float2 (&into)[kBatch][HD / 64], int from) {
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const float* p = base + static_cast<size_t>(chunk + (from + j < live ? from + j : 0)) * stride + lane * 2;
#pragma unroll
          for (int h = 0; h < HD / 64; ++h)
            into[j][h] = from + j < live ? *reinterpret_cast<const float2*>(p + h * 64) : make_float2(0.0f, 0.0f);
        }
      };
      fetch(values, 0);
      const float round_max = fmaxf(m, warp_max(mine));
      const float carry = expf(m - round_max);  // what earlier rounds gathered, on the new maximum
      l *= carry;
#pragma unroll
      for (int h = 0; h < HD / 64; ++h) {
        acc[h].x *= carry;
        acc[h].y *= carry;
      }
      const float mine_weight = expf(mine - round_max);   // 0 for a lane without a split
      // The values come in batches of eight splits, the next batch's loads on
      // their way while this batch is added up (two batches of registers: a
      // block must stay small enough that the blocks of the kernels behind it,
      // which fetch their weights early, find room on the SM beside it).
#pragma unroll 1
      for (int from = 0; from < live; from += kBatch) {
        const bool more = from + kBatch < live;
        if (more) fetch(ahead, from + kBatch);
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
          const float weight = __shfl_sync(0xffffffffu, mine_weight, (from + j) & 31);
          const float sum = __shfl_sync(0xffffffffu, mine_sum, (from + j) & 31);
#pragma unroll
          for (int h = 0; h < HD / 64; ++h) {
            acc[h].x = fmaf(weight, values[j][h].x, acc[h].x);
            acc[h].y = fmaf(weight, values[j][h].y, acc[h].y);
          }
          l = fmaf(weight, sum, l);
        }
        if (more) {
#pragma unroll
          for (int j = 0; j < kBatch; ++j)
#pragma unroll
            for (int h = 0; h < HD / 64; ++h) values[j][h] = ahead[j][h];
        }
      }
      m = round_max;
    }
#pragma unroll
    for (int h = 0; h < HD / 64; ++h)
      *reinterpret_cast<__nv_bfloat162*>(s_x + token * PITCH + (h * 64 + lane * 2) * 2) =
          __floats2bfloat162_rn(acc[h].x / l, acc[h].y / l);
  }
  __syncthreads();
  const bool landed = barrier_wait(&barrier, 0, status);

  // ---- project: warp w takes rows 16w .. 16w + 15 of the slice
  const int g = lane >> 2, t = lane & 3;
  float d[MB][4];
#pragma unroll
  for (int j = 0; j < MB; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.0f;
  const unsigned char* w_lo = s_w + (warp * 16 + g) * PITCH + t * 4;
  const unsigned char* x_lo = s_x + g * PITCH + t * 4;
#pragma unroll
  for (int step = 0; step < HD / 16; ++step) {
    const int offset = step * 32;  // bytes along a row
    const uint32_t a0 = *reinterpret_cast<const uint32_t*>(w_lo + offset);
    const uint32_t a1 = *reinterpret_cast<const uint32_t*>(w_lo + 8 * PITCH + offset);
    const uint32_t a2 = *reinterpret_cast<const uint32_t*>(w_lo + offset + 16);
    const uint32_t a3 = *reinterpret_cast<const uint32_t*>(w_lo + 8 * PITCH + offset + 16);
#pragma unroll
    for (int j = 0; j < MB; ++j) {
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(x_lo + j * 8 * PITCH + offset);
      const uint32_t b1 = *reinterpret_cast<const uint32_t*>(x_lo + j * 8 * PITCH + offset + 16);
      asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
                   : "+f"(d[j][0]), "+f"(d[j][1]), "+f"(d[j][2]), "+f"(d[j][3])
                   : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
  }
  // d0, d1: row g of W (a column of the output), tokens 8j + 2t and + 1; d2, d3: row g + 8.
#pragma unroll
  for (int j = 0; j < MB; ++j) {
    s_out[j * 8 + 2 * t][warp * 16 + g] = d[j][0];
    s_out[j * 8 + 2 * t + 1][warp * 16 + g] = d[j][1];
    s_out[j * 8 + 2 * t][warp * 16 + g + 8] = d[j][2];
    s_out[j * 8 + 2 * t + 1][warp * 16 + g + 8] = d[j][3];
  }
  __syncthreads();
  if (!landed) return;  // the status word says so; nothing is written from a tile that never came
  for (int i = tid; i < tokens * kProjectColumns; i += kProjectThreads) {
    const int token = i / kProjectColumns, column = i - token * kProjectColumns;
    if (n0 + column < hidden)
      summands[(static_cast<size_t>(head) * tokens + token) * hidden + n0 + column] = s_out[token][column];
  }
}

constexpr int kProjectTokens = 64;  // the most tokens of a step the kernel takes

// Whether the kernel takes this projection: bfloat16 heads of 64 or 128
// values, up to 64 tokens, rows of W_o that the bulk copies can fetch.
static bool decode_project_takes(int head_dim, int tokens, const void* w, long long ldw) {
  return (head_dim == 64 || head_dim == 128) && tokens >= 1 && tokens <= kProjectTokens &&
         reinterpret_cast<uintptr_t>(w) % 16 == 0 && (ldw * 2) % 16 == 0;
}

template <int HD>
static cudaError_t launch_merge_project(const float* partial, const __nv_bfloat16* w, long long ldw, float* summands,
                                        const int* row_token, const int* positions, int rows, int tokens, int heads,
                                        int hidden, int max_splits, int window, int slots, int split_keys,
                                        float minus_huge, int* status, cudaStream_t stream) {
  const dim3 grid((hidden + kProjectColumns - 1) / kProjectColumns, heads);
#define GO(MB)                                                                                                       \
  {                                                                                                                  \
    auto kernel = decode_merge_project_kernel<HD, MB>;                                                               \
    const int shared = (kProjectColumns + MB * 8) * (HD * 2 + 16) + MB * 8 * (kProjectColumns + 1) * 4;              \
    if (shared > 48 * 1024) {                                                                                        \
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);             \
      if (e != cudaSuccess) return e;                                                                                \
    }                                                                                                                \
    return launch_chained(kernel, grid, dim3(kProjectThreads), shared, stream, partial, w, ldw, summands, row_token,  \
                          positions, rows, tokens, heads, hidden, max_splits, window, slots, split_keys, minus_huge,  \
                          status);                                                                                   \
  }
  if (tokens <= 8) GO(1)
  if (tokens <= 16) GO(2)
  if (tokens <= 32) GO(4)
  GO(8)
#undef GO
}

}  // namespace mxb
