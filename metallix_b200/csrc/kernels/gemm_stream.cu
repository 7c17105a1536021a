// out[M, N] = x[M, K] * W[N, K]^T for the few rows of a decode step (M <= 16),
// bfloat16 in, float32 accumulate, with the copy engine doing the streaming.
//
// A block owns R rows of W (R output columns) over the whole K. One thread
// per row issues a single bulk copy (cp.async.bulk) of that row into shared
// memory before the block waits for the kernel ahead of it: the weights are
// never written by a kernel, so the whole of W is in flight while the
// producer of x is still running, and a row of any length costs one
// instruction instead of one 16-byte load per lane per 32 values of k (whose
// number in flight per SM is what bounded the load-based kernel at larger k).
// After the wait the rows of x arrive the same way; the eight warps take
// interleaved 16-wide steps of k from shared memory into mma.sync m16n8k16
// (W as the 16-row operand, x as the 8-column operand) and their partial sums
// are added in warp order, so an output element sees one order of additions
// whatever M is. Rows of both tiles are 16 bytes longer than k values, which
// spreads the rows a warp reads together over all banks.
//
// Optional epilogue: W holds gate rows then up rows (2 * inter rows); the block
// computes both for its R columns and writes silu(gate) * up (float32 inside),
// which the reference does as three element-wise passes
// (crates/models/qwen/src/forward.rs:1913-1917).
//
// Every wait on a barrier is bounded: if one runs out, the status word gets a
// bit and the block writes nothing.
#include "async_copy.cuh"
#include "common.cuh"

namespace mxb {

constexpr int kStreamWarps = 8;
constexpr int kStreamThreads = kStreamWarps * 32;
constexpr int kStreamSharedLimit = 200 * 1024;

__device__ __forceinline__ void stream_mma(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                           uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TOut> __device__ __forceinline__ void stream_store(TOut* p, float v) { *p = from_float<TOut>(v); }

// MB: 8-row blocks of x (M <= 8 * MB). R: rows of W per block and set, 8 or
// 16. SWIGLU: two sets of rows (gate, up) per block.
template <int MB, bool SWIGLU, typename TOut, int R>
__global__ void __launch_bounds__(kStreamThreads)
gemm_stream_kernel(TOut* __restrict__ out, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   int m, int n, int k, long long ldx, long long ldw, long long ldo, int inter, int* status) {
  constexpr int SETS = SWIGLU ? 2 : 1;
  constexpr int W_ROWS = SETS * R, X_ROWS = MB * 8;
  extern __shared__ __align__(128) unsigned char stream_shared[];
  __shared__ __align__(8) uint64_t barriers[2];  // the rows of W, the rows of x
  __shared__ float s_part[kStreamWarps][R][X_ROWS + 1];
  const int pitch = k * 2 + 16;  // bytes per row of a tile
  unsigned char* s_w = stream_shared;
  unsigned char* s_x = s_w + static_cast<size_t>(W_ROWS) * pitch;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int columns = SWIGLU ? inter : n;
  const int n0 = blockIdx.x * R;

  chain_release();
  if (tid == 0) {
    barrier_init(&barriers[0], W_ROWS);
    barrier_init(&barriers[1], X_ROWS);
    barrier_init_fence();
  }
  __syncthreads();
  if (tid < W_ROWS) {
    const int set = tid / R, r = tid - set * R;
    if (n0 + r < columns) {
      barrier_arrive_expect(&barriers[0], static_cast<uint32_t>(k) * 2);
      bulk_copy(s_w + static_cast<size_t>(tid) * pitch, w + (static_cast<long long>(set) * inter + n0 + r) * ldw,
                static_cast<uint32_t>(k) * 2, &barriers[0]);
    } else {
      barrier_arrive(&barriers[0]);  // a row past the matrix: its results are not stored
    }
  }
  chain_wait();
  if (tid < X_ROWS) {
    if (tid < m) {
      barrier_arrive_expect(&barriers[1], static_cast<uint32_t>(k) * 2);
      bulk_copy(s_x + static_cast<size_t>(tid) * pitch, x + static_cast<long long>(tid) * ldx,
                static_cast<uint32_t>(k) * 2, &barriers[1]);
    } else {
      barrier_arrive(&barriers[1]);
    }
  }
  const bool landed = barrier_wait(&barriers[0], 0, status) && barrier_wait(&barriers[1], 0, status);

  float acc[SETS][MB][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int j = 0; j < MB; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.0f;
  const int steps = k / 16;
  const unsigned char* w_lo = s_w + static_cast<size_t>(g) * pitch + t * 4;
  const unsigned char* x_lo = s_x + static_cast<size_t>(g) * pitch + t * 4;
#pragma unroll 4
  for (int step = warp; step < steps; step += kStreamWarps) {
    const int offset = step * 32;  // bytes along a row
    uint32_t b0[MB], b1[MB];
#pragma unroll
    for (int j = 0; j < MB; ++j) {
      const unsigned char* row = x_lo + static_cast<size_t>(j) * 8 * pitch + offset;
      b0[j] = *reinterpret_cast<const uint32_t*>(row);
      b1[j] = *reinterpret_cast<const uint32_t*>(row + 16);
    }
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
      const unsigned char* row = w_lo + static_cast<size_t>(s) * R * pitch + offset;
      const uint32_t a0 = *reinterpret_cast<const uint32_t*>(row);
      const uint32_t a2 = *reinterpret_cast<const uint32_t*>(row + 16);
      uint32_t a1 = 0u, a3 = 0u;
      if (R == 16) {
        a1 = *reinterpret_cast<const uint32_t*>(row + static_cast<size_t>(8) * pitch);
        a3 = *reinterpret_cast<const uint32_t*>(row + static_cast<size_t>(8) * pitch + 16);
      }
#pragma unroll
      for (int j = 0; j < MB; ++j) stream_mma(acc[s][j], a0, a1, a2, a3, b0[j], b1[j]);
    }
  }
  // c0, c1: W row g, x rows 8j + 2t, 8j + 2t + 1; c2, c3: W row g + 8.
  constexpr int ITEMS = (R * X_ROWS + kStreamThreads - 1) / kStreamThreads;
  float sums[SETS][ITEMS];
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
    if (s > 0) __syncthreads();  // the previous set has been summed
#pragma unroll
    for (int j = 0; j < MB; ++j) {
      s_part[warp][g][j * 8 + 2 * t] = acc[s][j][0];
      s_part[warp][g][j * 8 + 2 * t + 1] = acc[s][j][1];
      if (R == 16) {
        s_part[warp][g + 8][j * 8 + 2 * t] = acc[s][j][2];
        s_part[warp][g + 8][j * 8 + 2 * t + 1] = acc[s][j][3];
      }
    }
    __syncthreads();
#pragma unroll
    for (int item = 0; item < ITEMS; ++item) {
      const int i = tid + item * kStreamThreads;
      const int r = i % R, row_m = i / R;
      float sum = 0.0f;
      if (row_m < X_ROWS) {
#pragma unroll
        for (int wp = 0; wp < kStreamWarps; ++wp) sum += s_part[wp][r][row_m];  // warp order: one order of additions
      }
      sums[s][item] = sum;
    }
  }
  if (!landed) return;  // the status word says why
#pragma unroll
  for (int item = 0; item < ITEMS; ++item) {
    const int i = tid + item * kStreamThreads;
    const int r = i % R, row_m = i / R;  // consecutive threads: consecutive columns
    const int column = n0 + r;
    if (row_m >= m || column >= columns) continue;
    float value = sums[0][item];
    if (SWIGLU) {
      // The library path rounds gate and up to bfloat16 before the activation;
      // keep the same rounding points so both paths agree.
      const float gate = to_float(from_float<__nv_bfloat16>(sums[0][item]));
      const float up = to_float(from_float<__nv_bfloat16>(sums[SETS - 1][item]));
      value = __fdividef(gate, 1.0f + __expf(-gate)) * up;  // the result is rounded to bfloat16 anyway
    }
    stream_store(out + static_cast<long long>(row_m) * ldo + column, value);
  }
}

static size_t stream_shared_bytes(int m_rows, int w_rows, int k) {
  return static_cast<size_t>(m_rows + w_rows) * (static_cast<size_t>(k) * 2 + 16);
}

template <int MB, bool SWIGLU, typename TOut, int R>
static int launch_stream_rows(void* out, const void* x, const void* w, int m, int n, int k, long long ldx,
                              long long ldw, long long ldo, int inter, int* status, cudaStream_t stream) {
  const int columns = SWIGLU ? inter : n;
  const size_t shared = stream_shared_bytes(MB * 8, (SWIGLU ? 2 : 1) * R, k);
  auto kernel = gemm_stream_kernel<MB, SWIGLU, TOut, R>;
  if (shared > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  return static_cast<int>(launch_chained_sized(static_cast<unsigned long long>(n) * k * 2, kernel,
                                               dim3((columns + R - 1) / R), dim3(kStreamThreads), shared, stream,
                                         static_cast<TOut*>(out), static_cast<const __nv_bfloat16*>(x),
                                         static_cast<const __nv_bfloat16*>(w), m, n, k, ldx, ldw, ldo, inter, status));
}

// Rows of W per block: 16 where that still leaves about two blocks per SM
// and fits shared memory, else 8.
static int stream_rows(int m_rows, int columns, int k, bool swiglu) {
  const int sets = swiglu ? 2 : 1;
  if (columns >= 4096 && stream_shared_bytes(m_rows, sets * 16, k) <= static_cast<size_t>(kStreamSharedLimit)) return 16;
  if (stream_shared_bytes(m_rows, sets * 8, k) <= static_cast<size_t>(kStreamSharedLimit)) return 8;
  return 0;
}

template <int MB, bool SWIGLU>
static int launch_stream(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                         long long ldx, long long ldw, long long ldo, int inter, int* status, cudaStream_t stream) {
  const int rows = stream_rows(MB * 8, SWIGLU ? inter : n, k, SWIGLU);
#define GO(TOUT, R) return launch_stream_rows<MB, SWIGLU, TOUT, R>(out, x, w, m, n, k, ldx, ldw, ldo, inter, status, stream)
  if (out_dtype == kBF16) { if (rows == 16) GO(__nv_bfloat16, 16); else GO(__nv_bfloat16, 8); }
  else { if (rows == 16) GO(float, 16); else GO(float, 8); }
#undef GO
}

}  // namespace mxb

using namespace mxb;

// Shapes the kernel takes: 1 <= m <= 16, k a multiple of 16, rows of x and W
// starting on 16-byte boundaries, and a block's rows of W and x fitting
// shared memory (200 KiB: k up to about 6,000 with 16 rows of x).
MXB_API int mxb_gemm_stream_supported(int m, int n, int k, long long ldx, long long ldw, int swiglu_inter) {
  if (m < 1 || m > 16 || n < 1 || k < 16 || k % 16 != 0 || ldx % 8 != 0 || ldw % 8 != 0) return 0;
  if (swiglu_inter != 0 && n != 2 * swiglu_inter) return 0;
  return stream_rows(m <= 8 ? 8 : 16, swiglu_inter ? swiglu_inter : n, k, swiglu_inter != 0) != 0 ? 1 : 0;
}

// swiglu_inter == 0: out[m, n] = x w^T. swiglu_inter == inter > 0: w is
// [2 * inter, k] (gate rows, then up rows), out is [m, inter].
MXB_API int mxb_gemm_stream(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                            long long ldx, long long ldw, long long ldo, int swiglu_inter, int* status,
                            cudaStream_t stream) {
  if (!mxb_gemm_stream_supported(m, n, k, ldx, ldw, swiglu_inter)) return static_cast<int>(cudaErrorInvalidValue);
  if (out_dtype != kBF16 && out_dtype != kF32) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return static_cast<int>(cudaErrorInvalidValue);
#define LAUNCH(MB)                                                                                                \
  return swiglu_inter ? launch_stream<MB, true>(out, out_dtype, x, w, m, n, k, ldx, ldw, ldo, swiglu_inter, status, stream) \
                      : launch_stream<MB, false>(out, out_dtype, x, w, m, n, k, ldx, ldw, ldo, 0, status, stream)
  if (m <= 8) { LAUNCH(1); }
  LAUNCH(2);
#undef LAUNCH
}

MXB_TIMELINE_EXPORT(mxb_timeline_gemm_stream)
