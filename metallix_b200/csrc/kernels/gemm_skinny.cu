// out[M, N] = x[M, K] * W[N, K]^T for the few rows of a decode step (M <= 64),
// bfloat16 in, float32 accumulate: a weight-streaming kernel.
//
// With a handful of rows the product is bound by reading W once, so the
// kernel is laid out around that read: one block owns 16 rows of W (16 output
// columns) over the whole K, its eight warps take interleaved 32-wide slices
// of K, and every lane fetches 16 contiguous bytes of W per row straight into
// the registers of a tensor-core operand (mma.sync m16n8k16 with W as the
// 16-row operand and x as the 8-column operand), several slices in flight at
// once. The permutation of k inside a 32-wide slice that this direct load
// implies is applied to both operands, so the dot product is unchanged. x is
// small and read through L2. The warps' partial sums are added in warp order,
// so an output element sees one order of additions whatever M is.
//
// Optional epilogue: W holds gate rows then up rows (2 * inter rows); the block
// computes both for its 16 columns and writes silu(gate) * up (float32 inside),
// which the reference does as three element-wise passes
// (crates/models/qwen/src/forward.rs:1913-1917).
#include "common.cuh"

namespace mxb {

constexpr int kSkinnyWarps = 8;
constexpr int kSkinnyThreads = kSkinnyWarps * 32;
constexpr int kSkinnyRows = 16;   // rows of W per block (8 for narrow outputs)
static_assert(kSkinnyRows == 16, "the tensor-core tile has 16 rows");
constexpr int kSkinnySlice = 32;  // k per warp iteration

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TOut> __device__ __forceinline__ void store_out(TOut* p, float v) { *p = from_float<TOut>(v); }

// MB: 8-row blocks of x (M <= 8 * MB). SWIGLU: gate/up pairs, see above.
// WROWS: rows of W per block, 16 or 8. With 8 the upper half of the 16-row
// operand is zero; narrow matrices then still spread over enough blocks to
// keep every SM reading.
template <int MB, bool SWIGLU, typename TOut, int WROWS>
__global__ void __launch_bounds__(kSkinnyThreads)
gemm_skinny_kernel(TOut* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, int m, int n, int k, long long ldx, long long ldw,
                   long long ldo, int inter) {
  constexpr int SETS = SWIGLU ? 2 : 1;
  __shared__ float s_part[kSkinnyWarps][WROWS][MB * 8 + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * WROWS;
  const int columns = SWIGLU ? inter : n;  // output columns
  // Rows of W this lane reads (clamped; rows beyond the end are masked at the store).
  const int row_lo = min(n0 + g, columns - 1), row_hi = min(n0 + g + 8, columns - 1);
  const __nv_bfloat16* w_lo[SETS];
  const __nv_bfloat16* w_hi[SETS];
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
    w_lo[s] = w + (static_cast<long long>(s) * inter + row_lo) * ldw + t * 8;
    w_hi[s] = w + (static_cast<long long>(s) * inter + row_hi) * ldw + t * 8;
  }
  const __nv_bfloat16* x_row[MB];
  bool x_ok[MB];
#pragma unroll
  for (int j = 0; j < MB; ++j) {
    x_ok[j] = j * 8 + g < m;
    x_row[j] = x + static_cast<long long>(x_ok[j] ? j * 8 + g : 0) * ldx + t * 8;
  }
  float acc[SETS][MB][4];
#pragma unroll
  for (int s = 0; s < SETS; ++s)
#pragma unroll
    for (int j = 0; j < MB; ++j) acc[s][j][0] = acc[s][j][1] = acc[s][j][2] = acc[s][j][3] = 0.0f;

  const int slices = k / kSkinnySlice;
  // The weights are never written by a kernel, so this warp's first slices of
  // W are fetched before waiting for the kernel that produces x.
  // Narrow blocks read one row of W per lane and have registers to spare:
  // they fetch up to 12 slices ahead (a k of 3072 is then wholly in flight).
  constexpr int PRE = MB <= 2 ? (WROWS == 8 && !SWIGLU ? 12 : 4) : 0;
  uint4 pre_lo[PRE > 0 ? PRE : 1][SETS], pre_hi[PRE > 0 ? PRE : 1][SETS];
  // A small product lets its successor start at once (it fetches weights
  // ahead); a large one only when this block is nearly done, so that the
  // successor's blocks, resident and waiting, do not take the places that
  // this kernel's later blocks need.
  const bool release_late = static_cast<long long>(n) * k > (12ll << 20);
  if (!release_late) chain_release();
#pragma unroll
  for (int i = 0; i < PRE; ++i) {
    const int slice = warp + i * kSkinnyWarps;
    if (slice < slices) {
#pragma unroll
      for (int s = 0; s < SETS; ++s) {
        pre_lo[i][s] = __ldg(reinterpret_cast<const uint4*>(w_lo[s] + slice * kSkinnySlice));
        pre_hi[i][s] = WROWS == 16 ? __ldg(reinterpret_cast<const uint4*>(w_hi[s] + slice * kSkinnySlice))
                                   : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
  chain_wait();
#pragma unroll
  for (int j = 0; j < MB; ++j) x_row[j] = behind_wait(x_row[j]);  // x is written by the kernel ahead
#pragma unroll
  for (int i = 0; i < PRE; ++i) {
    const int slice = warp + i * kSkinnyWarps;
    if (slice < slices) {
      const int k0 = slice * kSkinnySlice;
      uint4 b[MB];
#pragma unroll
      for (int j = 0; j < MB; ++j)
        b[j] = x_ok[j] ? *reinterpret_cast<const uint4*>(x_row[j] + k0) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int s = 0; s < SETS; ++s)
#pragma unroll
        for (int j = 0; j < MB; ++j) {
          mma_16816(acc[s][j], pre_lo[i][s].x, pre_hi[i][s].x, pre_lo[i][s].y, pre_hi[i][s].y, b[j].x, b[j].y);
          mma_16816(acc[s][j], pre_lo[i][s].z, pre_hi[i][s].z, pre_lo[i][s].w, pre_hi[i][s].w, b[j].z, b[j].w);
        }
    }
  }
#pragma unroll 4
  for (int slice = warp + PRE * kSkinnyWarps; slice < slices; slice += kSkinnyWarps) {
    const int k0 = slice * kSkinnySlice;
    uint4 a_lo[SETS], a_hi[SETS];
#pragma unroll
    for (int s = 0; s < SETS; ++s) {
      a_lo[s] = __ldg(reinterpret_cast<const uint4*>(w_lo[s] + k0));
      a_hi[s] = WROWS == 16 ? __ldg(reinterpret_cast<const uint4*>(w_hi[s] + k0)) : make_uint4(0u, 0u, 0u, 0u);
    }
    uint4 b[MB];
#pragma unroll
    for (int j = 0; j < MB; ++j)
      b[j] = x_ok[j] ? *reinterpret_cast<const uint4*>(x_row[j] + k0) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int s = 0; s < SETS; ++s)
#pragma unroll
      for (int j = 0; j < MB; ++j) {
        mma_16816(acc[s][j], a_lo[s].x, a_hi[s].x, a_lo[s].y, a_hi[s].y, b[j].x, b[j].y);
        mma_16816(acc[s][j], a_lo[s].z, a_hi[s].z, a_lo[s].w, a_hi[s].w, b[j].z, b[j].w);
      }
  }
  if (release_late) chain_release();
  // c0, c1: W row g, x rows 8j + 2t, 8j + 2t + 1; c2, c3: W row g + 8.
  constexpr int ITEMS = (WROWS * MB * 8 + kSkinnyThreads - 1) / kSkinnyThreads;
  float sums[SETS][ITEMS];
#pragma unroll
  for (int s = 0; s < SETS; ++s) {
    if (s > 0) __syncthreads();  // the previous set has been summed
#pragma unroll
    for (int j = 0; j < MB; ++j) {
      s_part[warp][g][j * 8 + 2 * t] = acc[s][j][0];
      s_part[warp][g][j * 8 + 2 * t + 1] = acc[s][j][1];
      if (WROWS == 16) {
        s_part[warp][g + 8][j * 8 + 2 * t] = acc[s][j][2];
        s_part[warp][g + 8][j * 8 + 2 * t + 1] = acc[s][j][3];
      }
    }
    __syncthreads();
#pragma unroll
    for (int item = 0; item < ITEMS; ++item) {
      const int i = tid + item * kSkinnyThreads;
      const int r = i % WROWS, row_m = i / WROWS;
      float sum = 0.0f;
      if (row_m < MB * 8) {
#pragma unroll
        for (int wp = 0; wp < kSkinnyWarps; ++wp) sum += s_part[wp][r][row_m];  // warp order: one order of additions
      }
      sums[s][item] = sum;
    }
  }
#pragma unroll
  for (int item = 0; item < ITEMS; ++item) {
    const int i = tid + item * kSkinnyThreads;
    const int r = i % WROWS, row_m = i / WROWS;  // consecutive threads: consecutive columns
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
    store_out(out + static_cast<long long>(row_m) * ldo + column, value);
  }
}

template <int MB, bool SWIGLU>
static int launch_skinny(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                         long long ldx, long long ldw, long long ldo, int inter, cudaStream_t stream) {
  const int columns = SWIGLU ? inter : n;
  // Narrow outputs take 8 rows of W per block so that at least ~2 blocks per SM exist.
  const bool narrow = columns <= 2048;
  dim3 grid((columns + (narrow ? 8 : 16) - 1) / (narrow ? 8 : 16));
  const unsigned long long streamed = static_cast<unsigned long long>(n) * k * 2;   // the bytes of W
#define GO(TOUT, WROWS) return static_cast<int>(launch_chained_sized(streamed, gemm_skinny_kernel<MB, SWIGLU, TOUT, WROWS>, grid, \
      dim3(kSkinnyThreads), 0, stream, static_cast<TOUT*>(out), static_cast<const __nv_bfloat16*>(x), \
      static_cast<const __nv_bfloat16*>(w), m, n, k, ldx, ldw, ldo, inter))
  if (out_dtype == kBF16) { if (narrow) GO(__nv_bfloat16, 8); else GO(__nv_bfloat16, 16); }
  else { if (narrow) GO(float, 8); else GO(float, 16); }
#undef GO
}

}  // namespace mxb

using namespace mxb;

// Shapes the kernel takes: 1 <= m <= 64, k a multiple of 32, rows of x and W
// starting on 16-byte boundaries.
MXB_API int mxb_gemm_skinny_supported(int m, int n, int k, long long ldx, long long ldw) {
  return m >= 1 && m <= 64 && n >= 1 && k >= 32 && k % 32 == 0 && ldx % 8 == 0 && ldw % 8 == 0 ? 1 : 0;
}

// swiglu_inter == 0: out[m, n] = x w^T. swiglu_inter == inter > 0: w is
// [2 * inter, k] (gate rows, then up rows), out is [m, inter].
MXB_API int mxb_gemm_skinny(void* out, int out_dtype, const void* x, const void* w, int m, int n, int k,
                            long long ldx, long long ldw, long long ldo, int swiglu_inter,
                            cudaStream_t stream) {
  if (!mxb_gemm_skinny_supported(m, n, k, ldx, ldw)) return static_cast<int>(cudaErrorInvalidValue);
  if (out_dtype != kBF16 && out_dtype != kF32) return static_cast<int>(cudaErrorInvalidValue);
  if (swiglu_inter != 0 && n != 2 * swiglu_inter) return static_cast<int>(cudaErrorInvalidValue);
#define LAUNCH(MB)                                                                                      \
  return swiglu_inter ? launch_skinny<MB, true>(out, out_dtype, x, w, m, n, k, ldx, ldw, ldo, swiglu_inter, stream) \
                      : launch_skinny<MB, false>(out, out_dtype, x, w, m, n, k, ldx, ldw, ldo, 0, stream)
  if (m <= 8) { LAUNCH(1); }
  if (m <= 16) { LAUNCH(2); }
  if (m <= 32) { LAUNCH(4); }
  LAUNCH(8);
#undef LAUNCH
}

MXB_TIMELINE_EXPORT(mxb_timeline_gemm_load)
