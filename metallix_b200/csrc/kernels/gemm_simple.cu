// C[M, N] = A[M, K] * W[N, K]^T on CUDA cores with float32 accumulation.
//
// This is the true 32-bit matrix product of the float32 path (tensor cores
// have no full-float32 input mode) and the plain twin of the tensor-core
// kernels. Every output element sums its K products in ascending k, in the
// same order whatever M is, so a row's result does not depend on what else is
// in the batch. W is [out, in] row-major and applied as x W^T, as in the
// reference's projection (crates/models/qwen/src/forward/projection.rs:257-265).
#include "common.cuh"

namespace mxb {

constexpr int kGemmTile = 64;   // rows and columns of C per block
constexpr int kGemmK = 16;      // k per shared-memory stage

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(256)
gemm_simple_kernel(TOut* __restrict__ c, const TIn* __restrict__ a, const TIn* __restrict__ w,
                   int m, int n, int k, long long lda, long long ldw, long long ldc) {
  __shared__ float sA[kGemmK][kGemmTile + 4];
  __shared__ float sW[kGemmK][kGemmTile + 4];
  const int tid = threadIdx.x;
  const int row0 = blockIdx.y * kGemmTile, col0 = blockIdx.x * kGemmTile;
  const int ty = tid / 16, tx = tid % 16;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int k0 = 0; k0 < k; k0 += kGemmK) {
    // 64 x 16 elements of each operand, 4 per thread
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int rr = e / kGemmK, kk = e % kGemmK;
      const int gr = row0 + rr, gc = col0 + rr, gk = k0 + kk;
      sA[kk][rr] = (gr < m && gk < k) ? to_float(a[gr * lda + gk]) : 0.0f;
      sW[kk][rr] = (gc < n && gk < k) ? to_float(w[gc * ldw + gk]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kGemmK; ++kk) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = sA[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = sW[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gr = row0 + ty * 4 + i;
    if (gr >= m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gc = col0 + tx * 4 + j;
      if (gc < n) c[gr * ldc + gc] = from_float<TOut>(acc[i][j]);
    }
  }
}

// out[t, i] = silu(gate_up[t, i]) * gate_up[t, inter + i], float32 inside:
// sigmoid(g) * g * u as the reference writes it
// (crates/models/qwen/src/forward.rs:1913-1917).
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gate_up, int inter,
                                size_t count) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const size_t t = i / inter, col = i - t * inter;
  const float g = to_float(gate_up[t * 2 * inter + col]);
  const float u = to_float(gate_up[t * 2 * inter + inter + col]);
  const float sig = 1.0f / (1.0f + expf(-g));
  out[i] = from_float<T>(sig * g * u);
}

// Eight bfloat16 values per thread (16-byte loads and stores).
__global__ void silu_mul_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ gate_up,
                                       int inter, size_t groups) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= groups) return;
  const int per_row = inter / 8;
  const size_t t = i / per_row, col = (i - t * per_row) * 8;
  const uint4 g4 = *reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + col);
  const uint4 u4 = *reinterpret_cast<const uint4*>(gate_up + t * 2 * inter + inter + col);
  const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
  uint32_t ow[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
    const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
    const float r0 = (1.0f / (1.0f + expf(-g0))) * g0 * u0;
    const float r1 = (1.0f / (1.0f + expf(-g1))) * g1 * u1;
    __nv_bfloat162 packed = __floats2bfloat162_rn(r0, r1);
    ow[j] = *reinterpret_cast<uint32_t*>(&packed);
  }
  *reinterpret_cast<uint4*>(out + t * inter + col) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

}  // namespace mxb

using namespace mxb;

MXB_API int mxb_gemm_simple(void* c, int c_dtype, const void* a, const void* w, int in_dtype, int m,
                            int n, int k, long long lda, long long ldw, long long ldc,
                            cudaStream_t stream) {
  if (m <= 0 || n <= 0) return 0;
  dim3 grid(ceil_div(n, kGemmTile), ceil_div(m, kGemmTile));
#define LAUNCH(TI, TO) gemm_simple_kernel<TI, TO><<<grid, 256, 0, stream>>>( \
      static_cast<TO*>(c), static_cast<const TI*>(a), static_cast<const TI*>(w), m, n, k, lda, ldw, ldc)
  if (in_dtype == kF32 && c_dtype == kF32) LAUNCH(float, float);
  else if (in_dtype == kBF16 && c_dtype == kBF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (in_dtype == kBF16 && c_dtype == kF32) LAUNCH(__nv_bfloat16, float);
  else return static_cast<int>(cudaErrorInvalidValue);
#undef LAUNCH
  return static_cast<int>(cudaGetLastError());
}

MXB_API int mxb_silu_mul(void* out, const void* gate_up, int dtype, long long tokens, int inter,
                         cudaStream_t stream) {
  const size_t count = static_cast<size_t>(tokens) * inter;
  if (count == 0) return 0;
  if (dtype == kBF16 && inter % 8 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
      reinterpret_cast<uintptr_t>(gate_up) % 16 == 0) {
    const size_t groups = count / 8;
    silu_mul_bf16x8_kernel<<<static_cast<unsigned>((groups + 255) / 256), 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), inter, groups);
    return static_cast<int>(cudaGetLastError());
  }
  const unsigned blocks = static_cast<unsigned>((count + 255) / 256);
  if (dtype == kF32)
    silu_mul_kernel<float><<<blocks, 256, 0, stream>>>(static_cast<float*>(out), static_cast<const float*>(gate_up), inter, count);
  else if (dtype == kBF16)
    silu_mul_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(gate_up), inter, count);
  else
    return static_cast<int>(cudaErrorInvalidValue);
  return static_cast<int>(cudaGetLastError());
}
