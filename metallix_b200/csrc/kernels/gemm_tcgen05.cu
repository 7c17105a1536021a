// C[M, N] = A[M, K] * W[N, K]^T in bfloat16 on the fifth-generation tensor
// cores: tcgen05.mma issued by one thread, operands staged in shared memory by
// TMA (cp.async.bulk.tensor with the 128-byte swizzle), the float32
// accumulator of a 128 x BN tile in tensor memory, read back with tcgen05.ld
// for the epilogue.
//
// One block computes one 128 x BN tile. Warp 0 feeds the pipeline (one lane
// issues the TMA loads), warp 1 owns tensor memory and issues the MMAs, warps
// 2..5 run the epilogue: plain store (bfloat16 or float32), or SwiGLU, where
// the B tile is made of 128 gate rows and the 128 up rows of the same columns
// and the block writes silu(gate) * up, so gate and up never reach memory
// (the reference does this as two products and three element-wise passes,
// crates/models/qwen/src/forward.rs:1904-1917).
//
// Every wait on a barrier is bounded: if it runs out, the status word gets a
// bit, the block stops issuing work, frees its tensor memory and leaves.
#include "tcgen05.cuh"

namespace mxb {

constexpr int kTcM = 128;     // rows of a tile
constexpr int kTcK = 64;      // k per stage: 64 bfloat16 = one 128-byte swizzle row
constexpr int kTcThreads = 192;

enum TcEpilogue : int { kTcStoreBf16 = 0, kTcStoreF32 = 1, kTcSwiGLU = 2 };

template <int BN, int STAGES_> struct TcConfig {
  static constexpr int kStageBytes = (kTcM + BN) * kTcK * 2;
  static constexpr int kStages = STAGES_;
  static constexpr int kSharedBytes = kStages * kStageBytes + 1024;  // + room to align the tiles to 1024 bytes
};

// EPI: see TcEpilogue. For kTcSwiGLU n is the output width (inter) and map_b
// covers the [2 * inter, k] weight in boxes of BN / 2 rows.
//
// The kernel is persistent: a block walks over tiles (tile, tile + gridDim.x,
// ...), with two accumulators in tensor memory, so the epilogue of one tile
// runs while the MMAs of the next fill the other accumulator and the TMA
// loads run ahead of both. Tiles are numbered with the row tile fastest:
// blocks working side by side share a tile of W.
template <int BN, int EPI, int STAGES_>
__global__ void __launch_bounds__(kTcThreads)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    void* __restrict__ out, int m, int n, int k, long long ldo, int* status) {
  using Config = TcConfig<BN, STAGES_>;
  constexpr int STAGES = Config::kStages;
  constexpr int OUT_COLUMNS = EPI == kTcSwiGLU ? BN / 2 : BN;  // output columns of a tile
  extern __shared__ unsigned char tc_shared_raw[];
  __shared__ __align__(8) uint64_t full_barrier[STAGES];
  __shared__ __align__(8) uint64_t empty_barrier[STAGES];
  __shared__ __align__(8) uint64_t accumulator_full[2];
  __shared__ __align__(8) uint64_t accumulator_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int failed;

  unsigned char* tiles = tc_shared_raw + ((1024 - (shared_address(tc_shared_raw) & 1023)) & 1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (m + kTcM - 1) / kTcM;
  const int n_tiles = (n + OUT_COLUMNS - 1) / OUT_COLUMNS;
  const int total_tiles = m_tiles * n_tiles;
  const int k_blocks = (k + kTcK - 1) / kTcK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      barrier_init(&full_barrier[s], 1);
      barrier_init(&empty_barrier[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(&accumulator_full[b], 1);
      barrier_init(&accumulator_empty[b], kTcThreads - 64);  // every epilogue thread arrives
    }
    barrier_init_fence();
    failed = 0;
  }
  if (warp == 1) {  // one warp allocates both accumulators' columns of tensor memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                 ::"r"(shared_address(&tmem_base_slot)), "r"(2 * BN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ---- producer: TMA loads of the A and B tiles of every k block of every tile
    if (lane == 0) {
      int step = 0;  // k blocks issued so far, over all tiles
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x) {
        const int m0 = (tile % m_tiles) * kTcM, n0 = (tile / m_tiles) * OUT_COLUMNS;
        for (int kb = 0; kb < k_blocks; ++kb, ++step) {
          const int stage = step % STAGES;
          const uint32_t parity = (step / STAGES) & 1;
          if (!barrier_wait(&empty_barrier[stage], parity ^ 1, status)) { failed = 1; break; }
          unsigned char* a_tile = tiles + stage * Config::kStageBytes;
          unsigned char* b_tile = a_tile + kTcM * kTcK * 2;
          barrier_arrive_expect(&full_barrier[stage], Config::kStageBytes);
          tma_load_2d(a_tile, &map_a, kb * kTcK, m0, &full_barrier[stage]);
          if (EPI == kTcSwiGLU) {
            tma_load_2d(b_tile, &map_b, kb * kTcK, n0, &full_barrier[stage]);                            // gate rows
            tma_load_2d(b_tile + (BN / 2) * kTcK * 2, &map_b, kb * kTcK, n + n0, &full_barrier[stage]);  // up rows
          } else {
            tma_load_2d(b_tile, &map_b, kb * kTcK, n0, &full_barrier[stage]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- one thread issues every MMA; completion frees the stage
    if (lane == 0) {
      constexpr uint32_t idesc = tc_instruction_descriptor(kTcM, BN);
      int step = 0, local = 0;
      for (int tile = blockIdx.x; tile < total_tiles && !failed; tile += gridDim.x, ++local) {
        const int buffer = local & 1;
        // The epilogue must have drained this accumulator (two tiles ago).
        if (!barrier_wait(&accumulator_empty[buffer], ((local >> 1) & 1) ^ 1, status)) { failed = 1; break; }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_d = tmem_base + buffer * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++step) {
          const int stage = step % STAGES;
          const uint32_t parity = (step / STAGES) & 1;
          if (!barrier_wait(&full_barrier[stage], parity, status)) { failed = 1; break; }
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint32_t a_address = shared_address(tiles + stage * Config::kStageBytes);
          const uint32_t b_address = a_address + kTcM * kTcK * 2;
#pragma unroll
          for (int kk = 0; kk < kTcK / 16; ++kk) {  // 16 k per instruction: 32 bytes further along the swizzled row
            tc_mma(tmem_d, tc_smem_descriptor(a_address + kk * 32), tc_smem_descriptor(b_address + kk * 32),
                   idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          tc_commit(&empty_barrier[stage]);
        }
        tc_commit(&accumulator_full[buffer]);  // arrives when this tile's accumulator is final
      }
    }
  } else {
    // ---- epilogue: warp w reads the 32 accumulator rows (lanes) (w % 4) * 32 ...
    const int lane_base = (warp & 3) * 32;
    int local = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++local) {
      const int buffer = local & 1;
      const int m0 = (tile % m_tiles) * kTcM, n0 = (tile / m_tiles) * OUT_COLUMNS;
      if (!barrier_wait(&accumulator_full[buffer], (local >> 1) & 1, status)) { failed = 1; break; }
      if (failed) break;
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int row = m0 + lane_base + lane;
      const uint32_t tmem_row = tmem_base + buffer * BN + (static_cast<uint32_t>(lane_base) << 16);
#pragma unroll 1
      for (int c = 0; c < OUT_COLUMNS; c += 32) {
        uint32_t acc[32];
        tc_load_32(tmem_row + c, acc);
        float values[32];
        if (EPI == kTcSwiGLU) {
          uint32_t up[32];
          tc_load_32(tmem_row + BN / 2 + c, up);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // gate and up take the rounding to bfloat16 they would get on their way through memory
            const float gate = to_float(from_float<__nv_bfloat16>(__uint_as_float(acc[i])));
            const float u = to_float(from_float<__nv_bfloat16>(__uint_as_float(up[i])));
            values[i] = __fdividef(gate, 1.0f + __expf(-gate)) * u;  // the result is rounded to bfloat16 anyway
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) values[i] = __uint_as_float(acc[i]);
        }
        if (row < m) {
          const int column = n0 + c;
          if (EPI == kTcStoreF32) {
            float* dst = static_cast<float*>(out) + static_cast<long long>(row) * ldo + column;
            if (column + 32 <= n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(values[i], values[i + 1], values[i + 2], values[i + 3]);
            } else {
              for (int i = 0; i < 32; ++i)
                if (column + i < n) dst[i] = values[i];
            }
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out) + static_cast<long long>(row) * ldo + column;
            if (column + 32 <= n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  __nv_bfloat162 pair = __floats2bfloat162_rn(values[i + 2 * j], values[i + 2 * j + 1]);
                  packed[j] = *reinterpret_cast<uint32_t*>(&pair);
                }
                *reinterpret_cast<uint4*>(dst + i) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
              }
            } else {
              for (int i = 0; i < 32; ++i)
                if (column + i < n) dst[i] = from_float<__nv_bfloat16>(values[i]);
            }
          }
        }
      }
      // This thread has read all it needs of the accumulator: hand it back.
      asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
      barrier_arrive(&accumulator_empty[buffer]);
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (failed && threadIdx.x == 0) {
    // A wait ran out somewhere. Give loads that may still be in flight a
    // millisecond before the block's shared memory goes back.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(2 * BN) : "memory");
  }
}

// ------------------------------------------------------------------ host side
int g_tc_bn = 0, g_tc_deep = -1;  // tuning overrides: tile width, deep (1) or shallow (0) pipeline

template <int BN, int EPI, int STAGES_>
static int launch_tc_staged(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int m, int n, int k,
                            long long ldo, int* status, cudaStream_t stream) {
  using Config = TcConfig<BN, STAGES_>;
  auto kernel = gemm_tcgen05_kernel<BN, EPI, STAGES_>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Config::kSharedBytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  constexpr int out_columns = EPI == kTcSwiGLU ? BN / 2 : BN;
  const int tiles = ((n + out_columns - 1) / out_columns) * ((m + kTcM - 1) / kTcM);
  static int sm_count = 0;
  if (sm_count == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
  }
  dim3 grid(tiles < sm_count ? tiles : sm_count);  // one block per SM walks over the tiles
  kernel<<<grid, kTcThreads, Config::kSharedBytes, stream>>>(map_a, map_b, out, m, n, k, ldo, status);
  return static_cast<int>(cudaGetLastError());
}

// Deep: the whole shared memory as pipeline (the default; a block owns its SM
// and tensor memory holds two accumulators). Shallow: half the stages.
template <int BN, int EPI>
static int launch_tc(const CUtensorMap& map_a, const CUtensorMap& map_b, void* out, int m, int n, int k,
                     long long ldo, int* status, cudaStream_t stream) {
  constexpr int deep = BN >= 256 ? 4 : (BN >= 128 ? 6 : 8);
  const bool shallow = g_tc_deep == 0;
  if (shallow) return launch_tc_staged<BN, EPI, deep / 2>(map_a, map_b, out, m, n, k, ldo, status, stream);
  return launch_tc_staged<BN, EPI, deep>(map_a, map_b, out, m, n, k, ldo, status, stream);
}

}  // namespace mxb

using namespace mxb;

// Shapes the kernel takes: k a multiple of 8 (row strides on 16-byte
// boundaries), rows of a and w contiguous, bases 16-byte aligned.
MXB_API int mxb_gemm_tcgen05_supported(int m, int n, int k, long long lda, long long ldw) {
  return m >= 1 && n >= 1 && k >= 8 && k % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 ? 1 : 0;
}

// epilogue: 0 bfloat16 out[m, n], 1 float32 out[m, n], 2 SwiGLU: w is
// [2 * n, k] (gate rows, then up rows) and out is bfloat16 [m, n].
MXB_API int mxb_gemm_tcgen05(void* out, const void* a, const void* w, int m, int n, int k, long long lda,
                             long long ldw, long long ldo, int epilogue, int* status, cudaStream_t stream) {
  if (!mxb_gemm_tcgen05_supported(m, n, k, lda, ldw)) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return static_cast<int>(cudaErrorInvalidValue);
  const int w_rows = epilogue == kTcSwiGLU ? 2 * n : n;
  // Narrow outputs take narrower tiles so that the grid still covers the GPU.
  const int m_tiles = (m + kTcM - 1) / kTcM;
  int bn = 256;
  if (epilogue == kTcSwiGLU) {
    // A SwiGLU tile of width bn holds bn / 2 gate and bn / 2 up rows. Timed
    // on [m, 1024] x [6144, 1024]: up to 128 rows 64 is fastest (10 against 14
    // us), at 256 rows 128 (12 against 15), from 512 rows on 256.
    bn = m <= 128 ? 64 : (m <= 256 ? 128 : 256);
  } else {
    // 118 tiles keep four fifths of the 148 SMs busy; below that, narrower tiles.
    if (m_tiles * ((n + 255) / 256) < 118) bn = 128;
    if (bn == 128 && m_tiles * ((n + 127) / 128) < 118) bn = 64;
  }
  if (g_tc_bn != 0) bn = g_tc_bn;
  CUtensorMap map_a, map_b;
  const int b_box = epilogue == kTcSwiGLU ? bn / 2 : bn;
  if (!make_map(&map_a, a, m, k, lda, kTcM) || !make_map(&map_b, w, w_rows, k, ldw, b_box))
    return static_cast<int>(cudaErrorInvalidValue);
  if (epilogue == kTcSwiGLU) {
    if (bn == 256) return launch_tc<256, kTcSwiGLU>(map_a, map_b, out, m, n, k, ldo, status, stream);
    if (bn == 128) return launch_tc<128, kTcSwiGLU>(map_a, map_b, out, m, n, k, ldo, status, stream);
    return launch_tc<64, kTcSwiGLU>(map_a, map_b, out, m, n, k, ldo, status, stream);
  }
  if (epilogue == kTcStoreF32) {
    if (bn == 256) return launch_tc<256, kTcStoreF32>(map_a, map_b, out, m, n, k, ldo, status, stream);
    if (bn == 128) return launch_tc<128, kTcStoreF32>(map_a, map_b, out, m, n, k, ldo, status, stream);
    return launch_tc<64, kTcStoreF32>(map_a, map_b, out, m, n, k, ldo, status, stream);
  }
  if (epilogue != kTcStoreBf16) return static_cast<int>(cudaErrorInvalidValue);
  if (bn == 256) return launch_tc<256, kTcStoreBf16>(map_a, map_b, out, m, n, k, ldo, status, stream);
  if (bn == 128) return launch_tc<128, kTcStoreBf16>(map_a, map_b, out, m, n, k, ldo, status, stream);
  return launch_tc<64, kTcStoreBf16>(map_a, map_b, out, m, n, k, ldo, status, stream);
}

// Tuning hook: force the tile width (64, 128, 256; 0 = choose) and the
// pipeline depth (1 deep, 0 shallow, -1 = choose).
MXB_API void mxb_gemm_tcgen05_tune(int bn, int deep) {
  mxb::g_tc_bn = bn;
  mxb::g_tc_deep = deep;
}
