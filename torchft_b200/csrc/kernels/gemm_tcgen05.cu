// Persistent bf16 GEMM for sm_100a: TMA -> 128B-swizzled shared memory -> tcgen05.mma with
// fp32 accumulators in tensor memory -> tcgen05.ld epilogue.
//
//   C[M,N] (+)= op(A) * op(B)
//
// Either operand may be K-major (rows of the stored matrix run along K) or MN-major
// (rows run along M resp. N), which covers the forward (X * W^T), data-gradient
// (dY * W) and weight-gradient (dY^T * X) products of a linear layer without any
// transposition pass.  One CTA per SM walks output tiles of 128 x 256; the 512 tensor
// memory columns hold two accumulators so the epilogue of one tile overlaps the main
// loop of the next.  Warp roles: warp 0 issues TMA loads, warp 1 issues MMAs, warps 2-5
// drain tensor memory.
//
// No thread-block clusters are used and every TMA load targets only the issuing CTA.
#include "common.cuh"
#include "tensormap.cuh"

namespace tft {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2;
constexpr uint32_t B_STAGE_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr int GROUP_M = 16;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

struct TileCoord {
  int m0, n0;
};

__device__ __forceinline__ TileCoord tile_coord(int t, int tiles_m, int tiles_n) {
  const int per_group = GROUP_M * tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int r = t - g * per_group;
  TileCoord c;
  c.m0 = (first_m + r % gm) * BM;
  c.n0 = (r / gm) * BN;
  return c;
}

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* C, int ldc, int row, int col0, int M, int N,
                                            const uint32_t (&r)[32], int accumulate);

template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* C, int ldc, int row,
                                                           int col0, int M, int N,
                                                           const uint32_t (&r)[32],
                                                           int accumulate) {
  if (row >= M) return;
  __nv_bfloat16* p = C + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (col0 + g * 8 >= N) break;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
    if (accumulate) {
      uint4 old = *reinterpret_cast<const uint4*>(p + g * 8);
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(o2[j]);
        v[2 * j] += f.x;
        v[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(v[0], v[1]);
    o.y = pack_bf16(v[2], v[3]);
    o.z = pack_bf16(v[4], v[5]);
    o.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4*>(p + g * 8) = o;
  }
}

template <>
__device__ __forceinline__ void store_chunk<float>(float* C, int ldc, int row, int col0, int M,
                                                   int N, const uint32_t (&r)[32],
                                                   int accumulate) {
  if (row >= M) return;
  float* p = C + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    if (col0 + g * 4 >= N) break;
    float4 v = make_float4(__uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]),
                           __uint_as_float(r[g * 4 + 2]), __uint_as_float(r[g * 4 + 3]));
    if (accumulate) {
      float4 o = *reinterpret_cast<const float4*>(p + g * 4);
      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
    }
    *reinterpret_cast<float4*>(p + g * 4) = v;
  }
}

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
            OutT* __restrict__ C, int M, int N, int K, int ldc, int accumulate, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bar_base = base + STAGES * STAGE_BYTES;
  // barrier slots: [0,S) full, [S,2S) empty, 2S..2S+1 tmem_full, 2S+2..2S+3 tmem_empty
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 5);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + BK - 1) / BK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sa, &tma_a, full_bar(stage), kb * BK, tc.m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * 8192, &tma_a, full_bar(stage), tc.m0 + 64 * j, kb * BK);
          }
          if (!B_MN) {
            tma_load_2d(sb, &tma_b, full_bar(stage), kb * BK, tc.n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * 8192, &tma_b, full_bar(stage), tc.n0 + 64 * j, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), (((it >> 1) & 1) ^ 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024)
                                        : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024)
                                        : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const TileCoord tc = tile_coord(t, tiles_m, tiles_n);
      const int buf = it & 1;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tc.m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (tc.n0 + c * 32 < N) store_chunk<OutT>(C, ldc, row, tc.n0 + c * 32, M, N, r, accumulate);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }

  __syncthreads();
  if (*abort_flag) {
    // Give loads that may still be in flight time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, static_cast<int>(kTimeoutBarrier));
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

static int g_sm_count = 0;

template <bool A_MN, bool B_MN, typename OutT>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, void* c, int M, int N, int K,
                   int ldc, int accumulate, int* status, cudaStream_t stream) {
  auto kfn = gemm_kernel<A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < g_sm_count ? tiles : g_sm_count;
  kfn<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, static_cast<OutT*>(c), M, N, K, ldc,
                                                 accumulate, status);
  return cudaGetLastError();
}

}  // namespace gemm
}  // namespace tft

// C[M,N] (+)= op(A) op(B), bf16 inputs, fp32 accumulation.
//   a_mn == 0: A stored [M, K] (row stride lda)      a_mn == 1: A stored [K, M]
//   b_mn == 0: B stored [N, K] (row stride ldb)      b_mn == 1: B stored [K, N]
//   out_fp32: C is float, otherwise bf16.  accumulate: C += instead of C =.
// Requirements: pointers 16-byte aligned, lda/ldb/ldc multiples of 8 elements, N % 8 == 0.
// status (optional device int) receives a non-zero code if a device-side wait gave up.
TFT_API int tft_gemm_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda,
                          int ldb, int ldc, int a_mn, int b_mn, int out_fp32, int accumulate,
                          int* status, cudaStream_t stream) {
  using namespace tft;
  using namespace tft::gemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8) ||
      (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
      (reinterpret_cast<uintptr_t>(c) & 15))
    return -1;  // misaligned pointer or leading dimension
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn)
    ok = make_tensormap(&ta, a, 2, 2, K, M, 1, uint64_t(lda) * 2, 0, BK, BM, 1, 1);
  else
    ok = make_tensormap(&ta, a, 2, 2, M, K, 1, uint64_t(lda) * 2, 0, 64, BK, 1, 1);
  if (!ok) return -2;  // tensor map of A rejected
  if (!b_mn)
    ok = make_tensormap(&tb, b, 2, 2, K, N, 1, uint64_t(ldb) * 2, 0, BK, BN, 1, 1);
  else
    ok = make_tensormap(&tb, b, 2, 2, N, K, 1, uint64_t(ldb) * 2, 0, 64, BK, 1, 1);
  if (!ok) return -3;  // tensor map of B rejected
  cudaGetLastError();  // drop stale errors left by other libraries on this thread

  cudaError_t e;
#define TFT_GEMM_DISPATCH(AM, BM_)                                                             \
  (out_fp32 ? launch<AM, BM_, float>(ta, tb, c, M, N, K, ldc, accumulate, status, stream)      \
            : launch<AM, BM_, __nv_bfloat16>(ta, tb, c, M, N, K, ldc, accumulate, status, stream))
  if (!a_mn && !b_mn) e = TFT_GEMM_DISPATCH(false, false);
  else if (!a_mn && b_mn) e = TFT_GEMM_DISPATCH(false, true);
  else if (a_mn && !b_mn) e = TFT_GEMM_DISPATCH(true, false);
  else e = TFT_GEMM_DISPATCH(true, true);
#undef TFT_GEMM_DISPATCH
  return static_cast<int>(e);
}
