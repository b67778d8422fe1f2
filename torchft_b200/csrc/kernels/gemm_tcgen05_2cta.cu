// Persistent bf16 GEMM for sm_100a on CTA pairs: two CTAs of a cluster (two SMs) compute one
// 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
//   C[M,N] (+)= op(A) * op(B)        (same operand layouts as gemm_tcgen05.cu)
//
// Per k-block each CTA brings in only ITS half of the tile: 128 rows of A and 128 of the tile's 256
// columns of B (32 KB instead of the 48 KB a single-CTA 128 x 256 tile needs), with ordinary TMA
// loads that target the issuing CTA's shared memory -- nothing here is a cluster-multicast load.  The
// even CTA of the pair (the leader) issues every MMA; the tensor cores of both SMs read A from their
// own shared memory and B from both halves, and each SM accumulates its 128 rows x 256 columns in its
// own tensor memory.  Halving the shared-memory fill per FLOP is what the pair buys.
//
// Synchronisation between the two CTAs:
//   full[s]    lives in the leader; the leader's producer arms it with the byte count of BOTH CTAs'
//              loads and both producers' TMA loads complete on it (cta_group::2 loads may signal the
//              partner's barrier).
//   empty[s]   lives in both; one tcgen05.commit of the leader arrives on both (commit multicast).
//   tfull[b]   lives in both; same mechanism, tells each CTA's epilogue warps that accumulator b is done.
//   tempty[b]  lives in the leader, 8 arrivals: the four epilogue warps of either CTA.
//
// Tail: with T tiles on G CTA pairs the last T mod G tiles would occupy a whole wave.  When they are
// at most G / 2 they are cut into halves of 256 x 128, which takes half a wave instead.
//
// Every wait is bounded (see common.cuh); a CTA that gives up records a status and leaves through the
// cluster barrier at the end like the others.
#include "common.cuh"
#include "tensormap.cuh"

namespace tft {
namespace gemm2 {

constexpr int BM = 256;  // per pair; 128 rows per CTA
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = 128 * BK * 2;
constexpr uint32_t B_STAGE_BYTES = 128 * BK * 2;
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;

// ---------------------------------------------------------------- cluster and cta_group::2 forms
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `smem_addr` (a shared::cta address of this CTA) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion is counted on a barrier that may live in
// the partner CTA (no multicast: one destination).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols));
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols));
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at the same shared-memory offset in BOTH CTAs of the pair once every MMA
// issued so far by this thread has retired.
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(mask)
      : "memory");
}

// ---------------------------------------------------------------- schedule
struct Schedule {
  int tiles_m, tiles_n;
  int whole_units;  // units [0, whole_units) are whole tiles
  int total_units;  // the rest are halves (256 x 128) of the remaining tiles
};
struct Unit {
  int m0, n0, ncols;
};

__host__ __device__ inline Schedule make_schedule(int M, int N, int pairs) {
  Schedule s;
  s.tiles_m = (M + BM - 1) / BM;
  s.tiles_n = (N + BN - 1) / BN;
  const int tiles = s.tiles_m * s.tiles_n;
  const int rest = tiles % pairs;
  if (rest > 0 && 2 * rest <= pairs && tiles > pairs) {
    s.whole_units = tiles - rest;
    s.total_units = s.whole_units + 2 * rest;
  } else {
    s.whole_units = tiles;
    s.total_units = tiles;
  }
  return s;
}

__device__ __forceinline__ Unit unit_at(const Schedule& s, int u) {
  int t = u, half = -1;
  if (u >= s.whole_units) {
    t = s.whole_units + ((u - s.whole_units) >> 1);
    half = (u - s.whole_units) & 1;
  }
  const int per_group = GROUP_M * s.tiles_n;
  const int g = t / per_group;
  const int first_m = g * GROUP_M;
  const int gm = min(GROUP_M, s.tiles_m - first_m);
  const int r = t - g * per_group;
  Unit out;
  out.m0 = (first_m + r % gm) * BM;
  out.n0 = (r / gm) * BN + (half > 0 ? BN / 2 : 0);
  out.ncols = half < 0 ? BN : BN / 2;
  return out;
}

// ---------------------------------------------------------------- epilogue stores
template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* C, int ldc, int row, int col0, int M, int N, const uint32_t (&r)[32],
                                            int accumulate);

template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* C, int ldc, int row, int col0, int M, int N,
                                                           const uint32_t (&r)[32], int accumulate) {
  if (row >= M) return;
  __nv_bfloat16* p = C + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (col0 + g * 8 >= N) break;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
    if (accumulate) {
      const uint4 old = *reinterpret_cast<const uint4*>(p + g * 8);
      const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(o2[j]);
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
__device__ __forceinline__ void store_chunk<float>(float* C, int ldc, int row, int col0, int M, int N,
                                                   const uint32_t (&r)[32], int accumulate) {
  if (row >= M) return;
  float* p = C + static_cast<size_t>(row) * ldc + col0;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    if (col0 + g * 4 >= N) break;
    float4 v = make_float4(__uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]), __uint_as_float(r[g * 4 + 2]),
                           __uint_as_float(r[g * 4 + 3]));
    if (accumulate) {
      const float4 o = *reinterpret_cast<const float4*>(p + g * 4);
      v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
    }
    *reinterpret_cast<float4*>(p + g * 4) = v;
  }
}

// ---------------------------------------------------------------- kernel
template <bool A_MN, bool B_MN, typename OutT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
             OutT* __restrict__ C, int M, int N, int K, int ldc, int accumulate, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // same offset in both CTAs: same kernel, same layout
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
  const uint32_t cta = cluster_ctarank();  // 0: leader of the pair
  const int pair = blockIdx.x >> 1;
  const int pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 8);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers of both CTAs are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const Schedule sched = make_schedule(M, N, pairs);
  const int kblocks = (K + BK - 1) / BK;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int u = pair; u < sched.total_units && ok; u += pairs) {
        const Unit un = unit_at(sched, u);
        const int my_m = un.m0 + static_cast<int>(cta) * 128;
        const int half_cols = un.ncols >> 1;  // this CTA's share of the unit's columns
        const int my_n = un.n0 + static_cast<int>(cta) * half_cols;
        const uint32_t my_bytes = A_STAGE_BYTES + static_cast<uint32_t>(half_cols) * BK * 2;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * STAGE_BYTES;
          const uint32_t sb = sa + A_STAGE_BYTES;
          const uint32_t full_in_leader = map_to_cta(full_bar(stage), 0);
          if (cta == 0) mbar_expect_tx(full_bar(stage), 2 * my_bytes);
          if (!A_MN) {
            tma_load_2d_pair(sa, &tma_a, full_in_leader, kb * BK, my_m);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(sa + j * 8192, &tma_a, full_in_leader, my_m + 64 * j, kb * BK);
          }
          for (int j = 0; j < half_cols / 64; ++j) {
            if (!B_MN)
              tma_load_2d_pair(sb + j * 8192, &tma_b, full_in_leader, kb * BK, my_n + 64 * j);
            else
              tma_load_2d_pair(sb + j * 8192, &tma_b, full_in_leader, my_n + 64 * j, kb * BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && cta == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int u = pair; u < sched.total_units && ok; u += pairs, ++it) {
        const Unit un = unit_at(sched, u);
        const uint32_t idesc = un.ncols == BN ? make_idesc_bf16(BM, BN, A_MN, B_MN) : make_idesc_bf16(BM, BN / 2, A_MN, B_MN);
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
            const uint64_t adesc = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 16, 1024);
            umma_bf16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(tfull_bar(buf));
      }
    }
  } else {
    const int q = warp & 3;  // tensor-memory lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int u = pair; u < sched.total_units && ok; u += pairs, ++it) {
      const Unit un = unit_at(sched, u);
      const int buf = it & 1;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = un.m0 + static_cast<int>(cta) * 128 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int c = 0; c < un.ncols / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (un.n0 + c * 32 < N) store_chunk<OutT>(C, ldc, row, un.n0 + c * 32, M, N, r, accumulate);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty_bar(buf), 0));
    }
  }

  __syncthreads();
  if (*abort_flag) {
    // Give loads that may still be in flight time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, static_cast<int>(kTimeoutBarrier));
  }
  tc_fence_before();
  cluster_sync_all();  // neither CTA's shared memory, barriers or tensor memory go away under its partner
  tc_fence_after();
  if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

static int g_pairs = 0;

template <bool A_MN, bool B_MN, typename OutT>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, void* c, int M, int N, int K, int ldc, int accumulate,
                   int* status, cudaStream_t stream) {
  auto kfn = gemm2_kernel<A_MN, B_MN, OutT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  if (g_pairs == 0) {
    // How many CTA pairs the device can hold at once (SMs pair up inside a GPC, so this can be a few
    // less than half the SM count).
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms / 2 * 2);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, kfn, &cfg) != cudaSuccess || clusters < 1) {
      cudaGetLastError();
      clusters = sms / 2;
    }
    g_pairs = clusters < sms / 2 ? clusters : sms / 2;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int pairs = tiles < g_pairs ? tiles : g_pairs;
  kfn<<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, static_cast<OutT*>(c), M, N, K, ldc, accumulate, status);
  return cudaGetLastError();
}

}  // namespace gemm2
}  // namespace tft

// Same contract as tft_gemm_bf16 (gemm_tcgen05.cu), computed on CTA pairs.
TFT_API int tft_gemm2_bf16(const void* a, const void* b, void* c, int M, int N, int K, int lda, int ldb, int ldc,
                           int a_mn, int b_mn, int out_fp32, int accumulate, int* status, cudaStream_t stream) {
  using namespace tft;
  using namespace tft::gemm2;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8) || (reinterpret_cast<uintptr_t>(a) & 15) ||
      (reinterpret_cast<uintptr_t>(b) & 15) || (reinterpret_cast<uintptr_t>(c) & 15))
    return -1;  // misaligned pointer or leading dimension
  CUtensorMap ta, tb;
  bool ok;
  if (!a_mn)
    ok = make_tensormap(&ta, a, 2, 2, K, M, 1, uint64_t(lda) * 2, 0, BK, 128, 1, 1);
  else
    ok = make_tensormap(&ta, a, 2, 2, M, K, 1, uint64_t(lda) * 2, 0, 64, BK, 1, 1);
  if (!ok) return -2;  // tensor map of A rejected
  if (!b_mn)
    ok = make_tensormap(&tb, b, 2, 2, K, N, 1, uint64_t(ldb) * 2, 0, BK, 64, 1, 1);
  else
    ok = make_tensormap(&tb, b, 2, 2, N, K, 1, uint64_t(ldb) * 2, 0, 64, BK, 1, 1);
  if (!ok) return -3;  // tensor map of B rejected
  cudaGetLastError();  // drop stale errors left by other libraries on this thread

  cudaError_t e;
#define TFT_GEMM2_DISPATCH(AM, BM_)                                                           \
  (out_fp32 ? launch<AM, BM_, float>(ta, tb, c, M, N, K, ldc, accumulate, status, stream)     \
            : launch<AM, BM_, __nv_bfloat16>(ta, tb, c, M, N, K, ldc, accumulate, status, stream))
  if (!a_mn && !b_mn) e = TFT_GEMM2_DISPATCH(false, false);
  else if (!a_mn && b_mn) e = TFT_GEMM2_DISPATCH(false, true);
  else if (a_mn && !b_mn) e = TFT_GEMM2_DISPATCH(true, false);
  else e = TFT_GEMM2_DISPATCH(true, true);
#undef TFT_GEMM2_DISPATCH
  return static_cast<int>(e);
}
