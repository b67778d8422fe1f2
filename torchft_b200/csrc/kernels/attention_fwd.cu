// Causal grouped-query flash attention, forward, on tcgen05 tensor cores.
//
// One CTA handles 128 query rows of one head.  Warp 0 streams K/V tiles with TMA
// (two stages), warp 1 issues the MMAs, warps 2-9 run the online softmax with TWO threads
// per query row (each owns 64 of the 128 key columns of a tile and half of the output
// columns; the row maximum is exchanged through shared memory):
//
//   S_j  = Q K_j^T          tcgen05.mma, fp32 scores in tensor memory (two buffers)
//   P_j  = exp2(S_j*c - m)  softmax threads read S from tensor memory, keep the running
//                           max / sum, and write P as bf16 into swizzled shared memory
//   PV_j = P_j V_j          tcgen05.mma into a third tensor-memory region
//   O    = O*alpha + PV_j   folded into registers by the softmax threads one tile later
//
// The MMA warp issues S_{j+1} before PV_j, so the score MMA of the next tile overlaps the
// softmax of the current one.  Only the diagonal tile applies the causal mask; all other
// tiles run a mask-free inner loop.  Output: O (bf16) and the base-2 log-sum-exp per row.
#include "attention_common.cuh"

namespace tft {
namespace attn {

template <int HD>
struct FwdSmem {
  static constexpr uint32_t TILE = BLK * HD * 2;
  static constexpr uint32_t Q = 0;
  static constexpr uint32_t K = Q + TILE;           // 2 stages
  static constexpr uint32_t V = K + 2 * TILE;       // 2 stages
  static constexpr uint32_t P = V + 2 * TILE;       // [128 x 128] bf16
  static constexpr uint32_t BARS = P + BLK * BLK * 2;
  static constexpr uint32_t XCHG = BARS + 256;      // float [2 parities][2 halves][128 rows]
  static constexpr uint32_t TOTAL = XCHG + 2 * 2 * BLK * 4 + 1024;
};

enum FwdBar { Q_FULL = 0, K_FULL0, K_FULL1, V_FULL0, V_FULL1, KV_EMPTY0, KV_EMPTY1, S_FULL0, S_FULL1, P_READY, PV_FULL, NUM_FWD_BARS };

constexpr int FWD_THREADS = 320;      // TMA warp, MMA warp, 8 softmax warps
constexpr int SOFTMAX_THREADS = 256;

__device__ __forceinline__ void softmax_group_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}

// Row maximum over 32 score columns; MASKED applies the causal condition col <= r.
template <bool MASKED>
__device__ __forceinline__ float chunk_max(const uint32_t (&sv)[32], int col0, int r, float mx) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float s = __uint_as_float(sv[i]);
    if (!MASKED || (col0 + i) <= r) mx = fmaxf(mx, s);
  }
  return mx;
}

template <bool MASKED>
__device__ __forceinline__ float chunk_exp(const uint32_t (&sv)[32], int col0, int r, float scale_log2, float m,
                                           float (&p)[32]) {
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float e = fast_exp2(__uint_as_float(sv[i]) * scale_log2 - m);
    p[i] = (!MASKED || (col0 + i) <= r) ? e : 0.f;
    sum += p[i];
  }
  return sum;
}

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, __nv_bfloat16* __restrict__ O, float* __restrict__ LSE,
                int S, int Hq, int Hkv, long long ldo, float scale_log2, int* status) {
  using L = FwdSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_FWD_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_FWD_BARS + 8);
  float* xchg = reinterpret_cast<float*>(smem + L::XCHG);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (S + BLK - 1) / BLK;
  const int qt = n_qtiles - 1 - blockIdx.x / Hq;  // heaviest tiles first, over all heads
  const int head = blockIdx.x % Hq, batch = blockIdx.y;
  const int kv_head = head / (Hq / Hkv);
  const int n_kv = qt + 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_FWD_BARS; ++i) mbar_init(bar(i), i == P_READY ? SOFTMAX_THREADS : 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_pv = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(Q_FULL), L::TILE);
      load_tile<HD>(base + L::Q, &tq, bar(Q_FULL), head, qt * BLK, batch);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar(KV_EMPTY0 + st), ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(K_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::K + st * L::TILE, &tk, bar(K_FULL0 + st), kv_head, j * BLK, batch);
        mbar_expect_tx(bar(V_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::V + st * L::TILE, &tv, bar(V_FULL0 + st), kv_head, j * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BLK, HD, false, true);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(bar(K_FULL0 + st), (j >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(tmem_s[st], kmajor_desc(base + L::Q, k), kmajor_desc(base + L::K + st * L::TILE, k), idesc_s,
                    k != 0);
        umma_commit(bar(S_FULL0 + st));
        return true;
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag);
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        const int st = j & 1;
        if (!mbar_wait(bar(P_READY), j & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(bar(V_FULL0 + st), (j >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_bf16(tmem_pv, kmajor_desc(base + L::P, k), mnmajor_desc(base + L::V + st * L::TILE, k), idesc_pv,
                    k != 0);
        umma_commit(bar(PV_FULL));
        umma_commit(bar(KV_EMPTY0 + st));
      }
    }
  } else {
    constexpr int OC = HD / 2;               // output columns owned by this thread
    const int q = warp & 3;                  // tensor-memory lane quarter of this warp
    const int half = (warp - 2) >> 2;        // which 64 key columns / which half of the output
    const int r = q * 32 + lane;             // row inside the tile
    const int row = qt * BLK + r;            // row inside the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    float o[OC];
#pragma unroll
    for (int i = 0; i < OC; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    // Giving up must not strand group mates at the named barrier.  A wait that runs out sets the
    // CTA-wide abort flag and the thread keeps walking to the next group barrier; right after a
    // barrier every thread reads the flag, so all 256 leave the loop at the same point.
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      const bool got_s = mbar_wait(bar(S_FULL0 + st), (j >> 1) & 1, abort_flag);
      tc_fence_after();
      const bool diag = (j == qt);
      float mx = -INFINITY;
      if (got_s) {
#pragma unroll 1
        for (int c = half * 2; c < half * 2 + 2; ++c) {
          uint32_t sv[32];
          tmem_ld_32x32(tmem_s[st] + lane_addr + c * 32, sv);
          tmem_ld_wait();
          mx = diag ? chunk_max<true>(sv, c * 32, r, mx) : chunk_max<false>(sv, c * 32, r, mx);
        }
      }
      float* xm = xchg + ((j & 1) * 2) * BLK;
      xm[half * BLK + r] = mx;
      softmax_group_sync();
      if (*abort_flag) { ok = false; break; }  // uniform: the flag was set before somebody's arrival
      mx = fmaxf(mx, xm[(half ^ 1) * BLK + r]);
      const float m_new = fmaxf(m, mx * scale_log2);
      const float alpha = fast_exp2(m - m_new);  // 0 on the first tile (m = -inf)
      if (j > 0) {
        if (!mbar_wait(bar(PV_FULL), (j - 1) & 1, abort_flag)) continue;  // leaves at the next barrier
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t pv[32];
          tmem_ld_32x32(tmem_pv + lane_addr + half * OC + c * 32, pv);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(pv[i])) * alpha;
        }
      }
      l *= alpha;
      m = m_new;
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t sv[32];
        tmem_ld_32x32(tmem_s[st] + lane_addr + c * 32, sv);
        tmem_ld_wait();
        float p[32];
        l += diag ? chunk_exp<true>(sv, c * 32, r, scale_log2, m, p) : chunk_exp<false>(sv, c * 32, r, scale_log2, m, p);
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 u;
          u.x = pack_bf16(p[t * 8 + 0], p[t * 8 + 1]);
          u.y = pack_bf16(p[t * 8 + 2], p[t * 8 + 3]);
          u.z = pack_bf16(p[t * 8 + 4], p[t * 8 + 5]);
          u.w = pack_bf16(p[t * 8 + 6], p[t * 8 + 7]);
          *reinterpret_cast<uint4*>(smem + L::P + swizzled_chunk(r, c * 4 + t)) = u;
        }
      }
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(bar(P_READY));
    }
    if (ok) {
      // every thread that left the loop normally takes this barrier, whatever its last wait said
      const bool got_pv = mbar_wait(bar(PV_FULL), (n_kv - 1) & 1, abort_flag);
      tc_fence_after();
      // total row sum = the two halves' partial sums (both were rescaled with the same maxima)
      float* xs = xchg + ((n_kv & 1) * 2) * BLK;
      xs[half * BLK + r] = l;
      softmax_group_sync();
      ok = got_pv && !*abort_flag;
      l += xs[(half ^ 1) * BLK + r];
    }
    if (ok) {
      const float inv = 1.f / l;
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t pv[32];
        tmem_ld_32x32(tmem_pv + lane_addr + half * OC + c * 32, pv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = (o[c * 32 + i] + __uint_as_float(pv[i])) * inv;
      }
      if (row < S) {
        __nv_bfloat16* dst = O + (static_cast<long long>(batch) * S + row) * ldo + head * HD + half * OC;
#pragma unroll
        for (int c = 0; c < OC / 8; ++c) {
          uint4 u;
          u.x = pack_bf16(o[c * 8 + 0], o[c * 8 + 1]);
          u.y = pack_bf16(o[c * 8 + 2], o[c * 8 + 3]);
          u.z = pack_bf16(o[c * 8 + 4], o[c * 8 + 5]);
          u.w = pack_bf16(o[c * 8 + 6], o[c * 8 + 7]);
          reinterpret_cast<uint4*>(dst)[c] = u;
        }
        if (half == 0) LSE[(static_cast<long long>(batch) * Hq + head) * S + row] = m + log2f(l);
      }
    }
    tc_fence_before();
  }

  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, static_cast<int>(kTimeoutBarrier));
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int HD>
int launch_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq, int Hkv,
               long long ldq, long long ldk, long long ldv, long long ldo, float scale, int* status,
               cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (!make_attn_tensormap(&tq, q, HD, Hq, S, B, ldq)) return -2;
  if (!make_attn_tensormap(&tk, k, HD, Hkv, S, B, ldk)) return -3;
  if (!make_attn_tensormap(&tv, v, HD, Hkv, S, B, ldv)) return -4;
  auto kfn = attn_fwd_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaGetLastError();
  dim3 grid(((S + BLK - 1) / BLK) * Hq, B, 1);
  kfn<<<grid, FWD_THREADS, FwdSmem<HD>::TOTAL, stream>>>(tq, tk, tv, static_cast<__nv_bfloat16*>(o), lse, S, Hq, Hkv,
                                                         ldo, scale * 1.4426950408889634f, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace attn
}  // namespace tft

// Causal attention forward.  q [B,S,Hq,hd], k/v [B,S,Hkv,hd] bf16 with token strides ldq/ldk/ldv
// (elements; views into a fused qkv buffer are fine), o [B,S,Hq,hd] bf16 with token stride
// ldo, lse [B,Hq,S] fp32 (base-2 log-sum-exp of the scaled scores).  hd is 64 or 128.
TFT_API int tft_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                         int Hkv, int hd, int ldq, int ldk, int ldv, float scale, int* status,
                         cudaStream_t stream) {
  using namespace tft::attn;
  if (Hq % Hkv || (ldq % 8) || (ldk % 8) || (ldv % 8)) return -1;
  const long long ldo = static_cast<long long>(Hq) * hd;
  if (hd == 128) return launch_fwd<128>(q, k, v, o, lse, B, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, status, stream);
  if (hd == 64) return launch_fwd<64>(q, k, v, o, lse, B, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, status, stream);
  return -1;
}
