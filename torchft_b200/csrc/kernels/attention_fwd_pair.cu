// Causal grouped-query flash attention, forward, two query tiles per CTA in ping-pong.
//
// One CTA handles 256 query rows of one head as two tiles A and B of 128 rows.  Every K/V tile that
// is streamed in (TMA, two stages, K and V released separately) is used by both.  The softmax of one
// tile runs while the tensor cores work on the other:
//
//   tensor core:   ... PV_A(j)  S_A(j+1)  PV_B(j)  S_B(j+1)  PV_A(j+1) ...
//   softmax A:              softmax of S_A(j+1) ................
//   softmax B:     softmax of S_B(j) .....            softmax of S_B(j+1) ...
//
// What lives where:
//   S = Q K^T      tcgen05.mma, fp32 scores in tensor memory, one 128-column region per tile
//   P              bf16, written by the softmax threads with tcgen05.st INTO the first 64 columns of
//                  the score region it was computed from (every score has been read before the
//                  columns it occupied are overwritten) and consumed from tensor memory as the A
//                  operand of the PV product: it never touches shared memory
//   O = sum P V    accumulated in tensor memory by the PV products themselves (accumulate flag)
//
// Because O is not carried in registers, rescaling it when the running row maximum moves would cost a
// tensor-memory round trip per key tile.  The maximum used for the exponents is therefore allowed to
// lag: it is raised (and O and the row sum rescaled) only when the true maximum has moved by more
// than 2^8, which after the first key tiles is rare.  P then ranges up to 256 instead of 1, exact in
// bf16 terms and far from overflow in the fp32 sums; the log-sum-exp that is stored is exact.
//
// One softmax thread per query row (warps 2-5: tile A, warps 6-9: tile B; a warp reads the
// tensor-memory lanes of its quarter), so no row statistic is exchanged between threads.  The MMA
// warp's program order gives every ordering the data needs: S_t(j+1) is issued after PV_t(j), and a
// commit completes only when everything issued before it has, so "scores of step j+1 are ready" also
// means "the PV product of step j has finished reading P and writing O".
//
// Every wait is bounded (common.cuh).  Output: O (bf16) and the base-2 log-sum-exp per row.
#include "attention_common.cuh"

#ifndef TFT_ATTN_POLY_OF_4
#define TFT_ATTN_POLY_OF_4 0
#endif

namespace tft {
namespace attn {

template <int HD>
struct PairSmem {
  static constexpr uint32_t TILE = BLK * HD * 2;
  static constexpr uint32_t Q = 0;             // tiles A and B
  static constexpr uint32_t K = Q + 2 * TILE;  // 2 stages
  static constexpr uint32_t V = K + 2 * TILE;  // 2 stages
  static constexpr uint32_t BARS = V + 2 * TILE;
  static constexpr uint32_t TOTAL = BARS + 256 + 1024;
};

enum PairBar {
  PQ_FULL = 0, PK_FULL0, PK_FULL1, PV_FULL0, PV_FULL1, PK_EMPTY0, PK_EMPTY1, PV_EMPTY0, PV_EMPTY1,
  PS_FULL_A, PS_FULL_B, PP_LO_A, PP_LO_B, PP_HI_A, PP_HI_B, PO_FULL_A, PO_FULL_B, NUM_PAIR_BARS
};

constexpr int PAIR_THREADS = 320;  // TMA warp, MMA warp, 4 softmax warps per tile
constexpr float LAZY_RESCALE_LOG2 = 8.0f;

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  uint32_t lo[16], hi[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { lo[i] = r[i]; hi[i] = r[16 + i]; }
  tmem_st_32x16(taddr, lo);
  tmem_st_32x16(taddr + 16, hi);
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Maximum of 32 score columns [col0, col0 + 32) of row r; MASKED applies the causal condition col <= r.
// Four independent chains of three-input maxima: 16 instructions, dependent depth 5.
template <bool MASKED>
__device__ __forceinline__ float chunk_row_max(const uint32_t (&sv)[32], int col0, int r) {
  float acc[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int i = 0; i < 32; i += 8) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int i0 = i + 2 * c, i1 = i0 + 1;
      const float a = (!MASKED || (col0 + i0) <= r) ? __uint_as_float(sv[i0]) : -INFINITY;
      const float b = (!MASKED || (col0 + i1) <= r) ? __uint_as_float(sv[i1]) : -INFINITY;
      acc[c] = max3(acc[c], a, b);
    }
  }
  return max3(fmaxf(acc[0], acc[1]), acc[2], acc[3]);
}

// 2^x on the FMA and integer pipes: x = n + f with n the nearest integer and f in [-0.5, 0.5]; 2^f from a
// cubic (relative error below 7e-4, a sixth of a bf16 ulp, and P is rounded to bf16 right after);
// 2^n by adding n to the exponent field.  Adding 1.5 * 2^23 puts n into the low mantissa bits of t,
// so shifting t left by 23 moves exactly those bits onto the exponent.  The MUFU unit computes 16
// exponentials per cycle and SM, the same time as the tile's two MMAs take; sending a share of the
// exponentials here takes the softmax off that limit.
constexpr int POLY_EXP2_OF_4 = TFT_ATTN_POLY_OF_4;  // how many of every four exponentials go this way
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -126.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(f, 0.0555041f, 0.2402265f);
  p = fmaf(p, f, 0.6931472f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
// exp2(s * scale - m) for the 32 score columns of chunk c, packed to bf16 and stored as P into the 16
// tensor-memory columns [c * 16, c * 16 + 16) of the tile's score region; returns the chunk's row sum.
template <bool MASKED>
__device__ __forceinline__ float chunk_softmax(const uint32_t (&sv)[32], int c, int r, float scale_log2, float m,
                                               uint32_t s_addr) {
  uint32_t packed[16];
  float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float x0 = __uint_as_float(sv[2 * i]) * scale_log2 - m;
    const float x1 = __uint_as_float(sv[2 * i + 1]) * scale_log2 - m;
    // columns 4k .. 4k+3: the first POLY_EXP2_OF_4 of them on the FMA pipe, the others on MUFU
    float e0 = ((2 * i) & 3) < POLY_EXP2_OF_4 ? poly_exp2(x0) : fast_exp2(x0);
    float e1 = ((2 * i + 1) & 3) < POLY_EXP2_OF_4 ? poly_exp2(x1) : fast_exp2(x1);
    if (MASKED) {
      if (c * 32 + 2 * i > r) e0 = 0.f;
      if (c * 32 + 2 * i + 1 > r) e1 = 0.f;
    }
    sum0 += e0;
    sum1 += e1;
    packed[i] = pack_bf16(e0, e1);
  }
  tmem_st_32x16(s_addr + c * 16, packed);
  return sum0 + sum1;
}

template <int HD>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
attn_fwd_pair_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                     const __grid_constant__ CUtensorMap tv, __nv_bfloat16* __restrict__ O, float* __restrict__ LSE,
                     int S, int Hq, int Hkv, long long ldo, float scale_log2, int* status) {
  using L = PairSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_PAIR_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_PAIR_BARS + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (S + BLK - 1) / BLK;
  const int n_pairs = (n_qtiles + 1) / 2;
  const int pair = n_pairs - 1 - blockIdx.x / Hq;  // heaviest pairs first, over all heads
  const int head = blockIdx.x % Hq, batch = blockIdx.y;
  const int kv_head = head / (Hq / Hkv);
  const int qt_a = 2 * pair, qt_b = 2 * pair + 1;
  const bool has_b = qt_b < n_qtiles;
  const int n_a = qt_a + 1;               // key tiles of tile A
  const int n_b = has_b ? qt_b + 1 : 0;   // key tiles of tile B
  const int n_steps = has_b ? n_b : n_a;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_PAIR_BARS; ++i) mbar_init(bar(i), (i >= PP_LO_A && i <= PP_HI_B) ? 128 : 1);
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
  // scores (and P) of tile t: 128 columns at t * 128; output accumulators behind them
  auto tmem_s = [&](int t) { return tmem_base + static_cast<uint32_t>(t) * 128u; };
  auto tmem_o = [&](int t) { return tmem_base + 256u + static_cast<uint32_t>(t) * HD; };

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(PQ_FULL), L::TILE * (has_b ? 2u : 1u));
      load_tile<HD>(base + L::Q, &tq, bar(PQ_FULL), head, qt_a * BLK, batch);
      if (has_b) load_tile<HD>(base + L::Q + L::TILE, &tq, bar(PQ_FULL), head, qt_b * BLK, batch);
      for (int j = 0; j < n_steps; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(PK_EMPTY0 + st), par, abort_flag)) break;
        mbar_expect_tx(bar(PK_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::K + st * L::TILE, &tk, bar(PK_FULL0 + st), kv_head, j * BLK, batch);
        if (!mbar_wait(bar(PV_EMPTY0 + st), par, abort_flag)) break;
        mbar_expect_tx(bar(PV_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::V + st * L::TILE, &tv, bar(PV_FULL0 + st), kv_head, j * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BLK, HD, false, true);
      auto issue_s = [&](int t, int j) {
        const int st = j & 1;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(tmem_s(t), kmajor_desc(base + L::Q + t * L::TILE, k), kmajor_desc(base + L::K + st * L::TILE, k),
                    idesc_s, k != 0);
        umma_commit(bar(PS_FULL_A + t));
      };
      // the PV product over keys [64 half, 64 half + 64) of the tile: 16 keys per step = 8 packed columns of P
      auto issue_pv = [&](int t, int j, int half) {
        const int st = j & 1;
#pragma unroll
        for (int kk = 0; kk < BLK / 32; ++kk) {
          const int k = half * (BLK / 32) + kk;
          umma_bf16_ts(tmem_o(t), tmem_s(t) + k * 8, mnmajor_desc(base + L::V + st * L::TILE, k), idesc_pv,
                       (j > 0 || k > 0) ? 1u : 0u);
        }
      };
      // P of the first 64 keys is ready before the exponentials of the last 64 are: start on it
      auto wait_issue_pv = [&](int t, int j) {
        if (!mbar_wait(bar(PP_LO_A + t), j & 1, abort_flag)) return false;
        tc_fence_after();
        issue_pv(t, j, 0);
        if (!mbar_wait(bar(PP_HI_A + t), j & 1, abort_flag)) return false;
        tc_fence_after();
        issue_pv(t, j, 1);
        return true;
      };
      bool ok = mbar_wait(bar(PQ_FULL), 0, abort_flag) && mbar_wait(bar(PK_FULL0), 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        if (has_b) issue_s(1, 0);
        umma_commit(bar(PK_EMPTY0));
      }
      for (int j = 0; j < n_steps && ok; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar(PV_FULL0 + st), (j >> 1) & 1, abort_flag)) { ok = false; break; }
        if (j < n_a) {
          if (!wait_issue_pv(0, j)) { ok = false; break; }
          if (j == n_a - 1) umma_commit(bar(PO_FULL_A));
        }
        const bool have_next = j + 1 < n_steps;
        if (have_next) {
          if (!mbar_wait(bar(PK_FULL0 + ((j + 1) & 1)), ((j + 1) >> 1) & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
        }
        if (j + 1 < n_a) issue_s(0, j + 1);
        if (j < n_b) {
          if (!wait_issue_pv(1, j)) { ok = false; break; }
          if (j == n_b - 1) umma_commit(bar(PO_FULL_B));
        }
        umma_commit(bar(PV_EMPTY0 + st));
        if (j + 1 < n_b) issue_s(1, j + 1);
        if (have_next) umma_commit(bar(PK_EMPTY0 + ((j + 1) & 1)));
      }
    }
  } else {
    const int t = (warp - 2) >> 2;   // 0: tile A, 1: tile B
    const int q = warp & 3;          // tensor-memory lane quarter of this warp
    const int r = q * 32 + lane;     // row inside the tile
    const int qt = t == 0 ? qt_a : qt_b;
    const int row = qt * BLK + r;    // row inside the sequence
    const int n_kv = t == 0 ? n_a : n_b;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t s_addr = tmem_s(t) + lane_addr;
    const uint32_t o_addr = tmem_o(t) + lane_addr;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const bool got = mbar_wait(bar(PS_FULL_A + t), j & 1, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }  // warp-uniform: tcgen05.ld/st are warp-wide
      tc_fence_after();
      const bool diag = (j == qt);
      // ---- the whole score row of this thread in registers: four loads in flight, one wait
      uint32_t s0[32], s1[32], s2[32], s3[32];
      tmem_ld_32x32(s_addr, s0);
      tmem_ld_32x32(s_addr + 32, s1);
      tmem_ld_32x32(s_addr + 64, s2);
      tmem_ld_32x32(s_addr + 96, s3);
      tmem_ld_wait();
      float mx;
      if (diag) {
        mx = fmaxf(fmaxf(chunk_row_max<true>(s0, 0, r), chunk_row_max<true>(s1, 32, r)),
                   fmaxf(chunk_row_max<true>(s2, 64, r), chunk_row_max<true>(s3, 96, r)));
      } else {
        mx = fmaxf(fmaxf(chunk_row_max<false>(s0, 0, r), chunk_row_max<false>(s1, 32, r)),
                   fmaxf(chunk_row_max<false>(s2, 64, r), chunk_row_max<false>(s3, 96, r)));
      }
      const float m_true = fmaxf(m, mx * scale_log2);
      if (j == 0) {
        m = m_true;  // nothing accumulated yet: PV(0) overwrites O
      } else {
        const bool raise = (m_true - m) > LAZY_RESCALE_LOG2;
        if (__any_sync(0xffffffffu, raise)) {
          const float alpha = raise ? fast_exp2(m - m_true) : 1.f;
          if (raise) m = m_true;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t ov[32];
            tmem_ld_32x32(o_addr + c * 32, ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, ov);
          }
          tmem_st_wait();
        }
      }
      // ---- exponentials, row sum, P (bf16, packed two per column) over the score columns just read
      float part[4];
      if (diag) {
        part[0] = chunk_softmax<true>(s0, 0, r, scale_log2, m, s_addr);
        part[1] = chunk_softmax<true>(s1, 1, r, scale_log2, m, s_addr);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar(PP_LO_A + t));
        part[2] = chunk_softmax<true>(s2, 2, r, scale_log2, m, s_addr);
        part[3] = chunk_softmax<true>(s3, 3, r, scale_log2, m, s_addr);
      } else {
        part[0] = chunk_softmax<false>(s0, 0, r, scale_log2, m, s_addr);
        part[1] = chunk_softmax<false>(s1, 1, r, scale_log2, m, s_addr);
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar(PP_LO_A + t));
        part[2] = chunk_softmax<false>(s2, 2, r, scale_log2, m, s_addr);
        part[3] = chunk_softmax<false>(s3, 3, r, scale_log2, m, s_addr);
      }
      l += (part[0] + part[1]) + (part[2] + part[3]);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(PP_HI_A + t));
    }
    if (ok && n_kv > 0) {
      const bool got = mbar_wait(bar(PO_FULL_A + t), 0, abort_flag);
      if (__all_sync(0xffffffffu, got)) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* dst = O + (static_cast<long long>(batch) * S + row) * ldo + head * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t ov[32];
          tmem_ld_32x32(o_addr + c * 32, ov);
          tmem_ld_wait();
          if (row < S) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 u;
              u.x = pack_bf16(__uint_as_float(ov[g * 8 + 0]) * inv, __uint_as_float(ov[g * 8 + 1]) * inv);
              u.y = pack_bf16(__uint_as_float(ov[g * 8 + 2]) * inv, __uint_as_float(ov[g * 8 + 3]) * inv);
              u.z = pack_bf16(__uint_as_float(ov[g * 8 + 4]) * inv, __uint_as_float(ov[g * 8 + 5]) * inv);
              u.w = pack_bf16(__uint_as_float(ov[g * 8 + 6]) * inv, __uint_as_float(ov[g * 8 + 7]) * inv);
              reinterpret_cast<uint4*>(dst + c * 32)[g] = u;
            }
          }
        }
        if (row < S) LSE[(static_cast<long long>(batch) * Hq + head) * S + row] = m + log2f(l);
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
int launch_fwd_pair(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq, int Hkv,
                    long long ldq, long long ldk, long long ldv, long long ldo, float scale, int* status,
                    cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (!make_attn_tensormap(&tq, q, HD, Hq, S, B, ldq)) return -2;
  if (!make_attn_tensormap(&tk, k, HD, Hkv, S, B, ldk)) return -3;
  if (!make_attn_tensormap(&tv, v, HD, Hkv, S, B, ldv)) return -4;
  auto kfn = attn_fwd_pair_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaGetLastError();
  const int n_qtiles = (S + BLK - 1) / BLK;
  dim3 grid(((n_qtiles + 1) / 2) * Hq, B, 1);
  kfn<<<grid, PAIR_THREADS, PairSmem<HD>::TOTAL, stream>>>(tq, tk, tv, static_cast<__nv_bfloat16*>(o), lse, S, Hq, Hkv,
                                                           ldo, scale * 1.4426950408889634f, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace attn
}  // namespace tft

// Same contract as tft_attn_fwd (attention_fwd.cu); two query tiles per CTA.  scale must be positive.
TFT_API int tft_attn_fwd_pair(const void* q, const void* k, const void* v, void* o, float* lse, int B, int S, int Hq,
                              int Hkv, int hd, int ldq, int ldk, int ldv, float scale, int* status,
                              cudaStream_t stream) {
  using namespace tft::attn;
  if (Hq % Hkv || (ldq % 8) || (ldk % 8) || (ldv % 8) || !(scale > 0.f)) return -1;
  const long long ldo = static_cast<long long>(Hq) * hd;
  if (hd == 128) return launch_fwd_pair<128>(q, k, v, o, lse, B, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, status, stream);
  if (hd == 64) return launch_fwd_pair<64>(q, k, v, o, lse, B, S, Hq, Hkv, ldq, ldk, ldv, ldo, scale, status, stream);
  return -1;
}
