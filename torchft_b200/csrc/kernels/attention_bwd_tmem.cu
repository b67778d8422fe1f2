// Causal grouped-query flash attention, backward, with P and dS kept in tensor memory.
//
// Same three-kernel split and the same contract as attention_bwd.cu (delta, dK/dV, dQ); what changes
// is where the softmax threads put their results.  There P and dS go to shared memory as swizzled bf16
// tiles, which costs a shared-memory write pass, an async-proxy fence and a serialising "buffer free"
// handshake per operand.  Here they are written with tcgen05.st over the fp32 values they were
// computed from and consumed by the gradient MMAs as the A operand FROM tensor memory:
//
//   attn_dq_tmem_kernel     one CTA per (query tile, head).  S = Q K_j^T alternates between two score
//                           regions, dP = dO V_j^T has one.  The softmax threads pull both into
//                           registers (all loads in flight, one wait), report that (the dP region is
//                           then free for tile j+1), form dS = P (dP - delta) and store it, packed,
//                           into the score region they read S from.  dQ += dS K_j takes A = dS from
//                           tensor memory.  The MMAs of tile j+1 run under the softmax of tile j.
//   attn_dkdv_tmem_kernel   one CTA per (key tile, kv head), transposed: S^T = K Q_i^T and
//                           dP^T = V dO_i^T put the KEY rows on the tensor-memory lanes, so P^T and
//                           dS^T come out in the layout that dV += P^T dO_i and dK += dS^T Q_i need as
//                           A operands.  The row statistics (log-sum-exp and delta) are then per
//                           COLUMN; every item's 2 x 128 values are staged in shared memory.  Items
//                           are cut into halves of 64 query columns that alternate between two sets
//                           of score regions, so the softmax of one half runs under the MMAs of the
//                           neighbouring ones.
//
// A thread overwrites only tensor-memory columns it has read itself (each of the two threads of a row
// packs its 64 values into the first 32 columns of its own 64-column half), so no thread can clobber
// a value another warp still needs.  Waits are bounded as everywhere (common.cuh).
#include "attention_common.cuh"

namespace tft {
namespace attn {

// dS (or P) of 32 score columns as 16 packed bf16 pairs.
__device__ __forceinline__ void pack32(const float (&v)[32], uint32_t (&out)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) out[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
}

// Tensor-memory column of k-step `k` (16 contraction indices = 8 packed columns) of an A operand that
// the two threads of a row wrote into the first 32 columns of their own 64-column halves.
__device__ __forceinline__ uint32_t packed_kstep(uint32_t region, int k) {
  return region + (k < 4 ? k * 8 : 64 + (k - 4) * 8);
}

// ------------------------------------------------------------------ dQ
template <int HD>
struct DqTmemSmem {
  static constexpr int KSTAGES = 3, VSTAGES = 2;
  static constexpr uint32_t TILE = BLK * HD * 2;
  static constexpr uint32_t Q = 0, DO = TILE, K = 2 * TILE, V = K + KSTAGES * TILE;
  static constexpr uint32_t BARS = V + VSTAGES * TILE;
  static constexpr uint32_t TOTAL = BARS + 256 + 1024;
};
enum DqTmemBar {
  TQ_QDO_FULL = 0, TQ_K_FULL0, TQ_K_FULL1, TQ_K_FULL2, TQ_K_EMPTY0, TQ_K_EMPTY1, TQ_K_EMPTY2, TQ_V_FULL0, TQ_V_FULL1,
  TQ_V_EMPTY0, TQ_V_EMPTY1, TQ_SDP_FULL, TQ_LOADED, TQ_DS_READY, TQ_DONE, NUM_TQ_BARS
};

template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_dq_tmem_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                    const float* __restrict__ LSE, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dQ,
                    int S, int Hq, int Hkv, long long lddq, float scale, float scale_log2, int* status) {
  using L = DqTmemSmem<HD>;
  constexpr int KS = L::KSTAGES, VS = L::VSTAGES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_TQ_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_TQ_BARS + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (S + BLK - 1) / BLK;
  const int qt = n_tiles - 1 - blockIdx.x / Hq;  // heaviest first over all heads
  const int head = blockIdx.x % Hq, batch = blockIdx.y;
  const int kv_head = head / (Hq / Hkv);
  const int n_kv = qt + 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_TQ_BARS; ++i) mbar_init(bar(i), (i == TQ_LOADED || i == TQ_DS_READY) ? 256 : 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
    tma_prefetch_desc(&tdo);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  auto t_s = [&](int j) { return tmem_base + static_cast<uint32_t>(j & 1) * 128u; };  // scores, later dS, of tile j
  const uint32_t t_dp = tmem_base + 256, t_dq = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(TQ_QDO_FULL), 2 * L::TILE);
      load_tile<HD>(base + L::Q, &tq, bar(TQ_QDO_FULL), head, qt * BLK, batch);
      load_tile<HD>(base + L::DO, &tdo, bar(TQ_QDO_FULL), head, qt * BLK, batch);
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % KS, vs = j % VS;
        if (!mbar_wait(bar(TQ_K_EMPTY0 + ks), ((j / KS) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(TQ_K_FULL0 + ks), L::TILE);
        load_tile<HD>(base + L::K + ks * L::TILE, &tk, bar(TQ_K_FULL0 + ks), kv_head, j * BLK, batch);
        if (!mbar_wait(bar(TQ_V_EMPTY0 + vs), ((j / VS) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(TQ_V_FULL0 + vs), L::TILE);
        load_tile<HD>(base + L::V + vs * L::TILE, &tv, bar(TQ_V_FULL0 + vs), kv_head, j * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_q = make_idesc_bf16(BLK, HD, false, true);
      auto issue_s = [&](int j) -> bool {  // S(j) = Q K_j^T into the score region of tile j
        const int ks = j % KS;
        if (!mbar_wait(bar(TQ_K_FULL0 + ks), (j / KS) & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(t_s(j), kmajor_desc(base + L::Q, k), kmajor_desc(base + L::K + ks * L::TILE, k), idesc_s, k != 0);
        return true;
      };
      auto issue_dp = [&](int j) -> bool {  // dP(j) = dO V_j^T; with it the inputs of softmax(j) are complete
        const int vs = j % VS;
        if (!mbar_wait(bar(TQ_V_FULL0 + vs), (j / VS) & 1, abort_flag)) return false;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_bf16(t_dp, kmajor_desc(base + L::DO, k), kmajor_desc(base + L::V + vs * L::TILE, k), idesc_s, k != 0);
        umma_commit(bar(TQ_SDP_FULL));
        umma_commit(bar(TQ_V_EMPTY0 + vs));
        return true;
      };
      bool ok = mbar_wait(bar(TQ_QDO_FULL), 0, abort_flag);
      if (ok) ok = issue_s(0) && issue_dp(0);
      if (ok && n_kv > 1) ok = issue_s(1);
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          // the softmax threads hold S(j) and dP(j) in registers: the dP region may be overwritten
          if (!mbar_wait(bar(TQ_LOADED), j & 1, abort_flag)) { ok = false; break; }
          if (!issue_dp(j + 1)) { ok = false; break; }
        }
        if (!mbar_wait(bar(TQ_DS_READY), j & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dQ += dS K_j   (contraction over the 128 key rows; A = dS from tensor memory)
        const uint32_t sk = base + L::K + (j % KS) * L::TILE;
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_bf16_ts(t_dq, packed_kstep(t_s(j), k), mnmajor_desc(sk, k), idesc_q, (j | k) != 0);
        umma_commit(bar(TQ_K_EMPTY0 + (j % KS)));
        // the score region of tile j is free again once those MMAs have run (in order): tile j+2 goes there
        if (j + 2 < n_kv && !issue_s(j + 2)) { ok = false; break; }
      }
      if (ok) umma_commit(bar(TQ_DONE));
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;  // two threads per row: key columns [0,64) and [64,128)
    const int r = q * 32 + lane;
    const int row = qt * BLK + r;
    const bool row_ok = row < S;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const long long stat = (static_cast<long long>(batch) * Hq + head) * S + row;
    const float lse = row_ok ? LSE[stat] : 0.f;
    const float dl = row_ok ? delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const bool got = mbar_wait(bar(TQ_SDP_FULL), j & 1, abort_flag);
      if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (j == qt);
      const uint32_t my_s = t_s(j) + lane_addr + half * 64;
      uint32_t sv[2][32], dv[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_32x32(my_s + cc * 32, sv[cc]);
        tmem_ld_32x32(t_dp + lane_addr + half * 64 + cc * 32, dv[cc]);
      }
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(bar(TQ_LOADED));
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c0 = half * 64 + cc * 32;
        float ds[32];
        if (diag || !row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool keep = row_ok && (c0 + i) <= r;
            const float p = keep ? fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse) : 0.f;
            ds[i] = p * (__uint_as_float(dv[cc][i]) - dl);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p = fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse);
            ds[i] = p * (__uint_as_float(dv[cc][i]) - dl);
          }
        }
        uint32_t packed[16];
        pack32(ds, packed);
        tmem_st_32x16(my_s + cc * 16, packed);  // over score columns this thread has already read
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(TQ_DS_READY));
    }
    if (ok) {
      const bool done = mbar_wait(bar(TQ_DONE), 0, abort_flag);
      if (__all_sync(0xffffffffu, done)) {
        tc_fence_after();
        const long long tok = static_cast<long long>(batch) * S + row;
        store_acc<HD / 2>(t_dq + lane_addr + half * (HD / 2), dQ + tok * lddq + head * HD + half * (HD / 2), scale, row_ok);
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
int launch_dq_tmem(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                   const float* lse, const float* delta, void* dq, int B, int S, int Hq, int Hkv, long long lddq,
                   float scale, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_dq_tmem_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DqTmemSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int n_tiles = (S + BLK - 1) / BLK;
  attn_dq_tmem_kernel<HD><<<dim3(n_tiles * Hq, B, 1), 320, DqTmemSmem<HD>::TOTAL, stream>>>(
      tq, tk, tv, tdo, lse, delta, static_cast<__nv_bfloat16*>(dq), S, Hq, Hkv, lddq, scale,
      scale * 1.4426950408889634f, status);
  return static_cast<int>(cudaGetLastError());
}

// ------------------------------------------------------------------ dK, dV (transposed scores)
// An item (one query head of the group x one query tile) is processed as two HALF ITEMS of 64 query
// columns.  Each half item has its own pair of 64-column score regions, so while the softmax threads
// work on one half item the tensor cores run the gradient products of the previous one and the score
// products of the next: the ping-pong that a full item, which would fill the score regions alone,
// cannot have next to two 128-column accumulators.
template <int HD>
struct DkvTmemSmem {
  static constexpr uint32_t TILE = BLK * HD * 2;
  static constexpr uint32_t K = 0, V = TILE, Q = 2 * TILE /*2 stages*/, DO = 4 * TILE /*2 stages*/;
  static constexpr uint32_t STATS = 6 * TILE;  // float [2 buffers][lse 128 | delta 128]
  static constexpr uint32_t BARS = STATS + 2 * 2 * BLK * 4;
  static constexpr uint32_t TOTAL = BARS + 256 + 1024;
};
enum DkvTmemBar {
  TK_KV_FULL = 0, TK_Q_FULL0, TK_Q_FULL1, TK_DO_FULL0, TK_DO_FULL1, TK_Q_EMPTY0, TK_Q_EMPTY1, TK_DO_EMPTY0, TK_DO_EMPTY1,
  TK_SDP_FULL0, TK_SDP_FULL1, TK_PDS_READY0, TK_PDS_READY1, TK_ACC_DONE, NUM_TK_BARS
};

// Column of k-step kk (16 of a half item's 64 query columns) inside a 64-column region whose two
// threads per row each packed their 32 values into the first 16 columns of their own 32-column half.
__device__ __forceinline__ uint32_t half_item_kstep(uint32_t region, int kk) {
  return region + (kk < 2 ? kk * 8 : 32 + (kk - 2) * 8);
}

template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_dkdv_tmem_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                      const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                      const float* __restrict__ LSE, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK,
                      __nv_bfloat16* __restrict__ dV, int S, int Hq, int Hkv, long long lddk, long long lddv, float scale,
                      float scale_log2, int* status) {
  using L = DkvTmemSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_TK_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_TK_BARS + 8);
  float* stats = reinterpret_cast<float*>(smem + L::STATS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (S + BLK - 1) / BLK;
  const int jt = blockIdx.x / Hkv;  // key tile; early key tiles have the most work and come first
  const int kv_head = blockIdx.x % Hkv, batch = blockIdx.y;
  const int G = Hq / Hkv;
  const int per_head = n_tiles - jt;
  const int n_items = G * per_head;  // (query head of the group, query tile at or after the key tile)
  const int n_halves = 2 * n_items;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_TK_BARS; ++i) mbar_init(bar(i), (i == TK_PDS_READY0 || i == TK_PDS_READY1) ? 256 : 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tq);
    tma_prefetch_desc(&tk);
    tma_prefetch_desc(&tv);
    tma_prefetch_desc(&tdo);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // region set x of half item hh (x = hh & 1): S^T (later P^T) at x * 128, dP^T (later dS^T) at x * 128 + 64;
  // key rows on the lanes everywhere
  auto t_st = [&](int hh) { return tmem_base + static_cast<uint32_t>(hh & 1) * 128u; };
  auto t_dpt = [&](int hh) { return tmem_base + static_cast<uint32_t>(hh & 1) * 128u + 64u; };
  const uint32_t t_dv = tmem_base + 256, t_dk = tmem_base + 256 + HD;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(TK_KV_FULL), 2 * L::TILE);
      load_tile<HD>(base + L::K, &tk, bar(TK_KV_FULL), kv_head, jt * BLK, batch);
      load_tile<HD>(base + L::V, &tv, bar(TK_KV_FULL), kv_head, jt * BLK, batch);
      for (int t = 0; t < n_items; ++t) {
        const int head = kv_head * G + t / per_head;
        const int it = jt + t % per_head;
        const int st = t & 1;
        const uint32_t free_parity = ((t >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(TK_Q_EMPTY0 + st), free_parity, abort_flag)) break;
        mbar_expect_tx(bar(TK_Q_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::Q + st * L::TILE, &tq, bar(TK_Q_FULL0 + st), head, it * BLK, batch);
        if (!mbar_wait(bar(TK_DO_EMPTY0 + st), free_parity, abort_flag)) break;
        mbar_expect_tx(bar(TK_DO_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::DO + st * L::TILE, &tdo, bar(TK_DO_FULL0 + st), head, it * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, 64, false, false);   // 128 keys x 64 queries
      constexpr uint32_t idesc_g = make_idesc_bf16(BLK, HD, false, true);
      // S^T = K Q^T and dP^T = V dO^T for the 64 query rows of half item hh: the key tile is the A
      // operand (keys land on the lanes); the B operand is rows [64 s, 64 s + 64) of the item's Q / dO tile
      auto issue_sdp = [&](int hh) -> bool {
        const int t = hh >> 1, s = hh & 1, st = t & 1;
        if (s == 0) {  // first half of an item: its Q / dO stage must have landed
          const uint32_t ph = (t >> 1) & 1;
          if (!mbar_wait(bar(TK_Q_FULL0 + st), ph, abort_flag) || !mbar_wait(bar(TK_DO_FULL0 + st), ph, abort_flag)) return false;
          tc_fence_after();
        }
        const uint32_t sq = base + L::Q + st * L::TILE + s * 8192, sdo = base + L::DO + st * L::TILE + s * 8192;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_st(hh), kmajor_desc(base + L::K, k), kmajor_desc(sq, k), idesc_s, k != 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_dpt(hh), kmajor_desc(base + L::V, k), kmajor_desc(sdo, k), idesc_s, k != 0);
        umma_commit(bar(TK_SDP_FULL0 + (hh & 1)));
        return true;
      };
      bool ok = mbar_wait(bar(TK_KV_FULL), 0, abort_flag);
      if (ok && n_halves > 0) ok = issue_sdp(0) && issue_sdp(1);
      for (int hh = 0; hh < n_halves && ok; ++hh) {
        const int t = hh >> 1, s = hh & 1, st = t & 1;
        const uint32_t sq = base + L::Q + st * L::TILE, sdo = base + L::DO + st * L::TILE;
        if (!mbar_wait(bar(TK_PDS_READY0 + (hh & 1)), (hh >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dV += P^T dO and dK += dS^T Q over this half item's 64 query rows: A from tensor memory
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(t_dv, half_item_kstep(t_st(hh), kk), mnmajor_desc(sdo, 4 * s + kk), idesc_g, (hh | kk) != 0);
        if (s == 1) umma_commit(bar(TK_DO_EMPTY0 + st));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts(t_dk, half_item_kstep(t_dpt(hh), kk), mnmajor_desc(sq, 4 * s + kk), idesc_g, (hh | kk) != 0);
        if (s == 1) umma_commit(bar(TK_Q_EMPTY0 + st));
        // in order behind them: the scores of half item hh + 2 go into the regions just consumed
        if (hh + 2 < n_halves && !issue_sdp(hh + 2)) { ok = false; break; }
      }
      if (ok) umma_commit(bar(TK_ACC_DONE));
    }
  } else {
    const int q = warp & 3;
    const int hf = (warp - 2) >> 2;    // two threads per key row: columns [0,32) and [32,64) of the half item
    const int r = q * 32 + lane;       // key row inside the tile
    const int e = (warp - 2) * 32 + lane;  // 0..255: which statistic this thread fetches per item
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    // statistic of item t for this thread's slot: log-sum-exp (slots 0..127) or delta (128..255) of one
    // query row; +inf as log-sum-exp of a row beyond the sequence turns its probabilities into zeros
    auto fetch_stat = [&](int t) -> float {
      const int head = kv_head * G + t / per_head;
      const int qrow = (jt + t % per_head) * BLK + (e & 127);
      const long long at = (static_cast<long long>(batch) * Hq + head) * S + qrow;
      if (e < 128) return qrow < S ? LSE[at] : INFINITY;
      return qrow < S ? delta[at] : 0.f;
    };
    float next_stat = n_items > 0 ? fetch_stat(0) : 0.f;
    for (int hh = 0; hh < n_halves; ++hh) {
      const int t = hh >> 1, s = hh & 1;
      const int it = jt + t % per_head;
      float* my_stats = stats + (t & 1) * 2 * BLK;
      if (s == 0) {
        my_stats[e] = next_stat;
        if (t + 1 < n_items) next_stat = fetch_stat(t + 1);  // travels while this item is processed
      }
      const bool got = mbar_wait(bar(TK_SDP_FULL0 + (hh & 1)), (hh >> 1) & 1, abort_flag);
      if (s == 0) {
        asm volatile("bar.sync 1, 256;" ::: "memory");  // every statistic of this item is in shared memory
        if (*abort_flag) { ok = false; break; }  // uniform: whoever gave up set the flag before the barrier
      } else if (!__all_sync(0xffffffffu, got)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool diag = (it == jt);
      const int c0 = s * 64 + hf * 32;  // first query column (inside the tile) of this thread's 32
      const uint32_t my_st = t_st(hh) + lane_addr + hf * 32, my_dpt = t_dpt(hh) + lane_addr + hf * 32;
      uint32_t sv[32], dv[32];
      tmem_ld_32x32(my_st, sv);
      tmem_ld_32x32(my_dpt, dv);
      tmem_ld_wait();
      float p[32], ds[32];
#pragma unroll
      for (int i4 = 0; i4 < 8; ++i4) {
        const float4 ls = *reinterpret_cast<const float4*>(my_stats + c0 + i4 * 4);
        const float4 dl = *reinterpret_cast<const float4*>(my_stats + BLK + c0 + i4 * 4);
        const float lsv[4] = {ls.x, ls.y, ls.z, ls.w}, dlv[4] = {dl.x, dl.y, dl.z, dl.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i4 * 4 + u;
          float pv = fast_exp2(__uint_as_float(sv[i]) * scale_log2 - lsv[u]);
          if (diag && (c0 + i) < r) pv = 0.f;  // causal: query column >= key row
          p[i] = pv;
          ds[i] = pv * (__uint_as_float(dv[i]) - dlv[u]);
        }
      }
      uint32_t packed[16];
      pack32(p, packed);
      tmem_st_32x16(my_st, packed);   // over score columns this thread has already read
      pack32(ds, packed);
      tmem_st_32x16(my_dpt, packed);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar(TK_PDS_READY0 + (hh & 1)));
    }
    if (ok && n_items > 0) {
      const bool done = mbar_wait(bar(TK_ACC_DONE), 0, abort_flag);
      if (__all_sync(0xffffffffu, done)) {
        tc_fence_after();
        const int krow = jt * BLK + r;
        const long long tok = static_cast<long long>(batch) * S + krow;
        store_acc<HD / 2>(t_dv + lane_addr + hf * (HD / 2), dV + tok * lddv + kv_head * HD + hf * (HD / 2), 1.f, krow < S);
        store_acc<HD / 2>(t_dk + lane_addr + hf * (HD / 2), dK + tok * lddk + kv_head * HD + hf * (HD / 2), scale, krow < S);
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
int launch_dkdv_tmem(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                     const float* lse, const float* delta, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                     long long lddk, long long lddv, float scale, int* status, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_dkdv_tmem_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DkvTmemSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int n_tiles = (S + BLK - 1) / BLK;
  attn_dkdv_tmem_kernel<HD><<<dim3(n_tiles * Hkv, B, 1), 320, DkvTmemSmem<HD>::TOTAL, stream>>>(
      tq, tk, tv, tdo, lse, delta, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), S, Hq, Hkv, lddk,
      lddv, scale, scale * 1.4426950408889634f, status);
  return static_cast<int>(cudaGetLastError());
}

template <int HD>
int launch_bwd_tmem(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
                    float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, long long ldq,
                    long long ldk, long long ldv, long long lddq, long long lddk, long long lddv, float scale, int* status,
                    cudaStream_t stream, int parts) {
  CUtensorMap tq, tk, tv, tdo;
  if (!make_attn_tensormap(&tq, q, HD, Hq, S, B, ldq)) return -2;
  if (!make_attn_tensormap(&tk, k, HD, Hkv, S, B, ldk)) return -3;
  if (!make_attn_tensormap(&tv, v, HD, Hkv, S, B, ldv)) return -4;
  if (!make_attn_tensormap(&tdo, dout, HD, Hq, S, B, static_cast<long long>(Hq) * HD)) return -5;
  cudaGetLastError();
  const long long warps = static_cast<long long>(B) * S * Hq;
  if (parts & 1)
    attn_delta_kernel<HD><<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), delta, B, S, Hq);
  int rc = 0;
  if (parts & 2) rc = launch_dkdv_tmem<HD>(tq, tk, tv, tdo, lse, delta, dk, dv, B, S, Hq, Hkv, lddk, lddv, scale, status, stream);
  if (rc == 0 && (parts & 4)) rc = launch_dq_tmem<HD>(tq, tk, tv, tdo, lse, delta, dq, B, S, Hq, Hkv, lddq, scale, status, stream);
  return rc;
}

}  // namespace attn
}  // namespace tft

// dQ alone (delta must have been computed): the dQ kernel of this file, for use behind the dK/dV kernel
// of attention_bwd.cu or of this file.  Arguments as the corresponding ones of tft_attn_bwd.
TFT_API int tft_attn_dq_tmem(const void* dout, const void* q, const void* k, const void* v, const float* lse,
                             const float* delta, void* dq, int B, int S, int Hq, int Hkv, int hd, int ldq, int ldk,
                             int ldv, int lddq, float scale, int* status, cudaStream_t stream) {
  using namespace tft::attn;
  if (Hq % Hkv || (ldq % 8) || (ldk % 8) || (ldv % 8) || (lddq % 8)) return -1;
  CUtensorMap tq, tk, tv, tdo;
  if (!make_attn_tensormap(&tq, q, hd, Hq, S, B, ldq)) return -2;
  if (!make_attn_tensormap(&tk, k, hd, Hkv, S, B, ldk)) return -3;
  if (!make_attn_tensormap(&tv, v, hd, Hkv, S, B, ldv)) return -4;
  if (!make_attn_tensormap(&tdo, dout, hd, Hq, S, B, static_cast<long long>(Hq) * hd)) return -5;
  cudaGetLastError();
  if (hd == 128) return launch_dq_tmem<128>(tq, tk, tv, tdo, lse, delta, dq, B, S, Hq, Hkv, lddq, scale, status, stream);
  if (hd == 64) return launch_dq_tmem<64>(tq, tk, tv, tdo, lse, delta, dq, B, S, Hq, Hkv, lddq, scale, status, stream);
  return -1;
}

// Causal attention backward with P and dS in tensor memory: same contract as tft_attn_bwd
// (attention_bwd.cu); parts = 1 (delta) | 2 (dK/dV) | 4 (dQ) selects kernels, 7 runs all three.
TFT_API int tft_attn_bwd_tmem(const void* dout, const void* q, const void* k, const void* v, const void* o,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq,
                              int Hkv, int hd, int ldq, int ldk, int ldv, int lddq, int lddk, int lddv, float scale,
                              int* status, cudaStream_t stream, int parts) {
  using namespace tft::attn;
  if (Hq % Hkv || (ldq % 8) || (ldk % 8) || (ldv % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -1;
  if (hd == 128)
    return launch_bwd_tmem<128>(dout, q, k, v, o, lse, delta, dq, dk, dv, B, S, Hq, Hkv, ldq, ldk, ldv, lddq, lddk, lddv,
                                scale, status, stream, parts);
  if (hd == 64)
    return launch_bwd_tmem<64>(dout, q, k, v, o, lse, delta, dq, dk, dv, B, S, Hq, Hkv, ldq, ldk, ldv, lddq, lddk, lddv,
                               scale, status, stream, parts);
  return -1;
}
