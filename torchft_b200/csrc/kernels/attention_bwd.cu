// Causal grouped-query flash attention, backward, on tcgen05 tensor cores.
//
// Three kernels:
//   attn_delta_kernel   delta[row] = sum_d O[row,d] * dO[row,d]
//   attn_dkdv_kernel    one CTA per (key tile, kv head): loops over the query heads of the
//                       group and the query tiles at or after the key tile; dK and dV stay
//                       in tensor memory for the whole loop (no atomics, deterministic)
//   attn_dq_kernel      one CTA per (query tile, head): loops over key tiles, dQ stays in
//                       tensor memory
//
// Per tile pair both kernels recompute S = Q K^T and dP = dO V^T with tcgen05.mma into
// tensor memory; the softmax threads (one per query row) form P = exp2(S*c - LSE) and
// dS = P * (dP - delta) and write them as bf16 into swizzled shared memory, from where
// they feed the gradient MMAs as MN-major (transposed) or K-major operands.
#include "attention_common.cuh"

namespace tft {
namespace attn {

// ------------------------------------------------------------------ dK, dV
// Q and dO tiles are double buffered.  P and dS share ONE operand buffer: P is written first
// and consumed by the dV MMAs, then dS (kept in registers meanwhile) overwrites it for the dK
// MMAs.  That is what makes room for the second Q/dO stage.
template <int HD>
struct DkvSmem {
  static constexpr uint32_t TILE = BLK * HD * 2;
  static constexpr uint32_t K = 0, V = TILE, Q = 2 * TILE /*2 stages*/, DO = 4 * TILE /*2 stages*/;
  static constexpr uint32_t PDS = 6 * TILE;
  static constexpr uint32_t BARS = PDS + BLK * BLK * 2;
  static constexpr uint32_t TOTAL = BARS + 256 + 1024;
};
enum DkvBar { KV_FULL = 0, Q_FULL0, Q_FULL1, DO_FULL0, DO_FULL1, Q_EMPTY0, Q_EMPTY1, DO_EMPTY0, DO_EMPTY1, SDP_FULL, P_READY, P_FREE, DS_READY, DS_FREE, ACC_DONE, NUM_DKV_BARS };

template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_dkdv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                 const float* __restrict__ LSE, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK,
                 __nv_bfloat16* __restrict__ dV, int S, int Hq, int Hkv, long long lddk, long long lddv,
                 float scale, float scale_log2, int* status) {
  using L = DkvSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_DKV_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_DKV_BARS + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (S + BLK - 1) / BLK;
  // Blocks are numbered heaviest first over ALL heads (longest-processing-time order), so the
  // hardware scheduler hands late SMs the short tiles instead of a long straggler.
  const int jt = blockIdx.x / Hkv;  // key tile; early key tiles have the most work
  const int kv_head = blockIdx.x % Hkv, batch = blockIdx.y;
  const int G = Hq / Hkv;
  const int per_head = n_tiles - jt;
  const int n_items = G * per_head;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_DKV_BARS; ++i) mbar_init(bar(i), (i == P_READY || i == DS_READY) ? 256 : 1);
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
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 256 + HD;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(KV_FULL), 2 * L::TILE);
      load_tile<HD>(base + L::K, &tk, bar(KV_FULL), kv_head, jt * BLK, batch);
      load_tile<HD>(base + L::V, &tv, bar(KV_FULL), kv_head, jt * BLK, batch);
      for (int t = 0; t < n_items; ++t) {
        const int head = kv_head * G + t / per_head;
        const int it = jt + t % per_head;
        const int st = t & 1;
        const uint32_t free_parity = ((t >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(Q_EMPTY0 + st), free_parity, abort_flag)) break;
        mbar_expect_tx(bar(Q_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::Q + st * L::TILE, &tq, bar(Q_FULL0 + st), head, it * BLK, batch);
        if (!mbar_wait(bar(DO_EMPTY0 + st), free_parity, abort_flag)) break;
        mbar_expect_tx(bar(DO_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::DO + st * L::TILE, &tdo, bar(DO_FULL0 + st), head, it * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_g = make_idesc_bf16(BLK, HD, true, true);
      // S = Q K^T and dP = dO V^T of item t (its Q/dO stage must have landed)
      auto issue_sdp = [&](int t) -> bool {
        const int st = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(bar(Q_FULL0 + st), ph, abort_flag) || !mbar_wait(bar(DO_FULL0 + st), ph, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sq = base + L::Q + st * L::TILE, sdo = base + L::DO + st * L::TILE;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_s, kmajor_desc(sq, k), kmajor_desc(base + L::K, k), idesc_s, k != 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_dp, kmajor_desc(sdo, k), kmajor_desc(base + L::V, k), idesc_s, k != 0);
        umma_commit(bar(SDP_FULL));
        return true;
      };
      bool ok = mbar_wait(bar(KV_FULL), 0, abort_flag);
      if (ok && n_items > 0) ok = issue_sdp(0);
      for (int t = 0; t < n_items && ok; ++t) {
        const int st = t & 1;
        const uint32_t sq = base + L::Q + st * L::TILE, sdo = base + L::DO + st * L::TILE;
        // P_READY also means: the softmax threads are done reading S and dP of item t
        if (!mbar_wait(bar(P_READY), t & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dV += P^T dO   (contraction over the 128 query rows)
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_bf16(t_dv, mnmajor_desc(base + L::PDS, k), mnmajor_desc(sdo, k), idesc_g, (t | k) != 0);
        umma_commit(bar(DO_EMPTY0 + st));
        umma_commit(bar(P_FREE));
        // scores of the NEXT item run while the softmax threads finish dS of this one
        if (t + 1 < n_items && !issue_sdp(t + 1)) { ok = false; break; }
        if (!mbar_wait(bar(DS_READY), t & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dK += dS^T Q
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_bf16(t_dk, mnmajor_desc(base + L::PDS, k), mnmajor_desc(sq, k), idesc_g, (t | k) != 0);
        umma_commit(bar(Q_EMPTY0 + st));
        umma_commit(bar(DS_FREE));
      }
      if (ok) umma_commit(bar(ACC_DONE));
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;  // two threads per row: columns [0,64) and [64,128)
    const int r = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    float next_lse = 0.f, next_dl = 0.f;
    if (n_items > 0) {
      const int row0 = jt * BLK + r;
      const long long stat0 = (static_cast<long long>(batch) * Hq + kv_head * G) * S + row0;
      next_lse = row0 < S ? LSE[stat0] : 0.f;
      next_dl = row0 < S ? delta[stat0] : 0.f;
    }
    for (int t = 0; t < n_items; ++t) {
      const int it = jt + t % per_head;
      const int row = it * BLK + r;
      const bool row_ok = row < S;
      const float lse = next_lse, dl = next_dl;
      if (t + 1 < n_items) {  // statistics of the next item travel while this one is processed
        const int nhead = kv_head * G + (t + 1) / per_head;
        const int nrow = (jt + (t + 1) % per_head) * BLK + r;
        const long long nstat = (static_cast<long long>(batch) * Hq + nhead) * S + nrow;
        next_lse = nrow < S ? LSE[nstat] : 0.f;
        next_dl = nrow < S ? delta[nstat] : 0.f;
      }
      if (!mbar_wait(bar(SDP_FULL), t & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (it == jt);
      float p[2][32], ds[2][32];
      // all four tensor-memory loads are issued before the single wait, so their latencies overlap
      uint32_t sv[2][32], dv[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_32x32(t_s + lane_addr + (half * 2 + cc) * 32, sv[cc]);
        tmem_ld_32x32(t_dp + lane_addr + (half * 2 + cc) * 32, dv[cc]);
      }
      tmem_ld_wait();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        if (diag || !row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool keep = row_ok && (c * 32 + i) <= r;
            p[cc][i] = keep ? fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse) : 0.f;
            ds[cc][i] = p[cc][i] * (__uint_as_float(dv[cc][i]) - dl);
          }
        } else {  // mask-free fast path: every tile off the diagonal
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            p[cc][i] = fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse);
            ds[cc][i] = p[cc][i] * (__uint_as_float(dv[cc][i]) - dl);
          }
        }
      }
      // the operand buffer is free once the dK MMAs of the previous item have read dS from it
      if (t > 0 && !mbar_wait(bar(DS_FREE), (t - 1) & 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) store_row_chunk(smem + L::PDS, r, half * 2 + cc, p[cc]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(bar(P_READY));
      // ... and dS may replace P once the dV MMAs have read it
      if (!mbar_wait(bar(P_FREE), t & 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) store_row_chunk(smem + L::PDS, r, half * 2 + cc, ds[cc]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(bar(DS_READY));
    }
    if (ok && mbar_wait(bar(ACC_DONE), 0, abort_flag)) {
      tc_fence_after();
      const int krow = jt * BLK + r;
      const long long tok = static_cast<long long>(batch) * S + krow;
      store_acc<HD / 2>(t_dv + lane_addr + half * (HD / 2), dV + tok * lddv + kv_head * HD + half * (HD / 2), 1.f, krow < S);
      store_acc<HD / 2>(t_dk + lane_addr + half * (HD / 2), dK + tok * lddk + kv_head * HD + half * (HD / 2), scale, krow < S);
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

// ------------------------------------------------------------------ dK, dV with separate S and dP pipelines
// Same tiles, buffers and results as attn_dkdv_kernel; what changes is the order of the products.
// There, S and dP of item t+1 are issued together behind dV(t), so the softmax threads of item t+1
// wait for dV(t) + S(t+1) + dP(t+1).  Here the score path is S only: the softmax threads load S, form P
// and hand it over, and S(t+1) follows dV(t) directly; dP(t+1) is issued behind dK(t), where nobody
// waits for it (it is needed only after P(t+1) has been stored), and is loaded in a second step to form
// dS.  Tensor-core order per item: dV(t), S(t+1), dK(t), dP(t+1).
enum DksBar {
  KS_KV_FULL = 0, KS_Q_FULL0, KS_Q_FULL1, KS_DO_FULL0, KS_DO_FULL1, KS_Q_EMPTY0, KS_Q_EMPTY1, KS_DO_EMPTY0, KS_DO_EMPTY1,
  KS_S_FULL, KS_DP_FULL, KS_P_READY, KS_P_FREE, KS_DS_READY, KS_DS_FREE, KS_ACC_DONE, NUM_DKS_BARS
};

template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_dkdv_split_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                 const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                 const float* __restrict__ LSE, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dK,
                 __nv_bfloat16* __restrict__ dV, int S, int Hq, int Hkv, long long lddk, long long lddv,
                 float scale, float scale_log2, int* status) {
  using L = DkvSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_DKS_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_DKS_BARS + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (S + BLK - 1) / BLK;
  // Blocks are numbered heaviest first over ALL heads (longest-processing-time order), so the
  // hardware scheduler hands late SMs the short tiles instead of a long straggler.
  const int jt = blockIdx.x / Hkv;  // key tile; early key tiles have the most work
  const int kv_head = blockIdx.x % Hkv, batch = blockIdx.y;
  const int G = Hq / Hkv;
  const int per_head = n_tiles - jt;
  const int n_items = G * per_head;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_DKS_BARS; ++i) mbar_init(bar(i), (i == KS_P_READY || i == KS_DS_READY) ? 8 : 1);  // one arrival per softmax warp
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
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 256 + HD;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(KS_KV_FULL), 2 * L::TILE);
      load_tile<HD>(base + L::K, &tk, bar(KS_KV_FULL), kv_head, jt * BLK, batch);
      load_tile<HD>(base + L::V, &tv, bar(KS_KV_FULL), kv_head, jt * BLK, batch);
      for (int t = 0; t < n_items; ++t) {
        const int head = kv_head * G + t / per_head;
        const int it = jt + t % per_head;
        const int st = t & 1;
        const uint32_t free_parity = ((t >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(KS_Q_EMPTY0 + st), free_parity, abort_flag)) break;
        mbar_expect_tx(bar(KS_Q_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::Q + st * L::TILE, &tq, bar(KS_Q_FULL0 + st), head, it * BLK, batch);
        if (!mbar_wait(bar(KS_DO_EMPTY0 + st), free_parity, abort_flag)) break;
        mbar_expect_tx(bar(KS_DO_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::DO + st * L::TILE, &tdo, bar(KS_DO_FULL0 + st), head, it * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_g = make_idesc_bf16(BLK, HD, true, true);
      // S = Q K^T of item t (its Q stage must have landed)
      auto issue_s = [&](int t) -> bool {
        const int st = t & 1;
        if (!mbar_wait(bar(KS_Q_FULL0 + st), (t >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sq = base + L::Q + st * L::TILE;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_s, kmajor_desc(sq, k), kmajor_desc(base + L::K, k), idesc_s, k != 0);
        umma_commit(bar(KS_S_FULL));
        return true;
      };
      // dP = dO V^T of item t (its dO stage must have landed)
      auto issue_dp = [&](int t) -> bool {
        const int st = t & 1;
        if (!mbar_wait(bar(KS_DO_FULL0 + st), (t >> 1) & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sdo = base + L::DO + st * L::TILE;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_dp, kmajor_desc(sdo, k), kmajor_desc(base + L::V, k), idesc_s, k != 0);
        umma_commit(bar(KS_DP_FULL));
        return true;
      };
      bool ok = mbar_wait(bar(KS_KV_FULL), 0, abort_flag);
      if (ok && n_items > 0) ok = issue_s(0) && issue_dp(0);
      for (int t = 0; t < n_items && ok; ++t) {
        const int st = t & 1;
        const uint32_t sq = base + L::Q + st * L::TILE, sdo = base + L::DO + st * L::TILE;
        // P_READY also means: the softmax threads hold S of item t in registers, the score region is free
        if (!mbar_wait(bar(KS_P_READY), t & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dV += P^T dO   (contraction over the 128 query rows)
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_bf16(t_dv, mnmajor_desc(base + L::PDS, k), mnmajor_desc(sdo, k), idesc_g, (t | k) != 0);
        umma_commit(bar(KS_DO_EMPTY0 + st));
        umma_commit(bar(KS_P_FREE));
        // the scores of the NEXT item run while the softmax threads form dS of this one
        if (t + 1 < n_items && !issue_s(t + 1)) { ok = false; break; }
        // DS_READY also means: dP of item t is in registers, its region is free
        if (!mbar_wait(bar(KS_DS_READY), t & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // dK += dS^T Q
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k)
          umma_bf16(t_dk, mnmajor_desc(base + L::PDS, k), mnmajor_desc(sq, k), idesc_g, (t | k) != 0);
        umma_commit(bar(KS_Q_EMPTY0 + st));
        umma_commit(bar(KS_DS_FREE));
        // ... and dP of the next item behind the gradient products, off the path to the next scores
        if (t + 1 < n_items && !issue_dp(t + 1)) { ok = false; break; }
      }
      if (ok) umma_commit(bar(KS_ACC_DONE));
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;  // two threads per row: columns [0,64) and [64,128)
    const int r = q * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    bool ok = true;
    // Item t is query tile `it` of query head kv_head * G + hh; the row statistics of an item are
    // fetched, and its indices advanced, one item ahead, in the shadow of the wait for the dV product.
    int it = jt, hh = 0;
    float lse = 0.f, dl = 0.f;
    if (n_items > 0) {
      const int row0 = jt * BLK + r;
      const long long stat0 = (static_cast<long long>(batch) * Hq + kv_head * G) * S + row0;
      lse = row0 < S ? LSE[stat0] : 0.f;
      dl = row0 < S ? delta[stat0] : 0.f;
    }
    for (int t = 0; t < n_items; ++t) {
      const bool row_ok = it * BLK + r < S;
      if (!mbar_wait(bar(KS_S_FULL), t & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (it == jt);
      float p[2][32];
      {
        uint32_t sv[2][32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tmem_ld_32x32(t_s + lane_addr + (half * 2 + cc) * 32, sv[cc]);
        tmem_ld_wait();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = half * 2 + cc;
          if (diag || !row_ok) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const bool keep = row_ok && (c * 32 + i) <= r;
              p[cc][i] = keep ? fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse) : 0.f;
            }
          } else {  // mask-free fast path: every tile off the diagonal
#pragma unroll
            for (int i = 0; i < 32; ++i) p[cc][i] = fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse);
          }
        }
      }
      // the operand buffer is free once the dK MMAs of the previous item have read dS from it
      if (t > 0 && !mbar_wait(bar(KS_DS_FREE), (t - 1) & 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) store_row_chunk(smem + L::PDS, r, half * 2 + cc, p[cc]);
      fence_async_smem();
      tc_fence_before();
      __syncwarp();  // the lanes' stores and fences are ordered before the one arrival of the warp
      if (lane == 0) mbar_arrive(bar(KS_P_READY));
      // dP arrives behind the gradient products of the previous item; dS = P (dP - delta)
      if (!mbar_wait(bar(KS_DP_FULL), t & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t dv[2][32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tmem_ld_32x32(t_dp + lane_addr + (half * 2 + cc) * 32, dv[cc]);
        tmem_ld_wait();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc)
#pragma unroll
          for (int i = 0; i < 32; ++i) p[cc][i] *= (__uint_as_float(dv[cc][i]) - dl);
      }
      // the next item's place and statistics, before the wait below so that the loads travel under it
      int n_it = it + 1, n_hh = hh;
      if (n_it == n_tiles) {
        n_it = jt;
        ++n_hh;
      }
      float n_lse = 0.f, n_dl = 0.f;
      if (t + 1 < n_items) {
        const int nrow = n_it * BLK + r;
        const long long nstat = (static_cast<long long>(batch) * Hq + kv_head * G + n_hh) * S + nrow;
        n_lse = nrow < S ? LSE[nstat] : 0.f;
        n_dl = nrow < S ? delta[nstat] : 0.f;
      }
      // ... and dS may replace P once the dV MMAs have read it
      if (!mbar_wait(bar(KS_P_FREE), t & 1, abort_flag)) { ok = false; break; }
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) store_row_chunk(smem + L::PDS, r, half * 2 + cc, p[cc]);
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(KS_DS_READY));
      it = n_it;
      hh = n_hh;
      lse = n_lse;
      dl = n_dl;
    }
    if (ok && mbar_wait(bar(KS_ACC_DONE), 0, abort_flag)) {
      tc_fence_after();
      const int krow = jt * BLK + r;
      const long long tok = static_cast<long long>(batch) * S + krow;
      store_acc<HD / 2>(t_dv + lane_addr + half * (HD / 2), dV + tok * lddv + kv_head * HD + half * (HD / 2), 1.f, krow < S);
      store_acc<HD / 2>(t_dk + lane_addr + half * (HD / 2), dK + tok * lddk + kv_head * HD + half * (HD / 2), scale, krow < S);
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

// ------------------------------------------------------------------ dQ
// K tiles are double buffered, V (needed only for dP, early in an iteration) has one stage,
// and dS has two buffers so that the softmax of tile j+1 overlaps the dQ MMAs of tile j.
template <int HD>
struct DqSmem {
  static constexpr uint32_t TILE = BLK * HD * 2;
  static constexpr uint32_t Q = 0, DO = TILE, K = 2 * TILE /*2 stages*/, V = 4 * TILE /*1 stage*/;
  static constexpr uint32_t DS = 5 * TILE;  // 2 buffers of [128 x 128] bf16
  static constexpr uint32_t BARS = DS + 2 * BLK * BLK * 2;
  static constexpr uint32_t TOTAL = BARS + 256 + 1024;
};
enum DqBar { QDO_FULL = 0, DQ_K_FULL0, DQ_K_FULL1, DQ_V_FULL, DQ_K_EMPTY0, DQ_K_EMPTY1, DQ_V_EMPTY, DQ_SDP_FULL, DQ_DS_READY0, DQ_DS_READY1, DQ_DS_FREE0, DQ_DS_FREE1, DQ_DONE, NUM_DQ_BARS };

template <int HD>
__global__ void __launch_bounds__(320, 1)
attn_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
               const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
               const float* __restrict__ LSE, const float* __restrict__ delta, __nv_bfloat16* __restrict__ dQ,
               int S, int Hq, int Hkv, long long lddq, float scale, float scale_log2, int* status) {
  using L = DqSmem<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar0 = base + L::BARS;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(smem + L::BARS + 8 * NUM_DQ_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::BARS + 8 * NUM_DQ_BARS + 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tiles = (S + BLK - 1) / BLK;
  const int qt = n_tiles - 1 - blockIdx.x / Hq;  // heaviest first over all heads
  const int head = blockIdx.x % Hq, batch = blockIdx.y;
  const int kv_head = head / (Hq / Hkv);
  const int n_kv = qt + 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_DQ_BARS; ++i) mbar_init(bar(i), (i == DQ_DS_READY0 || i == DQ_DS_READY1) ? 256 : 1);
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
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dq = tmem_base + 256;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(QDO_FULL), 2 * L::TILE);
      load_tile<HD>(base + L::Q, &tq, bar(QDO_FULL), head, qt * BLK, batch);
      load_tile<HD>(base + L::DO, &tdo, bar(QDO_FULL), head, qt * BLK, batch);
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(bar(DQ_K_EMPTY0 + st), ((j >> 1) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(DQ_K_FULL0 + st), L::TILE);
        load_tile<HD>(base + L::K + st * L::TILE, &tk, bar(DQ_K_FULL0 + st), kv_head, j * BLK, batch);
        if (!mbar_wait(bar(DQ_V_EMPTY), (j & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(bar(DQ_V_FULL), L::TILE);
        load_tile<HD>(base + L::V, &tv, bar(DQ_V_FULL), kv_head, j * BLK, batch);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BLK, BLK, false, false);
      constexpr uint32_t idesc_q = make_idesc_bf16(BLK, HD, false, true);
      auto issue_sdp = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(bar(DQ_K_FULL0 + st), (j >> 1) & 1, abort_flag) || !mbar_wait(bar(DQ_V_FULL), j & 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = base + L::K + st * L::TILE;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_s, kmajor_desc(base + L::Q, k), kmajor_desc(sk, k), idesc_s, k != 0);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) umma_bf16(t_dp, kmajor_desc(base + L::DO, k), kmajor_desc(base + L::V, k), idesc_s, k != 0);
        umma_commit(bar(DQ_SDP_FULL));
        umma_commit(bar(DQ_V_EMPTY));
        return true;
      };
      bool ok = mbar_wait(bar(QDO_FULL), 0, abort_flag);
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        // dS of tile j is in shared memory, and S / dP of tile j have been read
        if (!mbar_wait(bar(DQ_DS_READY0 + st), (j >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // scores of the next tile first, so its softmax overlaps the dQ MMAs below
        if (j + 1 < n_kv && !issue_sdp(j + 1)) { ok = false; break; }
        // dQ += dS K_j   (contraction over the 128 key rows)
        const uint32_t sk = base + L::K + st * L::TILE, sds = base + L::DS + st * (BLK * BLK * 2);
#pragma unroll
        for (int k = 0; k < BLK / 16; ++k) umma_bf16(t_dq, kmajor_desc(sds, k), mnmajor_desc(sk, k), idesc_q, (j | k) != 0);
        umma_commit(bar(DQ_K_EMPTY0 + st));
        umma_commit(bar(DQ_DS_FREE0 + st));
      }
      if (ok) umma_commit(bar(DQ_DONE));
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;  // two threads per row: columns [0,64) and [64,128)
    const int r = q * 32 + lane;
    const int row = qt * BLK + r;
    const bool row_ok = row < S;
    const uint32_t lane_addr = static_cast<uint32_t>(q * 32) << 16;
    const long long stat = (static_cast<long long>(batch) * Hq + head) * S + row;
    const float lse = row_ok ? LSE[stat] : 0.f;
    const float dl = row_ok ? delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int st = j & 1;
      if (!mbar_wait(bar(DQ_SDP_FULL), j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool diag = (j == qt);
      float ds[2][32];
      uint32_t sv[2][32], dv[2][32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        tmem_ld_32x32(t_s + lane_addr + (half * 2 + cc) * 32, sv[cc]);
        tmem_ld_32x32(t_dp + lane_addr + (half * 2 + cc) * 32, dv[cc]);
      }
      tmem_ld_wait();
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = half * 2 + cc;
        if (diag || !row_ok) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const bool keep = row_ok && (c * 32 + i) <= r;
            const float p = keep ? fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse) : 0.f;
            ds[cc][i] = p * (__uint_as_float(dv[cc][i]) - dl);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p = fast_exp2(__uint_as_float(sv[cc][i]) * scale_log2 - lse);
            ds[cc][i] = p * (__uint_as_float(dv[cc][i]) - dl);
          }
        }
      }
      // this dS buffer was last read by the dQ MMAs of tile j-2
      if (!mbar_wait(bar(DQ_DS_FREE0 + st), ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
      uint8_t* dst = smem + L::DS + st * (BLK * BLK * 2);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) store_row_chunk(dst, r, half * 2 + cc, ds[cc]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(bar(DQ_DS_READY0 + st));
    }
    if (ok && mbar_wait(bar(DQ_DONE), 0, abort_flag)) {
      tc_fence_after();
      const long long tok = static_cast<long long>(batch) * S + row;
      store_acc<HD / 2>(t_dq + lane_addr + half * (HD / 2), dQ + tok * lddq + head * HD + half * (HD / 2), scale, row_ok);
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
int launch_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
               float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv, long long ldq,
               long long ldk, long long ldv, long long lddq, long long lddk, long long lddv, float scale,
               int* status, cudaStream_t stream, int parts = 7) {
  CUtensorMap tq, tk, tv, tdo;
  if (!make_attn_tensormap(&tq, q, HD, Hq, S, B, ldq)) return -2;
  if (!make_attn_tensormap(&tk, k, HD, Hkv, S, B, ldk)) return -3;
  if (!make_attn_tensormap(&tv, v, HD, Hkv, S, B, ldv)) return -4;
  if (!make_attn_tensormap(&tdo, dout, HD, Hq, S, B, static_cast<long long>(Hq) * HD)) return -5;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_dkdv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         DkvSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(attn_dkdv_split_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, DkvSmem<HD>::TOTAL);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaGetLastError();
  const float scale_log2 = scale * 1.4426950408889634f;
  const long long warps = static_cast<long long>(B) * S * Hq;
  if (parts & 1)
    attn_delta_kernel<HD><<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), delta, B, S, Hq);
  const int n_tiles = (S + BLK - 1) / BLK;
  if ((parts & 2) && (parts & 8))
    attn_dkdv_split_kernel<HD><<<dim3(n_tiles * Hkv, B, 1), 320, DkvSmem<HD>::TOTAL, stream>>>(
        tq, tk, tv, tdo, lse, delta, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), S, Hq, Hkv, lddk,
        lddv, scale, scale_log2, status);
  else if (parts & 2)
    attn_dkdv_kernel<HD><<<dim3(n_tiles * Hkv, B, 1), 320, DkvSmem<HD>::TOTAL, stream>>>(
        tq, tk, tv, tdo, lse, delta, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), S, Hq, Hkv, lddk,
        lddv, scale, scale_log2, status);
  if (parts & 4)
    attn_dq_kernel<HD><<<dim3(n_tiles * Hq, B, 1), 320, DqSmem<HD>::TOTAL, stream>>>(
        tq, tk, tv, tdo, lse, delta, static_cast<__nv_bfloat16*>(dq), S, Hq, Hkv, lddq, scale, scale_log2, status);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace attn
}  // namespace tft

// Causal attention backward.  dout and o are contiguous [B,S,Hq,hd]; q/k/v as in the forward;
// dq/dk/dv are written with token strides lddq/lddk/lddv (elements), so they may be views
// into a fused gradient buffer.  delta is [B,Hq,S] fp32 scratch provided by the caller.
TFT_API int tft_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o,
                         const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq, int Hkv,
                         int hd, int ldq, int ldk, int ldv, int lddq, int lddk, int lddv, float scale, int* status,
                         cudaStream_t stream) {
  using namespace tft::attn;
  if (Hq % Hkv || (ldq % 8) || (ldk % 8) || (ldv % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -1;
  if (hd == 128)
    return launch_bwd<128>(dout, q, k, v, o, lse, delta, dq, dk, dv, B, S, Hq, Hkv, ldq, ldk, ldv, lddq, lddk, lddv,
                           scale, status, stream);
  if (hd == 64)
    return launch_bwd<64>(dout, q, k, v, o, lse, delta, dq, dk, dv, B, S, Hq, Hkv, ldq, ldk, ldv, lddq, lddk, lddv,
                          scale, status, stream);
  return -1;
}

// The same with a choice of kernels: parts = 1 (delta) | 2 (dK/dV) | 4 (dQ) | 8 (the dK/dV kernel with
// separate S and dP pipelines instead of the serial one).  The kernels of attention_bwd_tmem.cu take the
// place of the ones left out.
TFT_API int tft_attn_bwd_parts(const void* dout, const void* q, const void* k, const void* v, const void* o,
                               const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int Hq,
                               int Hkv, int hd, int ldq, int ldk, int ldv, int lddq, int lddk, int lddv, float scale,
                               int* status, cudaStream_t stream, int parts) {
  using namespace tft::attn;
  if (Hq % Hkv || (ldq % 8) || (ldk % 8) || (ldv % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -1;
  if (hd == 128)
    return launch_bwd<128>(dout, q, k, v, o, lse, delta, dq, dk, dv, B, S, Hq, Hkv, ldq, ldk, ldv, lddq, lddk, lddv,
                           scale, status, stream, parts);
  if (hd == 64)
    return launch_bwd<64>(dout, q, k, v, o, lse, delta, dq, dk, dv, B, S, Hq, Hkv, ldq, ldk, ldv, lddq, lddk, lddv,
                          scale, status, stream, parts);
  return -1;
}
