// All-gather fused into its consumer GEMM (sm_100a, NVLink peer memory).
//
//   Y[M,N] = X[M,K] * W[N,K]^T      W is sharded by rows over `world` GPUs
//
// Every rank holds rows [r*N/world, (r+1)*N/world) of W at the same offset of its symmetric
// heap.  ONE kernel per rank both gathers the peers' rows into the local copy of W and runs
// the tcgen05 GEMM on it:
//
//   * a few "copy" CTAs pull the peers' row blocks over NVLink with bulk asynchronous copies
//     (peer global -> shared ring -> local global, one elected thread per CTA, no cluster
//     broadcast form) and publish one counter per 256-row block of W;
//   * the remaining CTAs are the persistent GEMM of gemm_tcgen05.cu.  They walk the output
//     tiles owner by owner, starting with the rows this rank owns (no wait at all), so the
//     transfer of block j+1 overlaps the tensor-core work on block j.  The TMA producer waits
//     (bounded) on a block's counter before its first load of that block.
//
// Copy CTAs and GEMM CTAs are blocks of one launch with one CTA per SM (the grid never exceeds
// the SM count), so the waits between them are waits inside one kernel.  Peer hand-shakes use
// the epoch-tagged start/end pads of the communicator; every wait has a time budget and
// reports through the status word instead of spinning forever.
//
// The reference leaves this pair to FSDP2 (all_gather_into_tensor on NCCL, then a cuBLAS GEMM,
// torchft/fsdp_test.py:63-64); it has no fused counterpart.
#include "p2p_common.cuh"
#include "tensormap.cuh"

namespace tft {
namespace aggemm {

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
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
// copy CTAs reuse the pipeline stages as a ring of bulk-copy buffers
constexpr uint32_t CHUNK_BYTES = 32768;
constexpr int RING = (STAGES * STAGE_BYTES) / CHUNK_BYTES;  // 6
constexpr int FLAG_ABORT = 0x40000000;

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename OutT>
__device__ __forceinline__ void store32(OutT* p, const uint32_t (&r)[32], int valid);
template <>
__device__ __forceinline__ void store32<__nv_bfloat16>(__nv_bfloat16* p, const uint32_t (&r)[32], int valid) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    if (g * 8 >= valid) break;
    uint4 o;
    o.x = pack_bf16(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
    o.y = pack_bf16(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
    o.z = pack_bf16(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
    o.w = pack_bf16(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
    *reinterpret_cast<uint4*>(p + g * 8) = o;
  }
}

struct Params {
  p2p::Comm comm;
  size_t w_off;          // byte offset of the gathered W[N,K] inside every heap
  int* block_ready;      // [N / BN] counters, zeroed before the launch
  int copy_ctas;
  int M, N, K, ldc;
  int* status;
};

// Marks every block counter as aborted so that no GEMM CTA keeps waiting for data.
__device__ void poison(const Params& p) {
  const int blocks = p.N / BN;
  for (int i = threadIdx.x; i < blocks; i += blockDim.x) atomicOr(p.block_ready + i, FLAG_ABORT);
}

// ---------------------------------------------------------------- copy role
__device__ void copy_role(const Params& p, uint8_t* smem, uint32_t base, uint32_t bar_base) {
  __shared__ int flag[2];
  __shared__ int is_last;
  const p2p::Comm& c = p.comm;
  // this rank's rows are final (the caller ordered the launch after their producer): tell the peers
  if (blockIdx.x == 0) p2p::signal_pad(c, p2p::START_PAD, c.seq, 1);
  if (!p2p::wait_pad(c, p2p::START_PAD, c.seq, nullptr, flag)) {
    poison(p);
    return;
  }
  const int blocks_per_rank = p.N / BN / c.world;
  const size_t block_bytes = static_cast<size_t>(BN) * p.K * 2;
  // every copy CTA moves an equal, 16-byte aligned share of EVERY block, so blocks complete in order
  const size_t share = ((block_bytes / p.copy_ctas) + 15) & ~size_t(15);
  const size_t lo = min(block_bytes, share * blockIdx.x);
  const size_t hi = min(block_bytes, lo + share);
  const int chunks_per_block = static_cast<int>((hi - lo + CHUNK_BYTES - 1) / CHUNK_BYTES);
  const int remote_blocks = blocks_per_rank * (c.world - 1);
  const long long total = static_cast<long long>(remote_blocks) * chunks_per_block;
  bool ok = true;

  if (threadIdx.x == 0 && total > 0) {
    auto ring_bar = [&](int s) { return bar_base + 8u * s; };
    for (int s = 0; s < RING; ++s) mbar_init(ring_bar(s), 1);
    mbar_fence_init();
    fence_proxy_async();  // the peers' rows were published to the generic proxy; the bulk copies read them through the async one
    volatile int local_abort = 0;
    auto locate = [&](long long i, const uint8_t** src, uint8_t** dst, uint32_t* bytes, int* blk) {
      const int rb = static_cast<int>(i / chunks_per_block);       // remote block in walk order
      const int ch = static_cast<int>(i - static_cast<long long>(rb) * chunks_per_block);
      const int owner = (c.rank + 1 + rb / blocks_per_rank) % c.world;
      const int b = owner * blocks_per_rank + rb % blocks_per_rank;
      const size_t off = p.w_off + static_cast<size_t>(b) * block_bytes + lo + static_cast<size_t>(ch) * CHUNK_BYTES;
      *src = c.heap[owner] + off;
      *dst = c.heap[c.rank] + off;
      const size_t left = (hi - lo) - static_cast<size_t>(ch) * CHUNK_BYTES;
      *bytes = static_cast<uint32_t>(left < CHUNK_BYTES ? left : CHUNK_BYTES);
      *blk = b;
    };
    auto issue_load = [&](long long i) {
      const uint8_t* src; uint8_t* dst; uint32_t bytes; int blk;
      locate(i, &src, &dst, &bytes, &blk);
      const int s = static_cast<int>(i % RING);
      mbar_expect_tx(ring_bar(s), bytes);
      bulk_g2s(base + s * CHUNK_BYTES, src, bytes, ring_bar(s));
    };
    const long long prime = total < RING ? total : RING;
    for (long long i = 0; i < prime; ++i) issue_load(i);
    for (long long i = 0; i < total; ++i) {
      const int s = static_cast<int>(i % RING);
      if (!mbar_wait(ring_bar(s), static_cast<uint32_t>((i / RING) & 1), &local_abort)) { ok = false; break; }
      const uint8_t* src; uint8_t* dst; uint32_t bytes; int blk;
      locate(i, &src, &dst, &bytes, &blk);
      bulk_s2g(dst, base + s * CHUNK_BYTES, bytes);
      bulk_commit();
      if (i >= 1 && i - 1 + RING < total) {
        bulk_wait_read<1>();  // the store of chunk i-1 no longer reads its buffer
        issue_load(i - 1 + RING);
      }
      if ((i + 1) % chunks_per_block == 0) {
        // this CTA's share of the block is in local memory: make it visible, then count it
        bulk_wait_all();
        fence_proxy_async();
        red_release_gpu_add(p.block_ready + blk, 1);
      }
    }
    if (!ok) {
      // loads still in flight target our shared memory: let them land before the CTA exits
      const long long t0 = clock64();
      while (clock64() - t0 < 4000000LL) { }
      bulk_wait_all();
      if (p.status) atomicCAS(p.status, 0, static_cast<int>(kTimeoutBarrier));
    }
    flag[0] = ok ? 1 : 0;
  } else if (threadIdx.x == 0) {
    // nothing to move for this CTA (more copy CTAs than 16-byte pieces): still counted per block
    for (int rb = 0; rb < remote_blocks; ++rb) {
      const int owner = (c.rank + 1 + rb / blocks_per_rank) % c.world;
      red_release_gpu_add(p.block_ready + owner * blocks_per_rank + rb % blocks_per_rank, 1);
    }
    flag[0] = 1;
  }
  __syncthreads();
  if (total > 0 && !flag[0]) poison(p);

  // end hand-shake: the last copy CTA tells the peers that this rank no longer reads their rows
  // and waits for the same word from them, so nobody's rows change under a reader
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* counter = reinterpret_cast<uint32_t*>(c.heap[c.rank]) + c.pad_base + p2p::DONE_COUNTER;
    const uint32_t ticket = atomicAdd(counter, 1u);
    is_last = (ticket == static_cast<uint32_t>(p.copy_ctas) - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (is_last) {
    p2p::signal_pad(c, p2p::END_PAD, c.seq, 0);
    p2p::wait_pad(c, p2p::END_PAD, c.seq, nullptr, flag);
  }
}

// ---------------------------------------------------------------- GEMM role
template <typename OutT>
__device__ void gemm_role(const Params& p, const CUtensorMap* tma_a, const CUtensorMap* tma_b, OutT* C,
                          uint8_t* smem, uint32_t base, uint32_t bar_base, int cta, int n_ctas) {
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 5);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 4); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(tma_a);
    tma_prefetch_desc(tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int tiles_m = (p.M + BM - 1) / BM;
  const int tiles_n = p.N / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  const int blocks_per_rank = tiles_n / p.comm.world;
  const int first_block = p.comm.rank * blocks_per_rank;
  // walk order: all row tiles of one block of W, blocks owner by owner starting with our own
  auto tile_of = [&](int t, int* m0, int* nb) {
    *nb = (first_block + t / tiles_m) % tiles_n;
    *m0 = (t % tiles_m) * BM;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int ready_upto = -1;  // walk position of the last block known to be complete
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        int m0, nb;
        tile_of(t, &m0, &nb);
        const int pos = t / tiles_m;
        if (pos >= blocks_per_rank && pos > ready_upto) {
          const unsigned long long t0 = p2p::now_ns();
          uint32_t it = 0;
          while (true) {
            const int v = ld_acquire_gpu(p.block_ready + nb);
            if (v & FLAG_ABORT) { ok = false; break; }
            if (v >= p.copy_ctas) break;
            if ((++it & 31u) == 0) {
              if (*abort_flag) { ok = false; break; }
              if (p2p::now_ns() - t0 > p.comm.budget_ns) {
                if (p.status) atomicCAS(p.status, 0, static_cast<int>(kTimeoutPeer));
                ok = false;
                break;
              }
              __nanosleep(200);
            }
          }
          if (!ok) { *abort_flag = 1; break; }
          fence_proxy_async();  // the block was written through another proxy than the TMA reads below
          ready_upto = pos;
        }
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          tma_load_2d(sa, tma_a, full_bar(stage), kb * BK, m0);
          tma_load_2d(sa + A_STAGE_BYTES, tma_b, full_bar(stage), kb * BK, nb * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, false);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas, ++it) {
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
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(d_tmem, make_smem_desc(sa + k * 32, 16, 1024), make_smem_desc(sb + k * 32, 16, 1024), idesc,
                      (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += n_ctas, ++it) {
      int m0, nb;
      tile_of(t, &m0, &nb);
      const int buf = it & 1;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
#pragma unroll 1
      for (int cch = 0; cch < BN / 32; ++cch) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + cch * 32, r);
        tmem_ld_wait();
        if (row < p.M) store32<OutT>(C + static_cast<size_t>(row) * p.ldc + nb * BN + cch * 32, r, 32);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(buf));
    }
  }

  __syncthreads();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, static_cast<int>(kTimeoutBarrier));
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename OutT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               OutT* __restrict__ C, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t bar_base = base + STAGES * STAGE_BYTES;
  if (static_cast<int>(blockIdx.x) < p.copy_ctas)
    copy_role(p, smem, base, bar_base);
  else
    gemm_role<OutT>(p, &tma_a, &tma_b, C, smem, base, bar_base, blockIdx.x - p.copy_ctas,
                    gridDim.x - p.copy_ctas);
}

}  // namespace aggemm
}  // namespace tft

// Y[M,N] = X[M,K] * W[N,K]^T with W gathered from the peers inside the same kernel.
//   heaps/rank/world/epoch_word/seq/timeout_ms/abort_word/status: the communicator, as for the
//       collectives of p2p_comm.cu (epoch_word carries the channel in bits 16-19)
//   w_off: byte offset of W[N,K] (row stride K) in every heap; rank r's rows are valid in heap r
//   block_ready: device int[N/256] scratch owned by the caller (cleared here on the stream)
//   copy_ctas: CTAs that move data (1..32); the rest of the SMs run the GEMM
// Requirements: world >= 2, N % (256 * world) == 0, K % 64 == 0, pointers 16-byte aligned.
// Returns 0, a negative validation code, or a CUDA error.
TFT_API int tft_ag_gemm_bf16(void* const* heaps, int rank, int world, unsigned epoch_word, unsigned seq,
                             int timeout_ms, const int* abort_word, int* status, const void* x, long long w_off,
                             void* y, int M, int N, int K, int ldx, int ldy, int* block_ready, int copy_ctas,
                             cudaStream_t stream) {
  using namespace tft;
  using namespace tft::aggemm;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 2 || world > p2p::MAX_RANKS || rank < 0 || rank >= world) return -4;
  if (N % (BN * world) || K % BK || (ldx % 8) || (ldy % 8) || (w_off & 15) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(y) & 15))
    return -1;
  if (copy_ctas < 1 || copy_ctas > 32) return -5;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (copy_ctas >= sm_count) return -5;
  const uint8_t* w_local = static_cast<const uint8_t*>(heaps[rank]) + w_off;
  CUtensorMap ta, tb;
  if (!make_tensormap(&ta, x, 2, 2, K, M, 1, uint64_t(ldx) * 2, 0, BK, BM, 1, 1)) return -2;
  if (!make_tensormap(&tb, w_local, 2, 2, K, N, 1, uint64_t(K) * 2, 0, BK, BN, 1, 1)) return -3;
  cudaGetLastError();
  auto kfn = ag_gemm_kernel<__nv_bfloat16>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaError_t e = cudaMemsetAsync(block_ready, 0, sizeof(int) * (N / BN), stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  Params p;
  p.comm = p2p::make_comm(heaps, rank, world, epoch_word, seq, timeout_ms, abort_word, status);
  p.w_off = static_cast<size_t>(w_off);
  p.block_ready = block_ready;
  p.copy_ctas = copy_ctas;
  p.M = M; p.N = N; p.K = K; p.ldc = ldy;
  p.status = status;
  const int tiles = ((M + BM - 1) / BM) * (N / BN);
  int gemm_ctas = sm_count - copy_ctas;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  kfn<<<copy_ctas + gemm_ctas, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, static_cast<__nv_bfloat16*>(y), p);
  return static_cast<int>(cudaGetLastError());
}
