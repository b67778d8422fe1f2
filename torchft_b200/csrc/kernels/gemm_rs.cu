// Weight-gradient GEMM fused with the reduce-scatter of its result over NVLink peer memory.
//
//   dW[M, N] = A^T B      A stored [K, M] (dY: tokens x out_features), B stored [K, N] (X: tokens x
//                         in_features), bf16 in, fp32 accumulation
//
// The rows of dW are sharded over the `world` ranks of a communicator: rank r ends up with rows
// [r * M / world, (r + 1) * M / world) of the SUM of all ranks' products, in `out` (bf16).  Nothing
// else is produced: the full local product never touches memory and no separate reduce-scatter
// kernel runs afterwards.  This replaces "wgrad GEMM into a full gradient buffer, then
// reduce_scatter_kernel" (the reference gets the same result from FSDP2's reduce_scatter_tensor
// after autograd's GEMM).
//
// Pipeline and tile shape are those of gemm_tcgen05.cu (TMA -> 128B-swizzled shared memory ->
// tcgen05.mma, two fp32 accumulators of 128 x 256 in tensor memory, tcgen05.ld epilogue); every TMA
// load reads this GPU's own memory.  What differs is the order of the tiles and the epilogue:
//
//   * Row blocks are visited owner by owner, starting with the rows owned by rank + 1 and ending
//     with this rank's own rows.  At any time the ranks therefore send to pairwise different
//     owners, and a rank reaches its own rows when the others have already produced theirs.
//   * The epilogue of a tile that a PEER owns rounds the accumulator to bf16 and writes it with plain
//     stores into that peer's staging area, slot [this rank]; after a system-scope fence one thread
//     publishes the tile with a release store of the call's tag (epoch, sequence number) into the
//     peer's flag [this rank][tile].
//   * The epilogue of an OWN tile waits until the flags of all peers carry this call's tag, adds the
//     staged partial tiles to its accumulator in fp32 in rank order (the sum is deterministic) and
//     writes -- or accumulates into -- the gradient shard.
//
// A rank may overwrite a peer's staging area only once that peer has finished reading what the
// previous call left there.  Stream order gives that: a rank signals "entered call seq" at the start
// of the kernel, which runs after its previous call has ended, and a peer's epilogue waits for that
// signal before its first remote store.  The main loop does not wait for it.
//
// All waits are bounded (time budget, host abort word, the communicator's status word) like those
// of p2p_comm.cu; a rank that gives up sets the status, drains and leaves.  Deadlock freedom needs
// every CTA of a rank resident at once (one CTA per SM, grid <= SM count): tiles for peers are
// produced without waiting for anyone's data, and own tiles come last in every CTA's list.
//
// Requirements: M % (128 * world) == 0, N % 256 == 0, lda / ldb / ldo multiples of 8 elements.
// Per-rank memory in the symmetric heap: staging M * N bf16 (slot of the own rank unused) at
// `stage_off`, flags world * (M / world / 128) * (N / 256) uint32 at `flag_off`.
// The staging area is private to this kernel and laid out for the link, not as a matrix:
// [source rank][tile of the shard][column half][128 rows][128 columns], so the 32 rows x 128 columns
// that one epilogue warp sends at a time are 8 KB of consecutive addresses.
#include "common.cuh"
#include "p2p_common.cuh"
#include "tensormap.cuh"

namespace tft {
namespace gemm_rs {

using namespace p2p;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr uint32_t A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2;
constexpr uint32_t STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
// Epilogue staging: each of the four epilogue warps owns 32 rows x 128 columns of bf16 (8 KB), used to
// turn "one thread holds 64 contiguous bytes of one row" (what tcgen05.ld delivers) into "one warp
// instruction writes 2 x 256 contiguous bytes".  Stores that cross NVLink are packetised per
// instruction and per contiguous run: 16-byte runs waste most of every packet, 256-byte runs fill it.
constexpr uint32_t EPI_WARP_BYTES = 32 * 128 * 2;
constexpr uint32_t EPI_BYTES = 4 * EPI_WARP_BYTES;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;

struct Tile {
  int m0, n0, owner, local;
};

// t-th tile in this rank's order: owners come as rank+1, ..., rank (own rows last).  Inside an owner's
// rows the tiles run down GROUP_M row blocks before moving to the next column block, so the tiles that
// the CTAs work on at the same time share a few row panels of A and a few column panels of B in L2.
constexpr int GROUP_M = 8;
__host__ __device__ inline Tile tile_of(int t, int tiles_n, int mblocks_per_rank, int rank, int world) {
  const int tiles_per_shard = mblocks_per_rank * tiles_n;
  const int period = t / tiles_per_shard;
  const int idx = t - period * tiles_per_shard;
  const int per_group = GROUP_M * tiles_n;
  const int g = idx / per_group;
  const int first = g * GROUP_M;
  const int gm = mblocks_per_rank - first < GROUP_M ? mblocks_per_rank - first : GROUP_M;
  const int r = idx - g * per_group;
  const int mb_local = first + r % gm;
  const int nb = r / gm;
  Tile x;
  x.owner = (rank + 1 + period) % world;
  x.m0 = (x.owner * mblocks_per_rank + mb_local) * BM;
  x.n0 = nb * BN;
  x.local = mb_local * tiles_n + nb;  // index of the tile inside its owner's shard
  return x;
}

__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Polls `slot` (this rank's own memory) until it holds `want`; bounded.  Returns false after
// recording why it gave up.
__device__ __forceinline__ bool wait_word(const Comm& c, const uint32_t* slot, uint32_t want, volatile int* abort_flag) {
  const unsigned long long t0 = now_ns();
  uint32_t it = 0;
  while (ld_acquire_sys(slot) != want) {
    if ((++it & 63u) == 0) {
      if (*abort_flag) return false;
      if (c.abort_word && *c.abort_word) {
        if (c.status) atomicCAS(c.status, 0, static_cast<int>(kAborted));
        return false;
      }
      if (now_ns() - t0 > c.budget_ns) {
        if (c.status) atomicCAS(c.status, 0, static_cast<int>(kTimeoutPeer));
        return false;
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, Comm comm,
               size_t stage_off, size_t flag_off, __nv_bfloat16* __restrict__ out, int ldo, int M, int N, int K,
               int accumulate) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  uint8_t* epi_smem = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES + EPI_BYTES);
  const uint32_t bar_base = base + STAGES * STAGE_BYTES + EPI_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  volatile uint32_t* tmem_holder = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 5);
  volatile int* wait_ok = reinterpret_cast<volatile int*>(bars + 2 * STAGES + 6);  // verdict shared by the epilogue warps

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull_bar(b), 1);
      mbar_init(tempty_bar(b), 4);
    }
    // a communicator that already lost a peer in this membership fails at once (see wait_pad)
    *abort_flag = (comm.status && *reinterpret_cast<volatile int*>(comm.status) != 0) ? 1 : 0;
    *wait_ok = 1;
    mbar_fence_init();
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_holder)), TMEM_COLS);
    tmem_relinquish();
  }
  // "this rank has entered call seq": its staging area may be overwritten from now on
  if (blockIdx.x == 0) signal_pad(comm, START_PAD, comm.seq, 1);  // threads 0 .. world-1 write one peer each
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  const int tiles_n = N / BN;
  const int mblocks_per_rank = M / BM / comm.world;
  const int tiles_per_shard = mblocks_per_rank * tiles_n;
  const int num_tiles = (M / BM) * tiles_n;
  const int kblocks = (K + BK - 1) / BK;
  const size_t shard_elems = static_cast<size_t>(M / comm.world) * N;
  const uint32_t tag = flag_value(comm.epoch, comm.seq, 1);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tc = tile_of(t, tiles_n, mblocks_per_rank, comm.rank, comm.world);
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tma_a, full_bar(stage), tc.m0 + 64 * j, kb * BK);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tma_b, full_bar(stage), tc.n0 + 64 * j, kb * BK);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, true, true);
      int stage = 0, it = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(tempty_bar(buf), (((it >> 1) & 1) ^ 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(d_tmem, make_smem_desc(sa + k * 2048, 8192, 1024), make_smem_desc(sb + k * 2048, 8192, 1024), idesc,
                      (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(tfull_bar(buf));
      }
    }
  } else {
    const int q = warp & 3;
    const int et = threadIdx.x - 64;  // 0..127 among the epilogue threads
    int it = 0;
    bool ok = true;
    bool peers_entered = false;
    const uint32_t* my_flags = reinterpret_cast<const uint32_t*>(comm.heap[comm.rank] + flag_off);  // [src][tile]
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      const Tile tc = tile_of(t, tiles_n, mblocks_per_rank, comm.rank, comm.world);
      const int buf = it & 1;
      if (!mbar_wait(tfull_bar(buf), (it >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool mine = tc.owner == comm.rank;
      // ---- waits of this tile: one thread per awaited word, verdict through shared memory
      if (mine || !peers_entered) {
        if (et < comm.world && et != comm.rank) {
          bool got;
          if (mine) {
            uint32_t* slot = const_cast<uint32_t*>(my_flags) + static_cast<size_t>(et) * tiles_per_shard + tc.local;
            got = wait_word(comm, slot, tag, abort_flag);
            // Consumed: clear it, so that a tag can never be mistaken for the one of a call 2^20
            // sequence numbers later.  The sender writes this word again only in a later call, which
            // it starts sending for only after this rank has entered that call.
            if (got) *reinterpret_cast<volatile uint32_t*>(slot) = 0u;
          } else {
            const uint32_t* slot = reinterpret_cast<const uint32_t*>(comm.heap[comm.rank]) + comm.pad_base + START_PAD + et;
            got = wait_word(comm, slot, flag_value(comm.epoch, comm.seq, 1), abort_flag);
          }
          if (!got) { *wait_ok = 0; *abort_flag = 1; }
        }
        epilogue_bar();
        if (!*wait_ok) { ok = false; break; }
        if (!mine) peers_entered = true;
      }
      const int row_in_shard = tc.m0 - tc.owner * (M / comm.world) + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      if (mine) {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = tc.n0 + c * 32;
          float acc[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(r[i]);
          // partial tiles of the peers, in rank order, three sources' loads in flight at a time
          const size_t in_tile = (static_cast<size_t>(c >> 2) * 128 + q * 32 + lane) * 128 + (c & 3) * 32;
          const __nv_bfloat16* staged = reinterpret_cast<const __nv_bfloat16*>(comm.heap[comm.rank] + stage_off) +
                                        static_cast<size_t>(tc.local) * (BM * BN) + in_tile;
          for (int s0 = 0; s0 < comm.world; s0 += 3) {
            uint4 v[3][4];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
              const int src = s0 + j;
              const bool take = src < comm.world && src != comm.rank;
#pragma unroll
              for (int g = 0; g < 4; ++g)
                v[j][g] = take ? ld_peer_v4(staged + static_cast<size_t>(src) * shard_elems + g * 8) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < 3; ++j) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j][g]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(h[i]);
                  acc[g * 8 + 2 * i] += f.x;
                  acc[g * 8 + 2 * i + 1] += f.y;
                }
              }
            }
          }
          __nv_bfloat16* dst = out + static_cast<size_t>(row_in_shard) * ldo + col;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            if (accumulate) {
              const uint4 old = *reinterpret_cast<const uint4*>(dst + g * 8);
              const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(oh[i]);
                acc[g * 8 + 2 * i] += f.x;
                acc[g * 8 + 2 * i + 1] += f.y;
              }
            }
            uint4 o;
            o.x = pack_bf16(acc[g * 8 + 0], acc[g * 8 + 1]);
            o.y = pack_bf16(acc[g * 8 + 2], acc[g * 8 + 3]);
            o.z = pack_bf16(acc[g * 8 + 4], acc[g * 8 + 5]);
            o.w = pack_bf16(acc[g * 8 + 6], acc[g * 8 + 7]);
            *reinterpret_cast<uint4*>(dst + g * 8) = o;
          }
        }
      } else {
        // Peer tile: through this warp's staging buffer, 128 columns at a time.  A row of the buffer is
        // 256 bytes = 16 chunks of 16 bytes; chunk j of row r sits at position j ^ (r & 15), which keeps
        // both the row-per-thread writes and the row-per-half-warp reads free of bank conflicts.
        uint4* buf4 = reinterpret_cast<uint4*>(epi_smem + q * EPI_WARP_BYTES);
        __nv_bfloat16* peer_tile = reinterpret_cast<__nv_bfloat16*>(comm.heap[tc.owner] + stage_off) +
                                   comm.rank * shard_elems + static_cast<size_t>(tc.local) * (BM * BN);
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + (half * 4 + c) * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
              o.y = pack_bf16(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
              o.z = pack_bf16(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
              o.w = pack_bf16(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
              buf4[lane * 16 + ((c * 4 + g) ^ (lane & 15))] = o;
            }
          }
          __syncwarp();
          if (half == 1) {
            // The accumulator has been read completely: hand the tensor-memory buffer back now, so the
            // next-but-one tile's MMAs need not wait for this tile's stores to cross the link.
            tc_fence_before();
            if (lane == 0) mbar_arrive(tempty_bar(buf));
          }
          const int chunk = lane & 15;
#pragma unroll 4
          for (int rr = 0; rr < 16; ++rr) {
            const int row = rr * 2 + (lane >> 4);
            const uint4 v = buf4[row * 16 + (chunk ^ (row & 15))];
            *reinterpret_cast<uint4*>(peer_tile + (static_cast<size_t>(half) * 128 + q * 32 + row) * 128 + chunk * 8) = v;
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      if (!mine) {
        // The barrier orders the 128 threads' peer stores before thread 0's release store, and a
        // release is cumulative: whoever acquires the flag sees all of them.
        epilogue_bar();
        if (et == 0) {
          uint32_t* flag = reinterpret_cast<uint32_t*>(comm.heap[tc.owner] + flag_off) +
                           static_cast<size_t>(comm.rank) * tiles_per_shard + tc.local;
          st_release_sys(flag, tag);
        }
      }
      __syncwarp();
      if (mine && lane == 0) mbar_arrive(tempty_bar(buf));  // peer tiles released theirs before the stores
    }
  }

  __syncthreads();
  if (*abort_flag) {
    // Give loads that may still be in flight time to land before shared memory is released.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    if (threadIdx.x == 0 && comm.status) atomicCAS(comm.status, 0, static_cast<int>(kTimeoutBarrier));
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm_rs
}  // namespace tft

// Bytes of staging and of flags that a call with these sizes uses in every rank's heap.
TFT_API long long tft_gemm_rs_stage_bytes(int M, int N) { return static_cast<long long>(M) * N * 2; }
TFT_API long long tft_gemm_rs_flag_bytes(int M, int N, int world) {
  return static_cast<long long>(M / 128) * (N / 256) * 4;  // world * tiles per shard
}

// out[M / world, N] (+)= rows of this rank of  sum over ranks of  A^T B.
//   a: [K, M] bf16 (row stride lda), b: [K, N] bf16 (row stride ldb), out: bf16 (row stride ldo), all local.
//   stage_off / flag_off: byte offsets of the staging area and the flags inside the symmetric heap.
// Returns -1 for misaligned arguments, -4 when M, N do not meet the divisibility rules, -5 when the
// grid would not be co-resident.
TFT_API int tft_gemm_rs_bf16(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                             const int* abort_word, int* status, const void* a, const void* b, void* out, int M, int N,
                             int K, int lda, int ldb, int ldo, long long stage_off, long long flag_off, int accumulate,
                             cudaStream_t stream) {
  using namespace tft;
  using namespace tft::gemm_rs;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (world < 2 || M % (BM * world) || N % BN) return -4;
  if ((lda % 8) || (ldb % 8) || (ldo % 8) || (stage_off & 255) || (flag_off & 15) ||
      (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -1;
  CUtensorMap ta, tb;
  if (!make_tensormap(&ta, a, 2, 2, M, K, 1, uint64_t(lda) * 2, 0, 64, BK, 1, 1)) return -2;
  if (!make_tensormap(&tb, b, 2, 2, N, K, 1, uint64_t(ldb) * 2, 0, 64, BK, 1, 1)) return -3;
  cudaGetLastError();
  static bool configured = false;
  static int sm_count = 0;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return static_cast<int>(e);
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured = true;
  }
  p2p::Comm c = p2p::make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const int tiles = (M / BM) * (N / BN);
  const int grid = tiles < sm_count ? tiles : sm_count;  // one CTA per SM: all resident at once
  if (grid < 1) return -5;
  gemm_rs_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, c, static_cast<size_t>(stage_off),
                                                            static_cast<size_t>(flag_off),
                                                            static_cast<__nv_bfloat16*>(out), ldo, M, N, K, accumulate);
  return static_cast<int>(cudaGetLastError());
}
