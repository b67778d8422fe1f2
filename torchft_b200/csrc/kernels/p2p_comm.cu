// Reconfigurable NVLink peer-to-peer collectives.
//
// Every rank owns a "symmetric heap": one cudaMalloc'ed region whose CUDA IPC handle is
// published to the peers, so each rank holds a device pointer to every peer's heap and
// the same byte offset names the same logical buffer everywhere.  Collectives are single
// kernels that load from / store to peer heaps directly over NVLink (no NCCL, no copy
// engine, no multicast objects):
//
//   allreduce      two-shot, fused: rank r reduces chunk r from all contributing peers
//                  (fp32 accumulation), scales it, and stores the result into chunk r of
//                  EVERY peer in the same pass.  A rank may take part without contributing
//                  (healing / spare replica): its loads are skipped.
//   reduce_scatter rank r reduces slice r from all peers into its own buffer.
//   all_gather     rank r pushes its slice r into every peer's buffer.
//
// Synchronisation uses 32-bit flags in a small header of each heap.  A flag value carries
// the epoch of the current membership (changes on every reconfigure), a sequence number
// and the sender's contribute bit, so a stale write from an earlier membership can never
// satisfy a wait.  Every wait is bounded by a wall-clock budget (globaltimer) and also
// watches a host-mapped abort word; on expiry the kernel records a status and returns.
#include "p2p_common.cuh"

#include <cstdio>
#include <mutex>

namespace tft {
namespace p2p {

// End of a collective: once the last block of this rank is done, tell the peers and wait
// until every peer said the same (so nobody still touches our heap when the kernel ends).
__device__ void finish(const Comm& c, int* smem_flag) {
  __syncthreads();
  __shared__ int is_last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* counter = reinterpret_cast<uint32_t*>(c.heap[c.rank]) + c.pad_base + DONE_COUNTER;
    const uint32_t ticket = atomicAdd(counter, 1u);
    is_last = (ticket == gridDim.x - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (is_last) {
    signal_pad(c, END_PAD, c.seq, 0);
    wait_pad(c, END_PAD, c.seq, nullptr, smem_flag);
  }
}

template <typename T>
struct Vec;
template <>
struct Vec<float> {
  static constexpr int N = 4;
  __device__ static void add(float (&acc)[8], const uint4& v) {
    acc[0] += __uint_as_float(v.x); acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z); acc[3] += __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const float (&acc)[8], float s) {
    return make_uint4(__float_as_uint(acc[0] * s), __float_as_uint(acc[1] * s), __float_as_uint(acc[2] * s),
                      __float_as_uint(acc[3] * s));
  }
};
template <>
struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void add(float (&acc)[8], const uint4& v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  __device__ static uint4 pack(const float (&acc)[8], float s) {
    return make_uint4(pack_bf16(acc[0] * s, acc[1] * s), pack_bf16(acc[2] * s, acc[3] * s),
                      pack_bf16(acc[4] * s, acc[5] * s), pack_bf16(acc[6] * s, acc[7] * s));
  }
};

// In place on heap offset `off`, `nvec` 16-byte vectors.  Rank r owns vectors
// [r*per, min((r+1)*per, nvec)).
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_kernel(Comm c, size_t off, long long nvec, float scale, int contribute) {
  __shared__ int flag[2];
  if (blockIdx.x == 0) signal_pad(c, START_PAD, c.seq, contribute);
  uint32_t mask = 0;
  if (!wait_pad(c, START_PAD, c.seq, &mask, flag)) return;
  const long long per = (nvec + c.world - 1) / c.world;
  const long long lo = per * c.rank;
  const long long hi = lo + per < nvec ? lo + per : nvec;
  // Each thread handles UNR vectors per round so that UNR * world loads are in flight per
  // thread: NVLink round trips are microseconds, bandwidth comes from memory-level parallelism.
  constexpr int UNR = 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < hi;
       i0 += stride * UNR) {
    uint4 in[UNR][MAX_RANKS];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        const int p = (c.rank + k) % c.world;  // start with the local copy, then walk the ring
        in[u][k] = make_uint4(0, 0, 0, 0);
        if (i < hi && (mask & (1u << p))) in[u][k] = ld_peer_v4(c.heap[p] + off + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      if (i >= hi) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        Vec<T>::add(acc, in[u][k]);
      }
      const uint4 out = Vec<T>::pack(acc, scale);
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        const int p = (c.rank + k) % c.world;
        *reinterpret_cast<uint4*>(c.heap[p] + off + i * 16) = out;
      }
    }
  }
  finish(c, flag);
}

// One-shot allreduce for buffers of at most ONE_SHOT_MAX_VEC vectors, in ONE block: every rank loads
// the whole buffer from every contributing peer, keeps its sums in registers across the end
// hand-shake (nobody may overwrite its buffer before all peers have read it) and then writes its own
// copy.  Against the two-shot kernel it saves the remote stores, the system-wide fence behind them
// and the inter-block counter; it moves world - 1 times the buffer instead of 2 (world - 1) / world.
constexpr int ONE_SHOT_THREADS = 1024, ONE_SHOT_VPT = 8;
constexpr long long ONE_SHOT_MAX_VEC = static_cast<long long>(ONE_SHOT_THREADS) * ONE_SHOT_VPT;  // 128 KiB
template <typename T>
__global__ void __launch_bounds__(ONE_SHOT_THREADS)
allreduce_oneshot_kernel(Comm c, size_t off, long long nvec, float scale, int contribute) {
  __shared__ int flag[2];
  signal_pad(c, START_PAD, c.seq, contribute);
  uint32_t mask = 0;
  if (!wait_pad(c, START_PAD, c.seq, &mask, flag)) return;
  uint4 out[ONE_SHOT_VPT];
#pragma unroll
  for (int u = 0; u < ONE_SHOT_VPT; ++u) {
    const long long i = threadIdx.x + static_cast<long long>(u) * ONE_SHOT_THREADS;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        const int p = (c.rank + k) % c.world;
        if (mask & (1u << p)) Vec<T>::add(acc, ld_peer_v4(c.heap[p] + off + i * 16));
      }
    }
    out[u] = Vec<T>::pack(acc, scale);
  }
  __syncthreads();  // every thread of this rank holds its sums: tell the peers, wait for theirs
  signal_pad(c, END_PAD, c.seq, 0);
  if (!wait_pad(c, END_PAD, c.seq, nullptr, flag)) return;
#pragma unroll
  for (int u = 0; u < ONE_SHOT_VPT; ++u) {
    const long long i = threadIdx.x + static_cast<long long>(u) * ONE_SHOT_THREADS;
    if (i < nvec) *reinterpret_cast<uint4*>(c.heap[c.rank] + off + i * 16) = out[u];
  }
}

// Slice r = vectors [r*slice_vec, (r+1)*slice_vec) of the buffer at `off`.
template <typename T>
__global__ void __launch_bounds__(512)
reduce_scatter_kernel(Comm c, size_t off, long long slice_vec, float scale) {
  __shared__ int flag[2];
  if (blockIdx.x == 0) signal_pad(c, START_PAD, c.seq, 1);
  if (!wait_pad(c, START_PAD, c.seq, nullptr, flag)) return;
  const size_t base = off + static_cast<size_t>(c.rank) * slice_vec * 16;
  // UNR * world peer loads are in flight per thread before the first add (see allreduce_kernel)
  constexpr int UNR = 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < slice_vec;
       i0 += stride * UNR) {
    uint4 in[UNR][MAX_RANKS];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        const int p = (c.rank + k) % c.world;
        in[u][k] = make_uint4(0, 0, 0, 0);
        if (i < slice_vec) in[u][k] = ld_peer_v4(c.heap[p] + base + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      if (i >= slice_vec) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        Vec<T>::add(acc, in[u][k]);
      }
      *reinterpret_cast<uint4*>(c.heap[c.rank] + base + i * 16) = Vec<T>::pack(acc, scale);
    }
  }
  finish(c, flag);
}

// Local half of the copy-engine reduce-scatter: own slice + (world - 1) staged slices, summed in the
// same order as reduce_scatter_kernel (own first, then rank+1, rank+2, ...), so both give the same bits.
template <typename T>
__global__ void __launch_bounds__(512)
sum_staged_kernel(uint8_t* __restrict__ own, const uint8_t* __restrict__ staged, long long slice_vec, int others,
                  float scale) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < slice_vec; i += stride) {
    uint4 in[MAX_RANKS];
    in[0] = *reinterpret_cast<const uint4*>(own + i * 16);
#pragma unroll
    for (int k = 1; k < MAX_RANKS; ++k) {
      if (k > others) break;
      in[k] = *reinterpret_cast<const uint4*>(staged + (static_cast<size_t>(k - 1) * slice_vec + i) * 16);
    }
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < MAX_RANKS; ++k) {
      if (k > others) break;
      Vec<T>::add(acc, in[k]);
    }
    *reinterpret_cast<uint4*>(own + i * 16) = Vec<T>::pack(acc, scale);
  }
}

__global__ void __launch_bounds__(512)
all_gather_kernel(Comm c, size_t off, long long slice_vec) {
  __shared__ int flag[2];
  if (blockIdx.x == 0) signal_pad(c, START_PAD, c.seq, 1);
  if (!wait_pad(c, START_PAD, c.seq, nullptr, flag)) return;
  const size_t base = off + static_cast<size_t>(c.rank) * slice_vec * 16;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < slice_vec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint4 v = *reinterpret_cast<const uint4*>(c.heap[c.rank] + base + i * 16);
#pragma unroll
    for (int k = 1; k < MAX_RANKS; ++k) {
      if (k >= c.world) break;
      const int p = (c.rank + k) % c.world;
      *reinterpret_cast<uint4*>(c.heap[p] + base + i * 16) = v;
    }
  }
  finish(c, flag);
}

// Root's buffer is copied into every peer (pull by the peers).
__global__ void __launch_bounds__(512)
broadcast_kernel(Comm c, size_t off, long long nvec, int root) {
  __shared__ int flag[2];
  if (blockIdx.x == 0) signal_pad(c, START_PAD, c.seq, 1);
  if (!wait_pad(c, START_PAD, c.seq, nullptr, flag)) return;
  if (c.rank != root) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      *reinterpret_cast<uint4*>(c.heap[c.rank] + off + i * 16) = ld_peer_v4(c.heap[root] + off + i * 16);
  }
  finish(c, flag);
}

__global__ void barrier_kernel(Comm c) {
  __shared__ int flag[2];
  if (blockIdx.x == 0) signal_pad(c, START_PAD, c.seq, 1);
  if (!wait_pad(c, START_PAD, c.seq, nullptr, flag)) return;
  finish(c, flag);
}

// ---------------------------------------------------------------- DiLoCo outer step, one kernel
// Phase 1 (like the allreduce): rank r loads vectors of chunk r of the LOCAL weights from every
// contributing replica, forms the averaged pseudo-gradient  mean_p(local_p) - global  in fp32 and
// stores it (rounded to the weight type) into chunk r of every replica's gradient buffer.
// Then all blocks of all replicas meet: the last block of a rank runs the end hand-shake with the
// peers and releases the rank's other blocks through `phase_flag` (every block is resident: the
// grid is at most one block per SM and goes out as a cooperative launch; nothing else should be
// queued to run beside it, since a cooperative grid waits until all of its blocks fit).
// Phase 2 (local): Nesterov momentum and the new global weights for the WHOLE buffer,
//     b = first ? g : mu * buf + g;   step = nesterov ? g + mu * b : b;   w = global - lr * step
// written to `global_out` / `mom_out`, which the host swaps in only if the step commits.
struct OuterArgs {
  size_t off_local, off_g;
  const void* global_in;
  const float* mom_in;
  void* global_out;
  float* mom_out;
  long long nvec;
  float inv_n, lr, mu;
  int nesterov, first, contribute;
  uint32_t* phase_flag;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(512)
diloco_outer_kernel(Comm c, OuterArgs a) {
  __shared__ int flag[2];
  __shared__ int is_last;
  constexpr int N = Vec<T>::N;
  if (blockIdx.x == 0) signal_pad(c, START_PAD, c.seq, a.contribute);
  uint32_t mask = 0;
  if (!wait_pad(c, START_PAD, c.seq, &mask, flag)) return;
  const long long per = (a.nvec + c.world - 1) / c.world;
  const long long lo = per * c.rank;
  const long long hi = lo + per < a.nvec ? lo + per : a.nvec;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const uint4* gin = static_cast<const uint4*>(a.global_in);
  constexpr int UNR = 2;
  for (long long i0 = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < hi; i0 += stride * UNR) {
    uint4 in[UNR][MAX_RANKS];
    uint4 gl[UNR];
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      gl[u] = make_uint4(0, 0, 0, 0);
      if (i < hi) gl[u] = gin[i];
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        const int p = (c.rank + k) % c.world;
        in[u][k] = make_uint4(0, 0, 0, 0);
        if (i < hi && (mask & (1u << p))) in[u][k] = ld_peer_v4(c.heap[p] + a.off_local + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < UNR; ++u) {
      const long long i = i0 + u * stride;
      if (i >= hi) break;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        Vec<T>::add(acc, in[u][k]);
      }
      float gw[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      Vec<T>::add(gw, gl[u]);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = acc[j] * a.inv_n - gw[j];
      const uint4 out = Vec<T>::pack(acc, 1.f);
#pragma unroll
      for (int k = 0; k < MAX_RANKS; ++k) {
        if (k >= c.world) break;
        const int p = (c.rank + k) % c.world;
        *reinterpret_cast<uint4*>(c.heap[p] + a.off_g + i * 16) = out;
      }
    }
  }
  // ---- every block of every replica has finished phase 1 before anyone reads its gradient buffer
  const uint32_t go = flag_value(c.epoch, c.seq, 1), stop = flag_value(c.epoch, c.seq, 0);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* counter = reinterpret_cast<uint32_t*>(c.heap[c.rank]) + c.pad_base + DONE_COUNTER;
    const uint32_t ticket = atomicAdd(counter, 1u);
    is_last = (ticket == gridDim.x - 1);
    if (is_last) *counter = 0;
  }
  __syncthreads();
  if (is_last) {
    signal_pad(c, END_PAD, c.seq, 0);
    const bool ok = wait_pad(c, END_PAD, c.seq, nullptr, flag);
    if (threadIdx.x == 0) st_release_gpu_u32(a.phase_flag, ok ? go : stop);
    if (!ok) return;
  } else {
    if (threadIdx.x == 0) {
      const unsigned long long t0 = now_ns();
      uint32_t it = 0;
      int ok = 0;
      while (true) {
        const uint32_t v = ld_acquire_gpu_u32(a.phase_flag);
        if (v == go) { ok = 1; break; }
        if (v == stop) break;
        if ((++it & 63u) == 0) {
          if (c.abort_word && *c.abort_word) {
            if (c.status) atomicCAS(c.status, 0, static_cast<int>(kAborted));
            break;
          }
          if (now_ns() - t0 > 2 * c.budget_ns) {  // the last block itself may wait a full budget for the peers
            if (c.status) atomicCAS(c.status, 0, static_cast<int>(kTimeoutPeer));
            break;
          }
          __nanosleep(100);
        }
      }
      flag[0] = ok;
    }
    __syncthreads();
    if (!flag[0]) return;
  }
  // ---- phase 2: local update of the whole buffer
  const float4* min4 = reinterpret_cast<const float4*>(a.mom_in);
  float4* mout4 = reinterpret_cast<float4*>(a.mom_out);
  uint4* gout = static_cast<uint4*>(a.global_out);
  // two vectors per thread and round: all loads of both are issued before the arithmetic
  constexpr int UNR2 = 2;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < a.nvec; i0 += stride * UNR2) {
    uint4 gv[UNR2], wv[UNR2];
    float4 mv[UNR2][N / 4];
#pragma unroll
    for (int u = 0; u < UNR2; ++u) {
      const long long i = i0 + u * stride;
      gv[u] = wv[u] = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int q = 0; q < N / 4; ++q) mv[u][q] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < a.nvec) {
        gv[u] = ld_peer_v4(c.heap[c.rank] + a.off_g + i * 16);
        wv[u] = gin[i];
        if (a.mu != 0.f && !a.first) {
#pragma unroll
          for (int q = 0; q < N / 4; ++q) mv[u][q] = min4[i * (N / 4) + q];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNR2; ++u) {
      const long long i = i0 + u * stride;
      if (i >= a.nvec) break;
      float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      Vec<T>::add(g, gv[u]);
      Vec<T>::add(w, wv[u]);
      if (a.mu != 0.f) {
        float b[8];
#pragma unroll
        for (int q = 0; q < N / 4; ++q) {
          b[4 * q] = mv[u][q].x; b[4 * q + 1] = mv[u][q].y; b[4 * q + 2] = mv[u][q].z; b[4 * q + 3] = mv[u][q].w;
        }
#pragma unroll
        for (int j = 0; j < N; ++j) {
          b[j] = a.first ? g[j] : a.mu * b[j] + g[j];
          const float step = a.nesterov ? g[j] + a.mu * b[j] : b[j];
          w[j] -= a.lr * step;
        }
#pragma unroll
        for (int q = 0; q < N / 4; ++q)
          mout4[i * (N / 4) + q] = make_float4(b[4 * q], b[4 * q + 1], b[4 * q + 2], b[4 * q + 3]);
      } else {
#pragma unroll
        for (int j = 0; j < N; ++j) w[j] -= a.lr * g[j];
      }
      gout[i] = Vec<T>::pack(w, 1.f);
    }
  }
}

static int grid_for(long long nvec, int max_blocks) {
  long long b = (nvec + 511) / 512;
  if (b < 1) b = 1;
  if (b > max_blocks) b = max_blocks;
  return static_cast<int>(b);
}

}  // namespace p2p
}  // namespace tft

using namespace tft::p2p;

TFT_API long long tft_p2p_header_bytes() { return static_cast<long long>(HEADER_BYTES); }

// Allocates a heap (zero-filled) and returns its 64-byte IPC handle.
TFT_API int tft_p2p_heap_alloc(long long bytes, void** ptr, unsigned char* handle64) {
  cudaError_t e = cudaMalloc(ptr, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemset(*ptr, 0, static_cast<size_t>(bytes));
  if (e != cudaSuccess) return static_cast<int>(e);
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
TFT_API int tft_p2p_heap_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }

TFT_API int tft_p2p_peer_open(const unsigned char* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
TFT_API int tft_p2p_peer_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }

// Pinned host word that kernels poll; the host sets it to 1 to abort waits.
TFT_API int tft_p2p_abort_word_alloc(int** host_ptr, int** dev_ptr) {
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(host_ptr), sizeof(int), cudaHostAllocMapped);
  if (e != cudaSuccess) return static_cast<int>(e);
  **host_ptr = 0;
  return static_cast<int>(cudaHostGetDevicePointer(reinterpret_cast<void**>(dev_ptr), *host_ptr, 0));
}

// Clears one channel of the own heap's signalling header (called at reconfigure, before the
// peers are told about the new membership).
TFT_API int tft_p2p_reset_channel(void* heap, int channel, cudaStream_t stream) {
  if (channel < 0 || channel >= 16) return -1;
  return static_cast<int>(cudaMemsetAsync(static_cast<uint8_t*>(heap) + channel * CHANNEL_WORDS * 4, 0,
                                          CHANNEL_WORDS * 4, stream));
}

// dtype: 0 = bf16, 1 = fp32.  Buffer: `bytes` at heap offset `off` (both multiples of 16).
TFT_API int tft_p2p_allreduce(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                              const int* abort_word, int* status, long long off, long long bytes, int dtype,
                              float scale, int contribute, int max_blocks, cudaStream_t stream) {
  if ((off | bytes) & 15) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const long long nvec = bytes / 16;
  const int grid = grid_for((nvec + world - 1) / world, max_blocks);
  if (dtype == 0)
    allreduce_kernel<__nv_bfloat16><<<grid, 512, 0, stream>>>(c, static_cast<size_t>(off), nvec, scale, contribute);
  else
    allreduce_kernel<float><<<grid, 512, 0, stream>>>(c, static_cast<size_t>(off), nvec, scale, contribute);
  return static_cast<int>(cudaGetLastError());
}

// The one-shot variant; bytes <= tft_p2p_allreduce_oneshot_max().  Every member must pick the same variant.
TFT_API long long tft_p2p_allreduce_oneshot_max() { return ONE_SHOT_MAX_VEC * 16; }
TFT_API int tft_p2p_allreduce_oneshot(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq,
                                      int timeout_ms, const int* abort_word, int* status, long long off, long long bytes,
                                      int dtype, float scale, int contribute, cudaStream_t stream) {
  if ((off | bytes) & 15) return -1;
  if (bytes > ONE_SHOT_MAX_VEC * 16) return -6;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const long long nvec = bytes / 16;
  if (dtype == 0)
    allreduce_oneshot_kernel<__nv_bfloat16><<<1, ONE_SHOT_THREADS, 0, stream>>>(c, static_cast<size_t>(off), nvec, scale, contribute);
  else
    allreduce_oneshot_kernel<float><<<1, ONE_SHOT_THREADS, 0, stream>>>(c, static_cast<size_t>(off), nvec, scale, contribute);
  return static_cast<int>(cudaGetLastError());
}

// The buffer holds `world` slices of slice_bytes each; rank r ends with the scaled sum in slice r.
TFT_API int tft_p2p_reduce_scatter(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq,
                                   int timeout_ms, const int* abort_word, int* status, long long off,
                                   long long slice_bytes, int dtype, float scale, int max_blocks,
                                   cudaStream_t stream) {
  if ((off | slice_bytes) & 15) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const long long nvec = slice_bytes / 16;
  const int grid = grid_for(nvec, max_blocks);
  if (dtype == 0)
    reduce_scatter_kernel<__nv_bfloat16><<<grid, 512, 0, stream>>>(c, static_cast<size_t>(off), nvec, scale);
  else
    reduce_scatter_kernel<float><<<grid, 512, 0, stream>>>(c, static_cast<size_t>(off), nvec, scale);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_p2p_all_gather(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                               const int* abort_word, int* status, long long off, long long slice_bytes,
                               int max_blocks, cudaStream_t stream) {
  if ((off | slice_bytes) & 15) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const long long nvec = slice_bytes / 16;
  all_gather_kernel<<<grid_for(nvec, max_blocks), 512, 0, stream>>>(c, static_cast<size_t>(off), nvec);
  return static_cast<int>(cudaGetLastError());
}

// Reduce-scatter with the data movement on the copy engines: a barrier kernel (one block; every
// rank's buffer is final), world - 1 cudaMemcpyAsync pulls of this rank's slice out of the peers'
// buffers into a local staging area (`stage`, (world - 1) * slice_bytes, need not be in the heap), a
// local kernel that adds own + staged slices in fp32 and scales, and -- if `closing` -- a second
// barrier after which the peers may overwrite their buffers.  SMs only run the local sum, which is
// bound by this GPU's HBM and short; nothing spins on NVLink loads beside the GEMMs.
// Takes sequence numbers seq (and seq + 1 with `closing`).
TFT_API int tft_p2p_reduce_scatter_ce(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq,
                                      int timeout_ms, const int* abort_word, int* status, long long off,
                                      long long slice_bytes, int dtype, float scale, void* stage, int closing,
                                      int max_blocks, cudaStream_t stream) {
  if ((off | slice_bytes) & 15 || (reinterpret_cast<uintptr_t>(stage) & 15)) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  const size_t mine = static_cast<size_t>(off) + static_cast<size_t>(rank) * static_cast<size_t>(slice_bytes);
  for (int k = 1; k < world; ++k) {
    const int p = (rank + k) % world;
    e = cudaMemcpyAsync(static_cast<uint8_t*>(stage) + static_cast<size_t>(k - 1) * slice_bytes, c.heap[p] + mine,
                        static_cast<size_t>(slice_bytes), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const long long nvec = slice_bytes / 16;
  const int grid = grid_for(nvec, max_blocks);
  if (dtype == 0)
    sum_staged_kernel<__nv_bfloat16><<<grid, 512, 0, stream>>>(c.heap[rank] + mine, static_cast<const uint8_t*>(stage),
                                                               nvec, world - 1, scale);
  else
    sum_staged_kernel<float><<<grid, 512, 0, stream>>>(c.heap[rank] + mine, static_cast<const uint8_t*>(stage), nvec,
                                                       world - 1, scale);
  e = cudaGetLastError();
  if (e != cudaSuccess || !closing) return static_cast<int>(e);
  c.seq = seq + 1;
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  return static_cast<int>(cudaGetLastError());
}

// Allreduce (+ scale) with the data movement on the copy engines, for buffers large enough that
// three one-block barriers do not matter: two-shot like allreduce_kernel, i.e. rank r reduces chunk r
// and everybody collects the reduced chunks.
//   barrier | pull chunk r of every peer into `stage` | local sum of own + staged, scaled, into own chunk r
//   barrier | pull the reduced chunk p from every peer p into the own buffer | barrier
// `stage`: (world - 1) * ceil(nvec / world) * 16 bytes of local memory.  A rank that must not
// contribute zeroes its buffer before the call (the host wrapper does).  Takes sequence numbers seq,
// seq + 1 and seq + 2.
TFT_API int tft_p2p_allreduce_ce(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                                 const int* abort_word, int* status, long long off, long long bytes, int dtype,
                                 float scale, void* stage, int max_blocks, cudaStream_t stream) {
  if ((off | bytes) & 15 || (reinterpret_cast<uintptr_t>(stage) & 15)) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const long long nvec = bytes / 16;
  const long long per = (nvec + world - 1) / world;
  auto lo = [&](int r) { return per * r < nvec ? per * r : nvec; };  // chunk r = vectors [lo(r), lo(r + 1))
  auto len = [&](int r) { return lo(r + 1) - lo(r); };
  cudaError_t e;
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  const long long mine = len(rank);
  if (mine > 0) {
    for (int k = 1; k < world; ++k) {
      const int p = (rank + k) % world;
      e = cudaMemcpyAsync(static_cast<uint8_t*>(stage) + static_cast<size_t>(k - 1) * mine * 16,
                          c.heap[p] + off + lo(rank) * 16, static_cast<size_t>(mine) * 16, cudaMemcpyDeviceToDevice, stream);
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    const int grid = grid_for(mine, max_blocks);
    if (dtype == 0)
      sum_staged_kernel<__nv_bfloat16><<<grid, 512, 0, stream>>>(c.heap[rank] + off + lo(rank) * 16,
                                                                 static_cast<const uint8_t*>(stage), mine, world - 1, scale);
    else
      sum_staged_kernel<float><<<grid, 512, 0, stream>>>(c.heap[rank] + off + lo(rank) * 16,
                                                         static_cast<const uint8_t*>(stage), mine, world - 1, scale);
    if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  }
  c.seq = seq + 1;
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  if ((e = cudaGetLastError()) != cudaSuccess) return static_cast<int>(e);
  for (int k = 1; k < world; ++k) {
    const int p = (rank + k) % world;
    if (len(p) <= 0) continue;
    e = cudaMemcpyAsync(c.heap[rank] + off + lo(p) * 16, c.heap[p] + off + lo(p) * 16, static_cast<size_t>(len(p)) * 16,
                        cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  c.seq = seq + 2;
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  return static_cast<int>(cudaGetLastError());
}

// All-gather by the copy engines: a barrier kernel (one block), world - 1 peer copies issued with
// cudaMemcpyAsync, a second barrier kernel.  No SM moves data, so a GEMM that runs beside it keeps
// its SMs, its issue slots and its share of the power budget.  `pull` != 0: this rank copies every
// peer's slice into its own buffer (all of this rank's data is local once its copies are done; the
// closing barrier only tells the peers that their slice is no longer being read).  `pull` == 0: this
// rank copies its slice into every peer's buffer (the closing barrier is what makes the received
// slices final).  Takes TWO sequence numbers: seq and seq + 1.
TFT_API int tft_p2p_all_gather_ce(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq,
                                  int timeout_ms, const int* abort_word, int* status, long long off,
                                  long long slice_bytes, int pull, cudaStream_t stream) {
  if ((off | slice_bytes) & 15) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  for (int k = 1; k < world; ++k) {
    const int p = (rank + k) % world;
    const int owner = pull ? p : rank;          // whose slice moves
    const int from = pull ? p : rank, to = pull ? rank : p;
    const size_t at = static_cast<size_t>(off) + static_cast<size_t>(owner) * static_cast<size_t>(slice_bytes);
    e = cudaMemcpyAsync(c.heap[to] + at, c.heap[from] + at, static_cast<size_t>(slice_bytes),
                        cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  c.seq = seq + 1;
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_p2p_broadcast(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                              const int* abort_word, int* status, long long off, long long bytes, int root,
                              int max_blocks, cudaStream_t stream) {
  if ((off | bytes) & 15) return -1;
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  const long long nvec = bytes / 16;
  broadcast_kernel<<<grid_for(nvec, max_blocks), 512, 0, stream>>>(c, static_cast<size_t>(off), nvec, root);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_p2p_barrier(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                            const int* abort_word, int* status, cudaStream_t stream) {
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  barrier_kernel<<<1, 32, 0, stream>>>(c);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// Live-recovery copy: a recovering rank pulls state straight out of a healthy peer's heap.
// No flags are involved (the control plane holds the source's checkpoint gate open while
// the copy runs), so the kernel contains no wait at all.
namespace tft {
namespace p2p {

__global__ void __launch_bounds__(512) pull_copy_kernel(uint8_t* __restrict__ dst, const uint8_t* src, long long nvec) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    *reinterpret_cast<uint4*>(dst + i * 16) = ld_peer_v4(src + i * 16);
}

}  // namespace p2p
}  // namespace tft

// dst: local device memory, src: peer-mapped device memory; both 16-byte aligned, bytes % 16 == 0.
TFT_API int tft_p2p_pull(void* dst, const void* src, long long bytes, int max_blocks, cudaStream_t stream) {
  if ((bytes & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) return -1;
  if (bytes == 0) return 0;
  const long long nvec = bytes / 16;
  tft::p2p::pull_copy_kernel<<<grid_for(nvec, max_blocks), 512, 0, stream>>>(
      static_cast<uint8_t*>(dst), static_cast<const uint8_t*>(src), nvec);
  return static_cast<int>(cudaGetLastError());
}

// The same copy by a copy engine instead of SMs: one cudaMemcpyAsync from the peer's mapped heap.
// Large transfers run at the link rate this way and leave the SMs alone; no alignment rule.
TFT_API int tft_p2p_pull_ce(void* dst, const void* src, long long bytes, cudaStream_t stream) {
  if (bytes <= 0) return 0;
  return static_cast<int>(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, stream));
}


// DiLoCo outer step fused with its allreduce (see diloco_outer_kernel).  `off_local` / `off_g` are heap
// offsets of the local weights and of the gradient buffer (n elements each, 16-byte aligned, padded
// to a multiple of 16 bytes); global_in/out and mom_in/out are ordinary device pointers of this rank.
// phase_flag: one device uint32 owned by the caller (any value on entry).
TFT_API int tft_diloco_outer(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                             const int* abort_word, int* status, long long off_local, long long off_g,
                             const void* global_in, const float* mom_in, void* global_out, float* mom_out,
                             long long n, int is_bf16, float inv_n, float lr, float mu, int nesterov, int first,
                             int contribute, unsigned* phase_flag, int max_blocks, cudaStream_t stream) {
  const long long bytes = n * (is_bf16 ? 2 : 4);
  if ((off_local | off_g) & 15) return -1;
  if ((reinterpret_cast<uintptr_t>(global_in) | reinterpret_cast<uintptr_t>(global_out) |
       reinterpret_cast<uintptr_t>(mom_in) | reinterpret_cast<uintptr_t>(mom_out)) & 15)
    return -1;
  if (bytes % 16) return -2;  // the caller pads its flat buffers
  Comm c = make_comm(heaps, rank, world, epoch, seq, timeout_ms, abort_word, status);
  OuterArgs a;
  a.off_local = static_cast<size_t>(off_local);
  a.off_g = static_cast<size_t>(off_g);
  a.global_in = global_in; a.mom_in = mom_in; a.global_out = global_out; a.mom_out = mom_out;
  a.nvec = bytes / 16;
  a.inv_n = inv_n; a.lr = lr; a.mu = mu; a.nesterov = nesterov; a.first = first; a.contribute = contribute;
  a.phase_flag = phase_flag;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  // All blocks wait for one another between the phases, so all of them must be resident at the same
  // time.  A cooperative launch is what guarantees that: the grid starts only once every block has a
  // slot (it queues behind kernels that hold SMs instead of starting partially and spinning), and a
  // grid that can never fit is refused with an error.  Never more blocks than SMs.
  const void* fn = is_bf16 ? reinterpret_cast<const void*>(&diloco_outer_kernel<__nv_bfloat16>)
                           : reinterpret_cast<const void*>(&diloco_outer_kernel<float>);
  int per_sm = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, 512, 0);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (per_sm < 1) return static_cast<int>(cudaErrorCooperativeLaunchTooLarge);
  int grid = grid_for(a.nvec, max_blocks < sm_count ? max_blocks : sm_count);
  void* params[] = {&c, &a};
  e = cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(512), params, 0, stream);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// A slice of the symmetric heap as the backing store of a torch.cuda.MemPool, so that tensors which
// a library allocates by itself (the gradient buckets of torch's DistributedDataParallel) come to
// lie inside the heap and the peer-memory collectives can work on them in place.  torch's caching
// allocator asks for whole segments and keeps them, so a bump pointer is enough; released segments
// are not reused (the pool is meant to be filled once, at set-up).
namespace {
struct PoolRegion {
  uint8_t* base;
  size_t bytes, cursor;
};
PoolRegion g_pool[64] = {};
std::mutex g_pool_mu;
}  // namespace

TFT_API int tft_pool_bind(int device, void* base, long long bytes) {
  if (device < 0 || device >= 64 || bytes < 0 || (reinterpret_cast<uintptr_t>(base) & 511)) return -1;
  std::lock_guard<std::mutex> g(g_pool_mu);
  g_pool[device] = PoolRegion{static_cast<uint8_t*>(base), static_cast<size_t>(bytes), 0};
  return 0;
}
TFT_API long long tft_pool_used(int device) {
  if (device < 0 || device >= 64) return -1;
  std::lock_guard<std::mutex> g(g_pool_mu);
  return static_cast<long long>(g_pool[device].cursor);
}
// Signatures of torch.cuda.memory.CUDAPluggableAllocator.  A null result makes torch report out-of-memory.
TFT_API void* tft_pool_malloc(ssize_t size, int device, cudaStream_t) {
  if (device < 0 || device >= 64 || size < 0) return nullptr;
  std::lock_guard<std::mutex> g(g_pool_mu);
  PoolRegion& r = g_pool[device];
  const size_t need = (static_cast<size_t>(size) + 511) & ~static_cast<size_t>(511);
  if (r.base == nullptr || r.cursor + need > r.bytes) {
    std::fprintf(stderr, "torchft_b200: heap pool of device %d exhausted (%zu of %zu bytes used, %zu asked)\n", device,
                 r.cursor, r.bytes, need);
    return nullptr;
  }
  void* p = r.base + r.cursor;
  r.cursor += need;
  return p;
}
TFT_API void tft_pool_free(void*, size_t, int, cudaStream_t) {}
