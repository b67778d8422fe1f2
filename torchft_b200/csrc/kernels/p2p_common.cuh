// Shared pieces of the NVLink peer-memory kernels: the communicator descriptor, the flag
// encoding, and the bounded start / end handshakes on the header of every rank's heap.
#pragma once
#include "common.cuh"

namespace tft {
namespace p2p {

constexpr int MAX_RANKS = 8;
constexpr size_t HEADER_BYTES = 4096;  // start pad, end pad, block counter
// The header holds 16 independent channels of 64 uint32 each, so several communicators
// (shard group, replica group, ...) can share one heap without touching each other's flags.
constexpr int CHANNEL_WORDS = 64;
constexpr int START_PAD = 0;  // uint32 index inside a channel
constexpr int END_PAD = 16;
constexpr int DONE_COUNTER = 32;

struct Comm {
  uint8_t* heap[MAX_RANKS];
  int rank, world;
  int pad_base;  // first uint32 of this communicator's channel
  uint32_t epoch;
  uint32_t seq;
  unsigned long long budget_ns;
  const volatile int* abort_word;
  int* status;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_peer_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

__device__ __forceinline__ uint32_t flag_value(uint32_t epoch, uint32_t seq, uint32_t contrib) {
  return (epoch << 21) | ((seq & 0xFFFFFu) << 1) | (contrib & 1u);
}

// Waits until pad[p] (in this rank's own heap) carries (epoch, seq) for every peer.
// Threads 0..world-1 of the calling block poll; the result is block-uniform.
// contrib_mask receives one bit per peer.  Returns false on time-out or abort.
__device__ inline bool wait_pad(const Comm& c, int pad, uint32_t seq, uint32_t* contrib_mask, int* smem_flag) {
  if (threadIdx.x == 0) {
    // A communicator whose status word is set has already lost a peer in this membership: later
    // collectives fail at once instead of sitting out the budget again (configure clears the word).
    smem_flag[0] = (c.status && *reinterpret_cast<volatile int*>(c.status) != 0) ? 0 : 1;
    smem_flag[1] = 0;
  }
  __syncthreads();
  if (smem_flag[0] != 0 && threadIdx.x < c.world) {
    const uint32_t* slot = reinterpret_cast<const uint32_t*>(c.heap[c.rank]) + c.pad_base + pad + threadIdx.x;
    const uint32_t want = flag_value(c.epoch, seq, 0) >> 1;
    const unsigned long long t0 = now_ns();
    uint32_t it = 0;
    while (true) {
      const uint32_t v = ld_acquire_sys(slot);
      if ((v >> 1) == want) {
        if (v & 1u) atomicOr(&smem_flag[1], 1 << threadIdx.x);
        break;
      }
      if ((++it & 63u) == 0) {
        if (c.abort_word && *c.abort_word) {
          smem_flag[0] = 0;
          if (c.status) atomicCAS(c.status, 0, static_cast<int>(kAborted));
          break;
        }
        if (now_ns() - t0 > c.budget_ns) {
          smem_flag[0] = 0;
          if (c.status) atomicCAS(c.status, 0, static_cast<int>(kTimeoutPeer));
          break;
        }
      }
    }
  }
  __syncthreads();
  if (contrib_mask) *contrib_mask = static_cast<uint32_t>(smem_flag[1]);
  return smem_flag[0] != 0;
}

// Block 0 announces (epoch, seq, contrib) in the given pad of every peer.
__device__ __forceinline__ void signal_pad(const Comm& c, int pad, uint32_t seq, uint32_t contrib) {
  if (threadIdx.x < c.world) {
    uint32_t* slot = reinterpret_cast<uint32_t*>(c.heap[threadIdx.x]) + c.pad_base + pad + c.rank;
    st_release_sys(slot, flag_value(c.epoch, seq, contrib));
  }
}

inline Comm make_comm(void* const* heaps, int rank, int world, unsigned epoch, unsigned seq, int timeout_ms,
                      const int* abort_word, int* status) {
  Comm c;
  for (int i = 0; i < MAX_RANKS; ++i) c.heap[i] = i < world ? static_cast<uint8_t*>(heaps[i]) : nullptr;
  c.rank = rank;
  c.world = world;
  c.epoch = epoch & 0x7FFu;                                  // bits 0-10: membership epoch
  c.pad_base = static_cast<int>((epoch >> 16) & 0xFu) * CHANNEL_WORDS;  // bits 16-19: channel
  c.seq = seq;
  c.budget_ns = static_cast<unsigned long long>(timeout_ms) * 1000000ull;
  c.abort_word = abort_word;
  c.status = status;
  return c;
}

}  // namespace p2p
}  // namespace tft
