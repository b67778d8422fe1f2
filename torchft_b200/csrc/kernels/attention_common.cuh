// Shared pieces of the tcgen05 flash-attention kernels (causal, grouped-query).
//
// Tiles are 128 query rows x 128 key rows.  Every operand tile lives in shared memory as
// 64-column sub-tiles of [128 rows x 128 bytes] with the 128-byte swizzle, which is what a
// TMA box of {64 elements, 1 head, 128 rows, 1 batch} produces.  The same bytes serve as
// a K-major operand (contraction over the head dimension) or as an MN-major operand
// (contraction over the 128 rows); only the descriptor differs.
#pragma once

#include "common.cuh"
#include "tensormap.cuh"

namespace tft {
namespace attn {

constexpr int BLK = 128;          // rows per tile (queries and keys)
constexpr int SUB_BYTES = 16384;  // one [128 x 64] bf16 sub-tile

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Loads a [128 rows x HD] tile of head `head`, rows row0.. of batch `batch` as HD/64 sub-tiles.
template <int HD>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int head, int row0,
                                          int batch) {
#pragma unroll
  for (int s = 0; s < HD / 64; ++s) tma_load_4d(dst + s * SUB_BYTES, tmap, bar, s * 64, head, row0, batch);
}

// Descriptor of k-step `k` (16 elements of the contraction) for a K-major operand whose
// contraction dimension spans the 64-column sub-tiles.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t base, int k) {
  return make_smem_desc(base + (k >> 2) * SUB_BYTES + (k & 3) * 32, 16, 1024);
}
// Descriptor of k-step `k` (16 ROWS of the tile) for an MN-major operand: the M/N extent
// runs along the columns (64 per sub-tile, next sub-tile SUB_BYTES further).
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t base, int k) {
  return make_smem_desc(base + k * 2048, SUB_BYTES, 1024);
}

// Byte offset of the 16-byte chunk holding columns [col8*8, col8*8+8) of row `row` inside a
// [128 x 128] bf16 tile stored as two swizzled sub-tiles.
__device__ __forceinline__ uint32_t swizzled_chunk(int row, int col8) {
  const int sub = col8 >> 3;
  const int ch = col8 & 7;
  return sub * SUB_BYTES + row * 128 + ((ch ^ (row & 7)) << 4);
}

__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ------------------------------------------------------------------ delta
template <int HD>
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, int B, int S, int Hq) {
  const long long gw = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * S * Hq;
  if (gw >= total) return;
  const int h = static_cast<int>(gw % Hq);
  const long long tok = gw / Hq;
  const int s = static_cast<int>(tok % S);
  const int b = static_cast<int>(tok / S);
  const __nv_bfloat16* o = O + (tok * Hq + h) * HD;
  const __nv_bfloat16* d = dO + (tok * Hq + h) * HD;
  float acc = 0.f;
  for (int i = lane * 2; i < HD; i += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + i));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d + i));
    acc += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0) delta[(static_cast<long long>(b) * Hq + h) * S + s] = acc;
}

// Writes 32 consecutive values of row r (columns c*32 .. c*32+31) as bf16 into a swizzled tile.
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int r, int c, const float (&v)[32]) {
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    uint4 u;
    u.x = pack_bf16(v[t * 8 + 0], v[t * 8 + 1]);
    u.y = pack_bf16(v[t * 8 + 2], v[t * 8 + 3]);
    u.z = pack_bf16(v[t * 8 + 4], v[t * 8 + 5]);
    u.w = pack_bf16(v[t * 8 + 6], v[t * 8 + 7]);
    *reinterpret_cast<uint4*>(tile + swizzled_chunk(r, c * 4 + t)) = u;
  }
}

// Drains a [128 x HD] fp32 accumulator from tensor memory into global bf16 rows.
template <int HD>
__device__ __forceinline__ void store_acc(uint32_t taddr, __nv_bfloat16* dst, float mul, bool valid) {
#pragma unroll 1
  for (int c = 0; c < HD / 32; ++c) {
    uint32_t a[32];
    tmem_ld_32x32(taddr + c * 32, a);
    tmem_ld_wait();
    if (valid) {
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        uint4 u;
        u.x = pack_bf16(__uint_as_float(a[t * 8 + 0]) * mul, __uint_as_float(a[t * 8 + 1]) * mul);
        u.y = pack_bf16(__uint_as_float(a[t * 8 + 2]) * mul, __uint_as_float(a[t * 8 + 3]) * mul);
        u.z = pack_bf16(__uint_as_float(a[t * 8 + 4]) * mul, __uint_as_float(a[t * 8 + 5]) * mul);
        u.w = pack_bf16(__uint_as_float(a[t * 8 + 6]) * mul, __uint_as_float(a[t * 8 + 7]) * mul);
        reinterpret_cast<uint4*>(dst + c * 32)[t] = u;
      }
    }
  }
}

// 4-D tensor map over x[batch, seq, heads, HD] (token stride `ld` elements) with boxes of
// {64, 1, 128, 1}.
inline bool make_attn_tensormap(CUtensorMap* out, const void* ptr, int hd, int heads, int seq, int batch,
                                long long ld) {
  auto fn = tensormap_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[4] = {static_cast<cuuint64_t>(hd), static_cast<cuuint64_t>(heads), static_cast<cuuint64_t>(seq),
                        static_cast<cuuint64_t>(batch)};
  cuuint64_t strides[3] = {static_cast<cuuint64_t>(hd) * 2, static_cast<cuuint64_t>(ld) * 2,
                           static_cast<cuuint64_t>(ld) * 2 * static_cast<cuuint64_t>(seq)};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  static thread_local bool context_bound = false;  // once per thread (not allowed during stream capture)
  if (!context_bound) {
    cudaFree(nullptr);  // binds the primary context on threads that have not used it yet
    context_bound = true;
  }
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace attn
}  // namespace tft
