// RMSNorm (forward with optional fused residual add, backward with weight-gradient
// partial sums) and rotary position embedding for bf16 activations.
//
// All kernels are bandwidth bound: every tensor is read once and written once, with
// 16-byte vector accesses, and row statistics stay in registers / shared memory.
#include "common.cuh"
#include "tft_noalloc.h"

#include <atomic>
#include <cstdio>

namespace tft {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the block; result valid in every thread.  `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  return u;
}

// One block per row.  VPT = 16-byte vectors per thread (dim = blockDim.x * 8 * VPT).
//   h = x (+ res);  y = h * rstd * w;  optionally writes h (when res != nullptr) and rstd.
template <int VPT>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ h_out, float* __restrict__ rstd_out, int dim,
                                   float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
  const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * dim) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float v[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    unpack8(xr[idx], v[i]);
    if (rr) {
      float r[8];
      unpack8(rr[idx], r);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] += r[j];
      // the residual stream is stored in bf16: normalise exactly what later layers will read
      uint4 hv = pack8(v[i]);
      reinterpret_cast<uint4*>(h_out + row * dim)[idx] = hv;
      unpack8(hv, v[i]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / dim + eps);
  if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    float wv[8], o[8];
    unpack8(wr[idx], wv);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = v[i][j] * rstd * wv[j];
    reinterpret_cast<uint4*>(y + row * dim)[idx] = pack8(o);
  }
}

// Backward.  Each block walks rows blockIdx.x, blockIdx.x + gridDim.x, ...
//   g = dy * w;  dx = rstd * (g - xhat * mean(g * xhat)),  xhat = x * rstd
//   dx (+)= dres (gradient arriving on the residual path, optional)
//   dw_partial[block, :] = sum over its rows of dy * xhat      (fp32 scratch)
template <int VPT>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int rows, int dim) {
  __shared__ float red[32];
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  float wv[VPT][8], acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    unpack8(wr[threadIdx.x + i * blockDim.x], wv[i]);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  }
  for (size_t row = blockIdx.x; row < static_cast<size_t>(rows); row += gridDim.x) {
    const float rstd = rstd_in[row];
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      float d[8];
      unpack8(reinterpret_cast<const uint4*>(dy + row * dim)[idx], d);
      unpack8(reinterpret_cast<const uint4*>(x + row * dim)[idx], xh[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        xh[i][j] *= rstd;
        g[i][j] = d[j] * wv[i][j];
        dot += g[i][j] * xh[i][j];
        acc[i][j] += d[j] * xh[i][j];
      }
    }
    dot = block_sum(dot, red) / dim;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int idx = threadIdx.x + i * blockDim.x;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
      if (dres) {
        float r[8];
        unpack8(reinterpret_cast<const uint4*>(dres + row * dim)[idx], r);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += r[j];
      }
      reinterpret_cast<uint4*>(dx + row * dim)[idx] = pack8(o);
    }
  }
  float* out = dw_partial + static_cast<size_t>(blockIdx.x) * dim;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int idx = threadIdx.x + i * blockDim.x;
    float4* o4 = reinterpret_cast<float4*>(out + idx * 8);
    o4[0] = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    o4[1] = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
  }
}

// dw[c] (+)= sum_p partial[p, c].  A block of 256 threads covers 32 columns with 8 slices of the
// partial rows each (a warp reads 128 contiguous bytes per row), so dim / 32 blocks share the work.
__global__ void rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw,
                                         int parts, int dim, int accumulate) {
  __shared__ float acc[8][33];
  const int col = threadIdx.x & 31, slice = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + col;
  float s = 0.f;
  if (c < dim)
    for (int p = slice; p < parts; p += 8) s += partial[static_cast<size_t>(p) * dim + c];
  acc[slice][col] = s;
  __syncthreads();
  if (slice == 0 && c < dim) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += acc[k][col];
    if (accumulate) t += __bfloat162float(dw[c]);
    dw[c] = __float2bfloat16(t);
  }
}

// Rotary embedding in place on x[tokens, heads, hd], pairing element i with i + hd/2.
// cs[pos, hd/2] holds (cos, sin) as float2.  sign = -1 applies the inverse rotation
// (the backward pass).  One thread handles 8 consecutive pairs of one (token, head).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float2* __restrict__ cs,
                            const int* __restrict__ positions, int tokens, int heads, int hd, int row_stride,
                            float sign, int seq_len) {
  const int half = hd / 2;
  const int vec_per_head = half / 8;
  const long long total = static_cast<long long>(tokens) * heads * vec_per_head;
  const long long gid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (gid >= total) return;
  const int v = static_cast<int>(gid % vec_per_head);
  const int head = static_cast<int>((gid / vec_per_head) % heads);
  const int tok = static_cast<int>(gid / (static_cast<long long>(vec_per_head) * heads));
  const int pos = positions ? positions[tok] : (seq_len > 0 ? tok % seq_len : tok);
  __nv_bfloat16* base = x + static_cast<size_t>(tok) * row_stride + head * hd + v * 8;
  float a[8], b[8];
  unpack8(*reinterpret_cast<const uint4*>(base), a);
  unpack8(*reinterpret_cast<const uint4*>(base + half), b);
  const float2* c = cs + static_cast<size_t>(pos) * half + v * 8;
  float oa[8], ob[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float co = c[j].x, si = c[j].y * sign;
    oa[j] = a[j] * co - b[j] * si;
    ob[j] = b[j] * co + a[j] * si;
  }
  *reinterpret_cast<uint4*>(base) = pack8(oa);
  *reinterpret_cast<uint4*>(base + half) = pack8(ob);
}

__global__ void rope_table_kernel(float2* __restrict__ cs, int max_pos, int half, float theta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= max_pos * half) return;
  const int pos = i / half, j = i % half;
  const float inv = powf(theta, -static_cast<float>(j) / half);
  float s, c;
  sincosf(pos * inv, &s, &c);
  cs[i] = make_float2(c, s);
}

static int norm_config(int dim, int* threads) {
  // dim = threads * 8 * VPT with threads a multiple of 32 and <= 512
  for (int vpt = 1; vpt <= 4; ++vpt) {
    if (dim % (8 * vpt)) continue;
    const int t = dim / (8 * vpt);
    if (t % 32 == 0 && t <= 512) {
      *threads = t;
      return vpt;
    }
  }
  return 0;
}

}  // namespace tft

using namespace tft;

// Number of dw partial rows the backward writes (size the scratch as parts * dim floats).
TFT_API int tft_rmsnorm_bwd_parts(int rows) { return rows < 592 ? rows : 592; }

TFT_API int tft_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                            int rows, int dim, float eps, cudaStream_t stream) {
  int threads = 0;
  const int vpt = norm_config(dim, &threads);
  if (!vpt || rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(res);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto H = static_cast<__nv_bfloat16*>(h_out);
  switch (vpt) {
    case 1: rmsnorm_fwd_kernel<1><<<rows, threads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps); break;
    case 2: rmsnorm_fwd_kernel<2><<<rows, threads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps); break;
    case 3: rmsnorm_fwd_kernel<3><<<rows, threads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps); break;
    default: rmsnorm_fwd_kernel<4><<<rows, threads, 0, stream>>>(X, R, W, Y, H, rstd, dim, eps); break;
  }
  return static_cast<int>(cudaGetLastError());
}

// scratch: tft_rmsnorm_bwd_parts(rows) * dim floats.  dw (+)= when accumulate != 0.
TFT_API int tft_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                            void* dx, void* dw, float* scratch, int rows, int dim, int accumulate,
                            cudaStream_t stream) {
  int threads = 0;
  const int vpt = norm_config(dim, &threads);
  if (!vpt || rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  const int parts = tft_rmsnorm_bwd_parts(rows);
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  switch (vpt) {
    case 1: rmsnorm_bwd_kernel<1><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
    case 2: rmsnorm_bwd_kernel<2><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
    case 3: rmsnorm_bwd_kernel<3><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
    default: rmsnorm_bwd_kernel<4><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
  }
  rmsnorm_dw_reduce_kernel<<<(dim + 31) / 32, 256, 0, stream>>>(scratch, static_cast<__nv_bfloat16*>(dw), parts,
                                                                  dim, accumulate);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_rope_table(void* cs, int max_pos, int hd, float theta, cudaStream_t stream) {
  const int half = hd / 2;
  const int n = max_pos * half;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, stream>>>(static_cast<float2*>(cs), max_pos, half, theta);
  return static_cast<int>(cudaGetLastError());
}

// x: [tokens, heads, hd] with token stride row_stride elements; hd % 16 == 0.
TFT_API int tft_rope(void* x, const void* cs, const int* positions, int tokens, int heads, int hd,
                     int row_stride, int inverse, int seq_len, cudaStream_t stream) {
  if (hd % 16 || row_stride % 8) return static_cast<int>(cudaErrorInvalidValue);
  const long long total = static_cast<long long>(tokens) * heads * (hd / 16);
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  rope_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
      static_cast<__nv_bfloat16*>(x), static_cast<const float2*>(cs), positions, tokens, heads, hd, row_stride,
      inverse ? -1.f : 1.f, seq_len);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------
// RMSNorm backward for callers that cannot allocate device memory.
//
// tft_rmsnorm_bwd above needs a caller-provided fp32 scratch buffer for the per-block
// partial sums of the weight gradient.  Some callers have no way to provide one: code that
// runs inside a region where cudaMalloc is forbidden or would deadlock (for instance a
// callback of another library's allocator, or a plug-in that is handed raw pointers and a
// stream and nothing else).  For them the variant below keeps the scratch in a fixed array
// that is part of this library's device image.  Declared in tft_noalloc.h.
//
// Limits and sharing rules:
//   * dim <= kNoAllocMaxDim (8192); at most kNoAllocParts (148) partial rows are used, so
//     the array is 148 * 8192 * 4 bytes = 4.6 MiB.  Every GPU on which this library is
//     loaded holds that much until the process exits.
//   * All calls on one device share the array and it keeps the last call's contents.  The
//     backward kernel overwrites every partial row it later reads, so nothing has to be
//     cleared between calls; but two calls that overlap on the GPU (different streams)
//     race on it.  Issue them on one stream or order them yourself.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress).  Make that first call outside of any stream capture.
//   * The lookup is for the current device, which therefore has to be the device of `stream`;
//     a stream of another device is refused (-11).
//   * No cudaMalloc, cudaFree or allocating library routine is called, ever.
namespace tft {

constexpr int kNoAllocMaxDim = 8192;
constexpr int kNoAllocParts = 148;
constexpr int kNoAllocMaxDevices = 64;

static __device__ __align__(256) float g_noalloc_scratch[kNoAllocParts * kNoAllocMaxDim];

// Device address of g_noalloc_scratch per device ordinal.  In host code the symbol's name
// is only a host-side stand-in, so the address is resolved through the runtime, once per
// device, with that device current.
// Atomic because any host thread may make the first call on a device; racing threads store the same
// address, so whichever store lands last changes nothing.
static std::atomic<float*> g_noalloc_ptr[kNoAllocMaxDevices];

static int noalloc_scratch(float** out, cudaStream_t stream) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= kNoAllocMaxDevices) return static_cast<int>(cudaErrorInvalidDevice);
  int stream_dev = dev;
  if (cudaStreamGetDevice(stream, &stream_dev) == cudaSuccess && stream_dev != dev) {
    std::fprintf(stderr, "tft_rmsnorm_bwd_noalloc: stream belongs to device %d but device %d is current\n",
                 stream_dev, dev);
    return -11;
  }
  cudaGetLastError();  // a failed query must not linger as this thread's last error
  float* cached = g_noalloc_ptr[dev].load(std::memory_order_acquire);
  if (cached == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    cached = static_cast<float*>(p);
    g_noalloc_ptr[dev].store(cached, std::memory_order_release);
  }
  *out = cached;
  return 0;
}

}  // namespace tft

TFT_API int tft_rmsnorm_bwd_noalloc_max_dim() { return tft::kNoAllocMaxDim; }

// Same contract as tft_rmsnorm_bwd minus the scratch argument.  Returns 0 on success,
// -10 if dim exceeds tft_rmsnorm_bwd_noalloc_max_dim() (a message goes to stderr), another
// negative / CUDA error code otherwise.
TFT_API int tft_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                    const void* dres, void* dx, void* dw, int rows, int dim, int accumulate,
                                    cudaStream_t stream) {
  if (dim > kNoAllocMaxDim) {
    std::fprintf(stderr,
                 "tft_rmsnorm_bwd_noalloc: dim %d exceeds the built-in scratch (max %d); use tft_rmsnorm_bwd "
                 "with a caller-provided buffer\n",
                 dim, kNoAllocMaxDim);
    return -10;
  }
  int threads = 0;
  const int vpt = norm_config(dim, &threads);
  if (!vpt || rows <= 0) return static_cast<int>(cudaErrorInvalidValue);
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch, stream);
  if (rc != 0) return rc;
  const int parts = rows < kNoAllocParts ? rows : kNoAllocParts;
  auto DY = static_cast<const __nv_bfloat16*>(dy);
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto W = static_cast<const __nv_bfloat16*>(w);
  auto DR = static_cast<const __nv_bfloat16*>(dres);
  auto DX = static_cast<__nv_bfloat16*>(dx);
  switch (vpt) {
    case 1: rmsnorm_bwd_kernel<1><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
    case 2: rmsnorm_bwd_kernel<2><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
    case 3: rmsnorm_bwd_kernel<3><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
    default: rmsnorm_bwd_kernel<4><<<parts, threads, 0, stream>>>(DY, X, W, rstd, DR, DX, scratch, rows, dim); break;
  }
  rmsnorm_dw_reduce_kernel<<<(dim + 31) / 32, 256, 0, stream>>>(scratch, static_cast<__nv_bfloat16*>(dw), parts,
                                                                  dim, accumulate);
  return static_cast<int>(cudaGetLastError());
}
