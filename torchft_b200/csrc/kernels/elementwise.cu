// Bandwidth-bound training kernels: SwiGLU, fused softmax cross-entropy (loss and
// gradient in one kernel), embedding gather / scatter-add, fused AdamW, and the DiLoCo
// outer step (pseudo-gradient, Nesterov update).  One pass over memory each, 16-byte
// vector accesses, fp32 math.
#include "common.cuh"

namespace tft {

__device__ __forceinline__ void ew_unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 ew_pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]);
  u.y = pack_bf16(f[2], f[3]);
  u.z = pack_bf16(f[4], f[5]);
  u.w = pack_bf16(f[6], f[7]);
  return u;
}

// ------------------------------------------------------------------ SwiGLU
// gu: [rows, 2*F] with the gate in columns [0,F) and the up projection in [F,2F).
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                  long long rows, int F) {
  const int vec_per_row = F / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    float g[8], u[8], o[8];
    ew_unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * F + c), g);
    ew_unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = g[j] / (1.f + __expf(-g[j])) * u[j];
    *reinterpret_cast<uint4*>(out + r * F + c) = ew_pack8(o);
  }
}

// dgu[:, :F] = dout * u * d silu(g);  dgu[:, F:] = dout * silu(g)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, long long rows, int F) {
  const int vec_per_row = F / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    ew_unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * F + c), g);
    ew_unpack8(*reinterpret_cast<const uint4*>(gu + r * 2 * F + F + c), u);
    ew_unpack8(*reinterpret_cast<const uint4*>(dout + r * F + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      const float silu = g[j] * s;
      du[j] = d[j] * silu;
      dg[j] = d[j] * u[j] * (s + silu * (1.f - s));
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + c) = ew_pack8(dg);
    *reinterpret_cast<uint4*>(dgu + r * 2 * F + F + c) = ew_pack8(du);
  }
}

// ------------------------------------------------------------------ cross entropy
// One block per row of logits [rows, V] (bf16).  Pass 1: online max / sum-exp.
// Pass 2 (in place): logits <- (softmax - onehot) * grad_scale.  loss[row] = lse - z_target.
// Rows whose target is ignore_index produce zero loss and zero gradient.
__global__ void xent_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets,
                            float* __restrict__ loss, int V, int ld, float grad_scale, long long ignore_index) {
  __shared__ float red_m[32], red_s[32];
  const size_t row = blockIdx.x;
  __nv_bfloat16* z = logits + row * ld;
  const long long tgt = targets[row];
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    ew_unpack8(reinterpret_cast<const uint4*>(z)[i], f);
    float lm = f[0];
#pragma unroll
    for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
    const float nm = fmaxf(m, lm);
    float ls = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ls += __expf(f[j] - nm);
    s = s * __expf(m - nm) + ls;
    m = nm;
  }
  // combine (m, s) pairs across the block
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
  __syncthreads();
  const int nw = blockDim.x >> 5;
  m = lane < nw ? red_m[lane] : -INFINITY;
  s = lane < nw ? red_s[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  const float lse = m + __logf(s);
  const bool ignored = tgt == ignore_index || tgt < 0 || tgt >= V;
  if (threadIdx.x == 0) loss[row] = ignored ? 0.f : lse - __bfloat162float(z[tgt]);
  __syncthreads();  // the target logit is read before it is overwritten below
  const float scale = ignored ? 0.f : grad_scale;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    float f[8];
    ew_unpack8(reinterpret_cast<const uint4*>(z)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] - lse);
      if (i * 8 + j == tgt) p -= 1.f;
      f[j] = p * scale;
    }
    reinterpret_cast<uint4*>(z)[i] = ew_pack8(f);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long n_tokens, int dim) {
  const int vec = dim / 8;
  const long long total = n_tokens * vec;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / vec;
    const int c = static_cast<int>(i % vec);
    reinterpret_cast<uint4*>(out + t * dim)[c] = reinterpret_cast<const uint4*>(table + tokens[t] * dim)[c];
  }
}

// dtable[tokens[t], :] += dout[t, :]   (bf16x2 atomics; dtable must be zeroed or hold earlier grads)
__global__ void embedding_bwd_kernel(const long long* __restrict__ tokens, const __nv_bfloat16* __restrict__ dout,
                                     __nv_bfloat16* __restrict__ dtable, long long n_tokens, int dim) {
  const int pairs = dim / 2;
  const long long total = n_tokens * pairs;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / pairs;
    const int c = static_cast<int>(i % pairs);
    const __nv_bfloat162 v = reinterpret_cast<const __nv_bfloat162*>(dout + t * dim)[c];
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + tokens[t] * dim) + c, v);
  }
}

// ------------------------------------------------------------------ AdamW
// p (bf16) updated in place from g (bf16) with fp32 moments; decoupled weight decay.
// bc1 = 1 - beta1^t, bc2 = 1 - beta2^t.  grad_scale multiplies g first (1/accumulation steps).
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2, float grad_scale) {
  const long long nvec = n / 8;
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float pf[8], gf[8];
    ew_unpack8(reinterpret_cast<const uint4*>(p)[i], pf);
    ew_unpack8(reinterpret_cast<const uint4*>(g)[i], gf);
    float4 m0 = reinterpret_cast<float4*>(m)[2 * i], m1 = reinterpret_cast<float4*>(m)[2 * i + 1];
    float4 v0 = reinterpret_cast<float4*>(v)[2 * i], v1 = reinterpret_cast<float4*>(v)[2 * i + 1];
    float mf[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vf[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gr = gf[j] * grad_scale;
      mf[j] = b1 * mf[j] + (1.f - b1) * gr;
      vf[j] = b2 * vf[j] + (1.f - b2) * gr * gr;
      const float denom = sqrtf(vf[j]) * inv_sqrt_bc2 + eps;
      pf[j] = pf[j] * (1.f - lr * wd) - lr * (mf[j] * inv_bc1) / denom;
    }
    reinterpret_cast<uint4*>(p)[i] = ew_pack8(pf);
    reinterpret_cast<float4*>(m)[2 * i] = make_float4(mf[0], mf[1], mf[2], mf[3]);
    reinterpret_cast<float4*>(m)[2 * i + 1] = make_float4(mf[4], mf[5], mf[6], mf[7]);
    reinterpret_cast<float4*>(v)[2 * i] = make_float4(vf[0], vf[1], vf[2], vf[3]);
    reinterpret_cast<float4*>(v)[2 * i + 1] = make_float4(vf[4], vf[5], vf[6], vf[7]);
  }
  // tail (n not a multiple of 8)
  const long long tail = nvec * 8 + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  if (tail < n) {
    const float gr = __bfloat162float(g[tail]) * grad_scale;
    const float mm = b1 * m[tail] + (1.f - b1) * gr;
    const float vv = b2 * v[tail] + (1.f - b2) * gr * gr;
    m[tail] = mm;
    v[tail] = vv;
    const float denom = sqrtf(vv) * inv_sqrt_bc2 + eps;
    p[tail] = __float2bfloat16(__bfloat162float(p[tail]) * (1.f - lr * wd) - lr * (mm * inv_bc1) / denom);
  }
}

// ------------------------------------------------------------------ DiLoCo outer step
template <typename T>
__device__ __forceinline__ float ld1(const T* p, long long i);
template <>
__device__ __forceinline__ float ld1<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld1<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void st1(T* p, long long i, float v);
template <>
__device__ __forceinline__ void st1<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st1<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

// local (in/out): on entry the local weights, on exit the pseudo-gradient local - global.
template <typename T>
__global__ void pseudograd_kernel(T* __restrict__ local, const T* __restrict__ global_w, long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    st1<T>(local, i, ld1<T>(local, i) - ld1<T>(global_w, i));
}

// g (in/out): averaged pseudo-gradient on entry, NEW global weights on exit.
// global_w (in/out): old -> new global weights.  buf: fp32 momentum.
template <typename T>
__global__ void nesterov_outer_kernel(T* __restrict__ g, T* __restrict__ global_w, float* __restrict__ buf,
                                      long long n, float lr, float mu, int nesterov, int first) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float grad = ld1<T>(g, i);
    float step = grad;
    if (mu != 0.f) {
      const float b = first ? grad : mu * buf[i] + grad;
      buf[i] = b;
      step = nesterov ? grad + mu * b : b;
    }
    const float w = ld1<T>(global_w, i) - lr * step;
    st1<T>(global_w, i, w);
    st1<T>(g, i, w);
  }
}

static inline int ew_grid(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = 148LL * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace tft

using namespace tft;

TFT_API int tft_swiglu_fwd(const void* gu, void* out, long long rows, int F, cudaStream_t stream) {
  if (F % 8) return static_cast<int>(cudaErrorInvalidValue);
  swiglu_fwd_kernel<<<ew_grid(rows * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), rows, F);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long rows, int F,
                           cudaStream_t stream) {
  if (F % 8) return static_cast<int>(cudaErrorInvalidValue);
  swiglu_bwd_kernel<<<ew_grid(rows * (F / 8), 256), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<const __nv_bfloat16*>(dout),
      static_cast<__nv_bfloat16*>(dgu), rows, F);
  return static_cast<int>(cudaGetLastError());
}

// logits [rows, V] bf16 (row stride ld) become the gradient; loss[rows] fp32.
TFT_API int tft_xent(void* logits, const long long* targets, float* loss, int rows, int V, int ld,
                     float grad_scale, long long ignore_index, cudaStream_t stream) {
  if (V % 8 || ld % 8) return static_cast<int>(cudaErrorInvalidValue);
  xent_kernel<<<rows, 1024, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), targets, loss, V, ld, grad_scale,
                                         ignore_index);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_embedding_fwd(const long long* tokens, const void* table, void* out, long long n_tokens, int dim,
                              cudaStream_t stream) {
  if (dim % 8) return static_cast<int>(cudaErrorInvalidValue);
  embedding_fwd_kernel<<<ew_grid(n_tokens * (dim / 8), 256), 256, 0, stream>>>(
      tokens, static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), n_tokens, dim);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_embedding_bwd(const long long* tokens, const void* dout, void* dtable, long long n_tokens, int dim,
                              cudaStream_t stream) {
  if (dim % 2) return static_cast<int>(cudaErrorInvalidValue);
  embedding_bwd_kernel<<<ew_grid(n_tokens * (dim / 2), 256), 256, 0, stream>>>(
      tokens, static_cast<const __nv_bfloat16*>(dout), static_cast<__nv_bfloat16*>(dtable), n_tokens, dim);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_adamw(void* p, const void* g, float* m, float* v, long long n, float lr, float b1, float b2,
                      float eps, float wd, int step, float grad_scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g)) & 15) return static_cast<int>(cudaErrorInvalidValue);
  if ((reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15) return static_cast<int>(cudaErrorInvalidValue);
  const float bc1 = 1.f - powf(b1, static_cast<float>(step));
  const float bc2 = 1.f - powf(b2, static_cast<float>(step));
  adamw_kernel<<<ew_grid(n / 8 + 8, 256), 256, 0, stream>>>(static_cast<__nv_bfloat16*>(p),
                                                            static_cast<const __nv_bfloat16*>(g), m, v, n, lr, b1,
                                                            b2, eps, wd, bc1, bc2, grad_scale);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_pseudograd(void* local, const void* global_w, long long n, int is_bf16, cudaStream_t stream) {
  if (is_bf16)
    pseudograd_kernel<__nv_bfloat16><<<ew_grid(n, 256), 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(local), static_cast<const __nv_bfloat16*>(global_w), n);
  else
    pseudograd_kernel<float><<<ew_grid(n, 256), 256, 0, stream>>>(static_cast<float*>(local),
                                                                  static_cast<const float*>(global_w), n);
  return static_cast<int>(cudaGetLastError());
}

TFT_API int tft_nesterov_outer(void* g, void* global_w, float* buf, long long n, float lr, float mu, int nesterov,
                               int first, int is_bf16, cudaStream_t stream) {
  if (is_bf16)
    nesterov_outer_kernel<__nv_bfloat16><<<ew_grid(n, 256), 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(g), static_cast<__nv_bfloat16*>(global_w), buf, n, lr, mu, nesterov, first);
  else
    nesterov_outer_kernel<float><<<ew_grid(n, 256), 256, 0, stream>>>(static_cast<float*>(g),
                                                                      static_cast<float*>(global_w), buf, n, lr, mu,
                                                                      nesterov, first);
  return static_cast<int>(cudaGetLastError());
}
