// Training-mode batch normalisation over NCHW fp32 activations fused with the clipped ReLU that
// follows it in the DeepSpeech2-style model: y = clamp(gamma * (x - mean) / sqrt(var + eps) + beta, 0, hi).
//
// The reference's counterpart is FusedBatchNorm (cuDNN's batch normalisation plus two helper
// kernels, tensorflow/core/kernels/fused_batch_norm_op.cu.cc:26-60) followed by a separate
// Relu6-style clipping kernel (core/kernels/relu_op_gpu.cu.cc). On B200 cuDNN's backward kernel
// for these shapes (32 channels, 0.9 M elements per channel) runs at a twentieth of the memory
// roofline; the two passes here read each tensor twice and write it once, nothing more:
//   forward : pass 1 per-channel sum and sum of squares (block partials, double atomics),
//             pass 2 normalise + scale + shift + clip, save mean / rstd, update the running statistics
//   backward: pass 1 per-channel sums of dz and dz * xhat, where dz = dy inside the clip range
//             (recomputed from x, so the forward output is not needed), pass 2
//             dx = gamma * rstd * (dz - mean(dz) - xhat * mean(dz * xhat)); dgamma, dbeta.
// Nothing here waits on anything: plain streaming kernels on the caller's stream.
#include "bn_clip.h"

#include <stdint.h>

#include <initializer_list>

namespace bc {
namespace gpu {

namespace {

constexpr int kThreads = 512;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum of two per-thread values over the block; the result is valid in thread 0.
__device__ __forceinline__ void block_sum2(float& a, float& b) {
  __shared__ float sa[kThreads / 32], sb[kThreads / 32];
  a = warp_sum(a);
  b = warp_sum(b);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sa[w] = a; sb[w] = b; }
  __syncthreads();
  if (w == 0) {
    a = l < kThreads / 32 ? sa[l] : 0.f;
    b = l < kThreads / 32 ? sb[l] : 0.f;
    a = warp_sum(a);
    b = warp_sum(b);
  }
}

// Work split: block (j, c) handles part j % parts of image j / parts of channel c, i.e. one
// contiguous run of the tensor (a whole H x W plane when parts == 1). A run is read with the
// widest vectors that the plane size allows (V = 4, 2 or 1 floats: planes start at multiples of
// HW floats), four vectors in flight per thread.
struct Run {
  size_t base;   // first element of the run in the tensor
  int len;       // elements
  __device__ Run(int C, int HW, int parts, int V) {
    const int n = blockIdx.x / parts, part = blockIdx.x % parts, c = blockIdx.y;
    int seg = (HW + parts - 1) / parts;
    seg = (seg + V - 1) / V * V;
    const int lo = min(HW, part * seg), hi = min(HW, lo + seg);
    base = ((size_t)n * C + c) * HW + lo;
    len = hi - lo;
  }
};

template <int V> struct Vec;
template <> struct Vec<1> { using T = float; };
template <> struct Vec<2> { using T = float2; };
template <> struct Vec<4> { using T = float4; };

template <int V>
__device__ __forceinline__ void load(const float* p, float* o) {
  const typename Vec<V>::T v = *reinterpret_cast<const typename Vec<V>::T*>(p);
  const float* f = reinterpret_cast<const float*>(&v);
#pragma unroll
  for (int i = 0; i < V; i++) o[i] = f[i];
}
template <int V>
__device__ __forceinline__ void store(float* p, const float* o) {
  typename Vec<V>::T v;
  float* f = reinterpret_cast<float*>(&v);
#pragma unroll
  for (int i = 0; i < V; i++) f[i] = o[i];
  *reinterpret_cast<typename Vec<V>::T*>(p) = v;
}

// Vectors per thread and iteration in the one-input kernels (their loads are all issued before
// the first value is used); the two-input kernels of the backward pass take two of each input.
constexpr int kUnroll = 4;

// Forward pass 1: acc[2c] += sum x, acc[2c + 1] += sum x^2 over the block's run.
template <int V>
__global__ void __launch_bounds__(kThreads) bn_stats_kernel(const float* __restrict__ x, double* __restrict__ acc, int C, int HW, int parts) {
  const Run run(C, HW, parts, V);
  const float* p = x + run.base;
  const int nvec = run.len / V;
  float s = 0.f, q = 0.f;
  int i = threadIdx.x;
  for (; i + (kUnroll - 1) * kThreads < nvec; i += kUnroll * kThreads) {
    float a[kUnroll][V];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) load<V>(p + (size_t)(i + u * kThreads) * V, a[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; u++)
#pragma unroll
      for (int e = 0; e < V; e++) { s += a[u][e]; q = fmaf(a[u][e], a[u][e], q); }
  }
  for (; i < nvec; i += kThreads) {
    float a[V];
    load<V>(p + (size_t)i * V, a);
#pragma unroll
    for (int e = 0; e < V; e++) { s += a[e]; q = fmaf(a[e], a[e], q); }
  }
  for (int r = nvec * V + threadIdx.x; r < run.len; r += kThreads) { s += p[r]; q = fmaf(p[r], p[r], q); }
  block_sum2(s, q);
  if (threadIdx.x == 0) {
    atomicAdd(acc + 2 * blockIdx.y, (double)s);
    atomicAdd(acc + 2 * blockIdx.y + 1, (double)q);
  }
}

// Forward pass 2. The first block of every channel also publishes the batch statistics and
// folds them into the running ones.
template <int V>
__global__ void __launch_bounds__(kThreads) bn_apply_kernel(const float* __restrict__ x, float* __restrict__ y, const double* __restrict__ acc,
                                                            const float* __restrict__ gamma, const float* __restrict__ beta,
                                                            float* __restrict__ save_mean, float* __restrict__ save_rstd,
                                                            float* running_mean, float* running_var, int N, int C, int HW, int parts,
                                                            float eps, float momentum, float clip_hi) {
  const int c = blockIdx.y;
  const Run run(C, HW, parts, V);
  const double m = (double)N * HW;
  const double mean_d = acc[2 * c] / m;
  double var_d = acc[2 * c + 1] / m - mean_d * mean_d;
  if (var_d < 0.0) var_d = 0.0;
  const float mean = (float)mean_d;
  const float rstd = rsqrtf((float)var_d + eps);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    save_mean[c] = mean;
    save_rstd[c] = rstd;
    if (running_mean) {
      const float unbiased = (float)(var_d * (m / (m > 1.0 ? m - 1.0 : 1.0)));
      running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mean;
      running_var[c] = (1.f - momentum) * running_var[c] + momentum * unbiased;
    }
  }
  const float scale = gamma[c] * rstd;
  const float shift = beta[c] - mean * scale;
  const float* p = x + run.base;
  float* o = y + run.base;
  const int nvec = run.len / V;
  auto f = [&](float v) { return fminf(fmaxf(fmaf(v, scale, shift), 0.f), clip_hi); };
  int i = threadIdx.x;
  for (; i + (kUnroll - 1) * kThreads < nvec; i += kUnroll * kThreads) {
    float a[kUnroll][V];
#pragma unroll
    for (int u = 0; u < kUnroll; u++) load<V>(p + (size_t)(i + u * kThreads) * V, a[u]);
#pragma unroll
    for (int u = 0; u < kUnroll; u++) {
#pragma unroll
      for (int e = 0; e < V; e++) a[u][e] = f(a[u][e]);
      store<V>(o + (size_t)(i + u * kThreads) * V, a[u]);
    }
  }
  for (; i < nvec; i += kThreads) {
    float a[V];
    load<V>(p + (size_t)i * V, a);
#pragma unroll
    for (int e = 0; e < V; e++) a[e] = f(a[e]);
    store<V>(o + (size_t)i * V, a);
  }
  for (int r = nvec * V + threadIdx.x; r < run.len; r += kThreads) o[r] = f(p[r]);
}

// dz of one element: dy where the pre-clip value lies strictly inside (0, hi), else 0 (the
// gradient rule of a hard clamp).
__device__ __forceinline__ float masked(float dy, float z, float clip_hi) { return (z > 0.f && z < clip_hi) ? dy : 0.f; }

// Backward pass 1: acc[2c] += sum dz, acc[2c + 1] += sum dz * xhat.
template <int V>
__global__ void __launch_bounds__(kThreads) bn_bwd_reduce_kernel(const float* __restrict__ x, const float* __restrict__ dy,
                                                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                 const float* __restrict__ save_mean, const float* __restrict__ save_rstd,
                                                                 double* __restrict__ acc, int C, int HW, int parts, float clip_hi) {
  const int c = blockIdx.y;
  const Run run(C, HW, parts, V);
  const float mean = save_mean[c], rstd = save_rstd[c], g = gamma[c], b = beta[c];
  const float* px = x + run.base;
  const float* pd = dy + run.base;
  const int nvec = run.len / V;
  float s1 = 0.f, s2 = 0.f;
  auto f = [&](float xv, float dv) {
    const float h = (xv - mean) * rstd;
    const float z = masked(dv, fmaf(h, g, b), clip_hi);
    s1 += z;
    s2 = fmaf(z, h, s2);
  };
  constexpr int U = 2;
  int i = threadIdx.x;
  for (; i + (U - 1) * kThreads < nvec; i += U * kThreads) {
    float a[U][V], d[U][V];
#pragma unroll
    for (int u = 0; u < U; u++) { load<V>(px + (size_t)(i + u * kThreads) * V, a[u]); load<V>(pd + (size_t)(i + u * kThreads) * V, d[u]); }
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
      for (int e = 0; e < V; e++) f(a[u][e], d[u][e]);
  }
  for (; i < nvec; i += kThreads) {
    float a[V], d[V];
    load<V>(px + (size_t)i * V, a);
    load<V>(pd + (size_t)i * V, d);
#pragma unroll
    for (int e = 0; e < V; e++) f(a[e], d[e]);
  }
  for (int r = nvec * V + threadIdx.x; r < run.len; r += kThreads) f(px[r], pd[r]);
  block_sum2(s1, s2);
  if (threadIdx.x == 0) {
    atomicAdd(acc + 2 * c, (double)s1);
    atomicAdd(acc + 2 * c + 1, (double)s2);
  }
}

// Backward pass 2.
template <int V>
__global__ void __launch_bounds__(kThreads) bn_bwd_apply_kernel(const float* __restrict__ x, const float* __restrict__ dy, float* __restrict__ dx,
                                                                const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                const float* __restrict__ save_mean, const float* __restrict__ save_rstd,
                                                                const double* __restrict__ acc, float* __restrict__ dgamma,
                                                                float* __restrict__ dbeta, int N, int C, int HW, int parts, float clip_hi) {
  const int c = blockIdx.y;
  const Run run(C, HW, parts, V);
  const float mean = save_mean[c], rstd = save_rstd[c], g = gamma[c], b = beta[c];
  const double m = (double)N * HW;
  const float s1 = (float)(acc[2 * c] / m), s2 = (float)(acc[2 * c + 1] / m);
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    dbeta[c] = (float)acc[2 * c];
    dgamma[c] = (float)acc[2 * c + 1];
  }
  const float k = g * rstd;
  const float* px = x + run.base;
  const float* pd = dy + run.base;
  float* po = dx + run.base;
  const int nvec = run.len / V;
  auto f = [&](float xv, float dv) {
    const float h = (xv - mean) * rstd;
    const float z = masked(dv, fmaf(h, g, b), clip_hi);
    return k * (z - s1 - h * s2);
  };
  constexpr int U = 2;
  int i = threadIdx.x;
  for (; i + (U - 1) * kThreads < nvec; i += U * kThreads) {
    float a[U][V], d[U][V];
#pragma unroll
    for (int u = 0; u < U; u++) { load<V>(px + (size_t)(i + u * kThreads) * V, a[u]); load<V>(pd + (size_t)(i + u * kThreads) * V, d[u]); }
#pragma unroll
    for (int u = 0; u < U; u++) {
#pragma unroll
      for (int e = 0; e < V; e++) a[u][e] = f(a[u][e], d[u][e]);
      store<V>(po + (size_t)(i + u * kThreads) * V, a[u]);
    }
  }
  for (; i < nvec; i += kThreads) {
    float a[V], d[V];
    load<V>(px + (size_t)i * V, a);
    load<V>(pd + (size_t)i * V, d);
#pragma unroll
    for (int e = 0; e < V; e++) a[e] = f(a[e], d[e]);
    store<V>(po + (size_t)i * V, a);
  }
  for (int r = nvec * V + threadIdx.x; r < run.len; r += kThreads) po[r] = f(px[r], pd[r]);
}

int sm_count_of_current_device() {
  int dev = 0, n = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  return n;
}

// Parts per plane: one unless N * C planes are fewer than four blocks per SM; never less than
// 2048 elements per part.
int parts_for(int N, int C, int HW) {
  const long want = 4L * sm_count_of_current_device();
  long parts = (want + (long)N * C - 1) / ((long)N * C);
  const long most = HW / 2048 > 0 ? HW / 2048 : 1;
  if (parts > most) parts = most;
  return (int)(parts < 1 ? 1 : parts);
}

// Vector width that every plane start and the four base pointers allow.
int vec_for(int HW, std::initializer_list<const void*> ptrs) {
  int v = HW % 4 == 0 ? 4 : (HW % 2 == 0 ? 2 : 1);
  for (const void* p : ptrs)
    while (v > 1 && ((uintptr_t)p % (4 * v)) != 0) v /= 2;
  return v;
}

}  // namespace

cudaError_t bn_clip_forward(const float* x, float* y, const float* gamma, const float* beta, float* running_mean, float* running_var,
                            float* save_mean, float* save_rstd, double* acc, int N, int C, int HW, float eps, float momentum,
                            float clip_hi, cudaStream_t stream) {
  if (N <= 0 || C <= 0 || HW <= 0 || C > 65535) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(acc, 0, sizeof(double) * 2 * C, stream);
  if (e != cudaSuccess) return e;
  const int parts = parts_for(N, C, HW);
  dim3 grid(N * parts, C);
  switch (vec_for(HW, {x, y})) {
    case 4:
      bn_stats_kernel<4><<<grid, kThreads, 0, stream>>>(x, acc, C, HW, parts);
      bn_apply_kernel<4><<<grid, kThreads, 0, stream>>>(x, y, acc, gamma, beta, save_mean, save_rstd, running_mean, running_var, N, C, HW,
                                                        parts, eps, momentum, clip_hi);
      break;
    case 2:
      bn_stats_kernel<2><<<grid, kThreads, 0, stream>>>(x, acc, C, HW, parts);
      bn_apply_kernel<2><<<grid, kThreads, 0, stream>>>(x, y, acc, gamma, beta, save_mean, save_rstd, running_mean, running_var, N, C, HW,
                                                        parts, eps, momentum, clip_hi);
      break;
    default:
      bn_stats_kernel<1><<<grid, kThreads, 0, stream>>>(x, acc, C, HW, parts);
      bn_apply_kernel<1><<<grid, kThreads, 0, stream>>>(x, y, acc, gamma, beta, save_mean, save_rstd, running_mean, running_var, N, C, HW,
                                                        parts, eps, momentum, clip_hi);
  }
  return cudaGetLastError();
}

cudaError_t bn_clip_backward(const float* x, const float* dy, const float* gamma, const float* beta, const float* save_mean,
                             const float* save_rstd, float* dx, float* dgamma, float* dbeta, double* acc, int N, int C, int HW,
                             float clip_hi, cudaStream_t stream) {
  if (N <= 0 || C <= 0 || HW <= 0 || C > 65535) return cudaErrorInvalidValue;
  cudaError_t e = cudaMemsetAsync(acc, 0, sizeof(double) * 2 * C, stream);
  if (e != cudaSuccess) return e;
  const int parts = parts_for(N, C, HW);
  dim3 grid(N * parts, C);
  switch (vec_for(HW, {x, dy, dx})) {
    case 4:
      bn_bwd_reduce_kernel<4><<<grid, kThreads, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, acc, C, HW, parts, clip_hi);
      bn_bwd_apply_kernel<4><<<grid, kThreads, 0, stream>>>(x, dy, dx, gamma, beta, save_mean, save_rstd, acc, dgamma, dbeta, N, C, HW, parts, clip_hi);
      break;
    case 2:
      bn_bwd_reduce_kernel<2><<<grid, kThreads, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, acc, C, HW, parts, clip_hi);
      bn_bwd_apply_kernel<2><<<grid, kThreads, 0, stream>>>(x, dy, dx, gamma, beta, save_mean, save_rstd, acc, dgamma, dbeta, N, C, HW, parts, clip_hi);
      break;
    default:
      bn_bwd_reduce_kernel<1><<<grid, kThreads, 0, stream>>>(x, dy, gamma, beta, save_mean, save_rstd, acc, C, HW, parts, clip_hi);
      bn_bwd_apply_kernel<1><<<grid, kThreads, 0, stream>>>(x, dy, dx, gamma, beta, save_mean, save_rstd, acc, dgamma, dbeta, N, C, HW, parts, clip_hi);
  }
  return cudaGetLastError();
}

}  // namespace gpu
}  // namespace bc
