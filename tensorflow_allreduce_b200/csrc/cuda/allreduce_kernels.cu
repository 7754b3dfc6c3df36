// Sum-allreduce over peer-mapped memory for sm_100a: one-shot, two-shot and NVLS (multimem)
// variants, with the averaging scale, the 16-bit <-> fp32 conversion and the momentum-SGD /
// Adam(W) parameter update fused behind the reduction.
//
// Reference behaviour covered here: RingAllreduce + elemwise_accum
// (tensorflow/contrib/mpi_collectives/ring.h:136-228, ring.cu.cc:48-66), the averaging divide
// (mpi_collectives/__init__.py:160-164) and the optimizer kernels it feeds
// (core/kernels/training_ops_gpu.cu.cc:82-145). None of the reference's structure is kept: there
// is no ring, because through NVSwitch every peer is one hop away.
//
//   one-shot : barrier | every rank loads all P copies of every element, sums, writes `out` | barrier
//   two-shot : barrier | rank r sums slice r over all P copies and stores the result into all P
//              buffers (in place) | barrier | local epilogue over the whole buffer
//   NVLS     : as two-shot, but the switch does the sum (multimem.ld_reduce) and the fan-out
//              (multimem.st), so each GPU moves N/P + N bytes instead of 2N(P-1)/P.
//
// Block b of a rank only ever waits for block b of its peers, and touches only elements that
// block b of the producing rank wrote, so per-block flag barriers are sufficient.
//
// Staged inputs: a tensor outside symmetric memory is copied into this rank's staging buffer by
// the kernel itself before the first barrier (ArRank::src), with the index mapping of the phase
// that reads it, so the rule above still holds and no separate copy launch is needed.
#include "collectives.h"
#include "device_prims.cuh"

#include <type_traits>

namespace bc {
namespace gpu {

using namespace dev;

namespace {

constexpr int ALGO_ONE = 1, ALGO_TWO = 2, ALGO_NVLS = 3;
constexpr int OPT_NONE = 0, OPT_SGD = 1, OPT_ADAM = 2, OPT_RED = 3;   // OPT_RED: no update, reduction chosen at run time

template <typename A>
__device__ __forceinline__ A combine(A a, A b, int red) {
  switch (red) {
    case 1: return a * b;
    case 2: return b < a ? b : a;
    case 3: return b > a ? b : a;
    default: return a + b;
  }
}
constexpr int kNvlsUnroll = 4;   // packs per batch; two batches are in flight per thread

template <typename T> struct Scalar;  // scalar load/store in the accumulator type
template <> struct Scalar<float> { using Acc = float; __device__ static Acc ld(const float* p) { return *p; } __device__ static void st(float* p, Acc v) { *p = v; } };
template <> struct Scalar<double> { using Acc = double; __device__ static Acc ld(const double* p) { return *p; } __device__ static void st(double* p, Acc v) { *p = v; } };
template <> struct Scalar<int32_t> { using Acc = int32_t; __device__ static Acc ld(const int32_t* p) { return *p; } __device__ static void st(int32_t* p, Acc v) { *p = v; } };
template <> struct Scalar<int64_t> { using Acc = long long; __device__ static Acc ld(const int64_t* p) { return *p; } __device__ static void st(int64_t* p, Acc v) { *p = v; } };
template <> struct Scalar<uint8_t> { using Acc = uint8_t; __device__ static Acc ld(const uint8_t* p) { return *p; } __device__ static void st(uint8_t* p, Acc v) { *p = v; } };
template <> struct Scalar<__nv_bfloat16> { using Acc = float; __device__ static Acc ld(const __nv_bfloat16* p) { return __bfloat162float(*p); } __device__ static void st(__nv_bfloat16* p, Acc v) { *p = __float2bfloat16_rn(v); } };
template <> struct Scalar<__half> { using Acc = float; __device__ static Acc ld(const __half* p) { return __half2float(*p); } __device__ static void st(__half* p, Acc v) { *p = __float2half_rn(v); } };

template <typename T> struct IsFloatGrad { static constexpr bool value = false; };
template <> struct IsFloatGrad<float> { static constexpr bool value = true; };
template <> struct IsFloatGrad<__nv_bfloat16> { static constexpr bool value = true; };
template <> struct IsFloatGrad<__half> { static constexpr bool value = true; };

__device__ __forceinline__ float sgd_step(float p, float g, float* buf, const OptHyper& h) {
  if (h.weight_decay != 0.f) g = fmaf(h.weight_decay, p, g);
  if (h.momentum != 0.f) {
    float b = h.first_step ? g : fmaf(h.momentum, *buf, (1.f - h.dampening) * g);
    *buf = b;
    g = h.nesterov ? fmaf(h.momentum, b, g) : b;
  }
  return fmaf(-h.lr, g, p);
}

// sqrt.approx / div.approx: about one and two units in the last place. The update is a product
// of several rounded factors anyway, and the IEEE sequences that the compiler emits for `sqrtf`
// and `/` cost tens of instructions per element: with them the Adam epilogue was bound by
// instruction issue (0.81 of the HBM copy rate), not by memory.
__device__ __forceinline__ float sqrt_fast(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float div_fast(float a, float b) {
  float y;
  asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(y) : "f"(a), "f"(b));
  return y;
}

// What an Adam step needs from the hyper-parameters, computed once per thread.
struct AdamConst {
  float step;         // torch form: lr / bc1;  TF form: lr * sqrt(bc2) / bc1
  float inv_sqrt_bc2; // torch form: 1 / sqrt(bc2);  TF form: 1
  float decay;        // decoupled weight decay: 1 - lr * wd, else 1
  float l2;           // coupled weight decay: wd, else 0
  __device__ explicit AdamConst(const OptHyper& h) {
    const float s2 = sqrtf(h.bias_c2);
    step = h.tf_epsilon_hat ? h.lr * s2 / h.bias_c1 : h.lr / h.bias_c1;
    inv_sqrt_bc2 = h.tf_epsilon_hat ? 1.f : 1.f / s2;
    decay = (h.weight_decay != 0.f && h.decoupled_wd) ? 1.f - h.lr * h.weight_decay : 1.f;
    l2 = (h.weight_decay != 0.f && !h.decoupled_wd) ? h.weight_decay : 0.f;
  }
};

__device__ __forceinline__ float adam_step(float p, float g, float* m, float* v, const OptHyper& h, const AdamConst& k) {
  p *= k.decay;
  g = fmaf(k.l2, p, g);
  const float mm = fmaf(h.beta1, *m, (1.f - h.beta1) * g);
  const float vv = fmaf(h.beta2, *v, (1.f - h.beta2) * g * g);
  *m = mm;
  *v = vv;
  // torch: p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps);  TF: p -= lr sqrt(bc2) / bc1 * m / (sqrt(v) + eps)
  const float denom = fmaf(sqrt_fast(vv), k.inv_sqrt_bc2, h.eps);
  return fmaf(-k.step, div_fast(mm, denom), p);
}

template <int OPT>
__device__ __forceinline__ float opt_step(float p, float g, float* s1, float* s2, const OptHyper& h, const AdamConst& k) {
  if (OPT == OPT_SGD) return sgd_step(p, g, s1, h);
  return adam_step(p, g, s1, s2, h, k);
}

// Sum of packs over all ranks' buffers, in rank order (identical on every rank), for the packs
// begin + first, begin + first + stride, ... below `end`. PP is the number of ranks when known
// at compile time (0: use the run-time P); U packs are fetched together so that U*P 16-byte
// loads per thread are in flight across NVLink. `sink(i, acc)` consumes each reduced pack.
template <typename T, int PP, int U, bool GEN, typename Sink>
__device__ __forceinline__ void reduce_range(const ArRank& R, int P, size_t begin, size_t end, size_t first, size_t stride, size_t limit, int red, Sink sink) {
  using PK = Pack<T>;
  constexpr int N = PP > 0 ? PP : kMaxRanks;
  for (size_t i0 = begin + first; i0 < end; i0 += stride * U) {
    uint4 v[U][N];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const size_t i = i0 + (size_t)u * stride;
      if (i < end && in_bounds(R.ctx, i < limit)) {
#pragma unroll
        for (int p = 0; p < N; p++)
          if (PP > 0 || p < P) v[u][p] = ld_stream16(R.in[p] + i * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      const size_t i = i0 + (size_t)u * stride;
      if (i < end && in_bounds(R.ctx, i < limit)) {
        typename PK::Acc acc[PK::kElems];
        PK::unpack(v[u][0], acc);
#pragma unroll
        for (int p = 1; p < N; p++) {
          if (PP > 0 || p < P) {
            typename PK::Acc tmp[PK::kElems];
            PK::unpack(v[u][p], tmp);
#pragma unroll
            for (int e = 0; e < PK::kElems; e++) acc[e] = GEN ? combine(acc[e], tmp[e], red) : acc[e] + tmp[e];
          }
        }
        sink(i, acc);
      }
    }
  }
}

template <typename T, bool GEN, typename Sink>
__device__ __forceinline__ void reduce_range_any(const ArRank& R, int P, size_t begin, size_t end, size_t first, size_t stride, size_t limit, int red, Sink sink) {
  switch (P) {
    case 2: reduce_range<T, 2, 4, GEN>(R, P, begin, end, first, stride, limit, red, sink); break;
    case 4: reduce_range<T, 4, 2, GEN>(R, P, begin, end, first, stride, limit, red, sink); break;
    case 8: reduce_range<T, 8, 1, GEN>(R, P, begin, end, first, stride, limit, red, sink); break;
    default: reduce_range<T, 0, 1, GEN>(R, P, begin, end, first, stride, limit, red, sink); break;
  }
}

template <typename T>
__device__ __forceinline__ typename Scalar<T>::Acc reduce_scalar(const ArRank& R, int P, size_t e, int red) {
  typename Scalar<T>::Acc acc = Scalar<T>::ld(reinterpret_cast<const T*>(R.in[0]) + e);
  for (int p = 1; p < P; p++) acc = combine(acc, Scalar<T>::ld(reinterpret_cast<const T*>(R.in[p]) + e), red);
  return acc;
}

// Epilogue for one pack of already reduced (and scaled) values.
template <typename T, int OPT>
__device__ __forceinline__ void epilogue_pack(const ArRank& R, const ArArgs& a, size_t i, typename Pack<T>::Acc* acc, int me) {
  using PK = Pack<T>;
  constexpr int E = PK::kElems;
  if constexpr (OPT == OPT_NONE || OPT == OPT_RED) {
    st_local16(reinterpret_cast<char*>(R.out) + i * 16, PK::pack(acc));
  } else if constexpr (IsFloatGrad<T>::value) {
    const OptHyper& h = a.opt;
    const AdamConst k(h);      // loop-invariant: the compiler computes it once per thread
    const size_t e0 = i * E;
    float p[E], s1[E], s2[E];
    // parameters in fp32: the tensor itself (fp32 model) or the master copy (16-bit model).
    // E floats of an fp32 array are one 16-byte access (E = 4) or one 32-byte access (E = 8).
    auto ld_f32 = [](const float* q, float* o) {
      if constexpr (E == 8) ld_local32(q, o);
      else Pack<float>::unpack(ld_local16(q), o);
    };
    auto st_f32 = [](float* q, const float* o) {
      if constexpr (E == 8) st_local32(q, o);
      else st_local16(q, Pack<float>::pack(o));
    };
    const float* p32 = sizeof(T) == 4 ? reinterpret_cast<const float*>(R.param) : R.master;
    if (p32) ld_f32(p32 + e0, p);
    else PK::unpack(ld_local16(reinterpret_cast<const char*>(R.param) + i * 16), p);
    const bool has_s1 = (OPT == OPT_ADAM) || (h.momentum != 0.f);
    if (has_s1 && !(OPT == OPT_SGD && h.first_step)) ld_f32(R.state1 + e0, s1);
    if (OPT == OPT_ADAM) ld_f32(R.state2 + e0, s2);
#pragma unroll
    for (int e = 0; e < E; e++) p[e] = opt_step<OPT>(p[e], acc[e], &s1[e], &s2[e], h, k);
    if (has_s1) st_f32(R.state1 + e0, s1);
    if (OPT == OPT_ADAM) st_f32(R.state2 + e0, s2);
    if (sizeof(T) == 4) {
      st_f32(reinterpret_cast<float*>(R.param) + e0, p);
    } else {
      if (R.master) st_f32(R.master + e0, p);
      st_local16(reinterpret_cast<char*>(R.param) + i * 16, PK::pack(p));
    }
    if (h.zero_grad) st_local16(R.in[me] + i * 16, make_uint4(0, 0, 0, 0));
  }
}

template <typename T, int OPT>
__device__ __forceinline__ void epilogue_scalar(const ArRank& R, const ArArgs& a, size_t e, typename Scalar<T>::Acc g, int me) {
  if constexpr (OPT == OPT_NONE || OPT == OPT_RED) {
    Scalar<T>::st(reinterpret_cast<T*>(R.out) + e, g);
  } else if constexpr (IsFloatGrad<T>::value) {
    const OptHyper& h = a.opt;
    float p;
    if (sizeof(T) == 4) p = reinterpret_cast<const float*>(R.param)[e];
    else p = R.master ? R.master[e] : Scalar<T>::ld(reinterpret_cast<const T*>(R.param) + e);
    float s1 = 0.f, s2 = 0.f;
    const bool has_s1 = (OPT == OPT_ADAM) || (h.momentum != 0.f);
    if (has_s1 && !(OPT == OPT_SGD && h.first_step)) s1 = R.state1[e];
    if (OPT == OPT_ADAM) s2 = R.state2[e];
    p = opt_step<OPT>(p, (float)g, &s1, &s2, h, AdamConst(h));
    if (has_s1) R.state1[e] = s1;
    if (OPT == OPT_ADAM) R.state2[e] = s2;
    if (sizeof(T) == 4) reinterpret_cast<float*>(R.param)[e] = p;
    else {
      if (R.master) R.master[e] = p;
      Scalar<T>::st(reinterpret_cast<T*>(R.param) + e, p);
    }
    if (h.zero_grad) Scalar<T>::st(reinterpret_cast<T*>(R.in[me]) + e, 0.f);
  }
}

// Copy of the packs begin + first, begin + first + stride, ... below `end` from `src` to `dst`
// (both local, 16-byte aligned), four independent loads in flight per thread (eight cost spills
// under the 64-register bound of two resident blocks per SM).
__device__ __forceinline__ void copy_packs(char* dst, const char* src, size_t begin, size_t end, size_t first, size_t stride) {
  constexpr int U = 4;
  size_t i = begin + first;
  for (; i + (U - 1) * stride < end; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) v[u] = ld_stream16(src + (i + u * stride) * 16);
#pragma unroll
    for (int u = 0; u < U; u++) st_local16(dst + (i + u * stride) * 16, v[u]);
  }
  for (; i < end; i += stride) st_local16(dst + i * 16, ld_stream16(src + i * 16));
}

// Time stamp k of a profiled launch (block 0 of the first rank slot only).
__device__ __forceinline__ void stamp(const ArArgs& a, int k) {
  if (a.prof && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) a.prof[k] = global_timer();
}

template <typename T>
__device__ __forceinline__ uint4 nvls_reduce(const char* mc) {
  if constexpr (sizeof(T) == 4) return multimem_ld_reduce_f32(mc);
  else if constexpr (std::is_same<T, __nv_bfloat16>::value) return multimem_ld_reduce_bf16(mc);
  else return multimem_ld_reduce_f16(mc);
}

template <typename T, int ALGO, int OPT>
__global__ void __launch_bounds__(512, 2) allreduce_kernel(const __grid_constant__ ArArgs a) {
  using PK = Pack<T>;
  using Acc = typename PK::Acc;
  constexpr int E = PK::kElems;
  const ArRank& R = a.r[blockIdx.y];
  const RankCtx& c = R.ctx;
  const int P = c.world, me = c.rank;
  const size_t npacks = a.count / E;
  const size_t tail0 = npacks * E;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;

  stamp(a, 0);
  if (P == 1) {
    // Single rank: the reduction is the identity; only the epilogue runs.
    const char* in0 = R.src ? R.src : R.in[0];
    for (size_t i = first; i < npacks; i += stride) {
      Acc acc[E];
      PK::unpack(ld_local16(in0 + i * 16), acc);
#pragma unroll
      for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
      epilogue_pack<T, OPT>(R, a, i, acc, 0);
    }
    if (blockIdx.x == 0)
      for (size_t e = tail0 + threadIdx.x; e < a.count; e += blockDim.x)
        epilogue_scalar<T, OPT>(R, a, e, finish<typename Scalar<T>::Acc>(Scalar<T>::ld(reinterpret_cast<const T*>(in0) + e), a.scale, a.idiv), 0);
    return;
  }

  if (R.src) {
    // Staged input: bring it into this rank's symmetric buffer. Every pack is written by the
    // thread index that reads it from all ranks in the next phase (one-shot: pack i by thread
    // i mod stride; two-phase: the same inside every rank's slice), so the per-block barrier
    // below is all the ordering that the readers need.
    if constexpr (ALGO == ALGO_ONE) {
      copy_packs(R.in[me], R.src, 0, npacks, first, stride);
    } else {
      for (int q = 0; q < P; q++) copy_packs(R.in[me], R.src, npacks * (size_t)q / P, npacks * (size_t)(q + 1) / P, first, stride);
    }
    if (blockIdx.x == 0)
      for (size_t e = tail0 + threadIdx.x; e < a.count; e += blockDim.x)
        reinterpret_cast<T*>(R.in[me])[e] = reinterpret_cast<const T*>(R.src)[e];
  }
  if (R.place && blockIdx.x == 0 && (int)threadIdx.x < P) c.meta[threadIdx.x][(size_t)me * 2] = R.place;

  // Mixed grids (two-phase algorithms only): all blocks copy in and run the local epilogue, the
  // first phase1_blocks alone talk to the peers. Two barriers among this rank's blocks replace
  // the "block b only touches what block b produced" rule: every block's copy-in is complete
  // before any block signals a peer, and every peer's results are complete before any block
  // starts the epilogue.
  const bool mixed = ALGO != ALGO_ONE && a.phase1_blocks > 0 && a.phase1_blocks < (int)gridDim.x;
  const bool in_p1 = !mixed || (int)blockIdx.x < a.phase1_blocks;
  const size_t stride1 = mixed ? (size_t)a.phase1_blocks * blockDim.x : stride;
  if (mixed && !local_barrier(c, c.local_base + gridDim.x, true)) return;

  uint32_t epoch = load_epoch(c);
  if (in_p1 && !peer_barrier(c, epoch)) { store_epoch(c, epoch); return; }
  stamp(a, 1);
  if (R.place && blockIdx.x == 0 && (int)threadIdx.x < P) {
    // In place on symmetric memory: every rank must have passed the same offset, or the peers'
    // buffers are not where this rank looks for them. The result is then wrong; say so.
    const unsigned long long theirs = *(const volatile unsigned long long*)&c.meta[me][(size_t)threadIdx.x * 2];
    if (theirs != R.place) atomicOr(c.status, kStatusLayout | (1u << threadIdx.x) | ((uint32_t)me << 8));
  }

  if constexpr (ALGO == ALGO_ONE) {
    reduce_range_any<T, OPT == OPT_RED>(R, P, 0, npacks, first, stride, npacks, a.red, [&](size_t i, Acc* acc) {
#pragma unroll
      for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
      epilogue_pack<T, OPT>(R, a, i, acc, me);
    });
    if (blockIdx.x == 0)
      for (size_t e = tail0 + threadIdx.x; e < a.count; e += blockDim.x)
        epilogue_scalar<T, OPT>(R, a, e, finish<typename Scalar<T>::Acc>(reduce_scalar<T>(R, P, e, a.red), a.scale, a.idiv), me);
    stamp(a, 2);
    // Peers may still be reading this rank's input: nobody leaves before everybody is done.
    peer_barrier(c, epoch);
    store_epoch(c, epoch);
    stamp(a, 3);
    stamp(a, 4);
    return;
  } else {
    // Phase 1: reduce this rank's slice and store the result into every rank's buffer.
    const size_t sbeg = npacks * (size_t)me / P, send = npacks * (size_t)(me + 1) / P;
    if (in_p1) {
    if constexpr (ALGO == ALGO_NVLS && IsFloatGrad<T>::value) {
      // Software pipeline of batches of kNvlsUnroll packs: the reductions of batch k+1 are issued
      // before the stores of batch k. The reduction keeps this GPU's outbound links busy (every
      // peer's share of the slice travels to the switch), the multicast store its inbound links;
      // issued back to back by all threads, the two directions would take turns instead of
      // running together, which halves the speed of messages with only one or two batches per
      // thread (tens of MiB).
      auto load_batch = [&](size_t i0, uint4* r) {
#pragma unroll
        for (int u = 0; u < kNvlsUnroll; u++) {
          const size_t i = i0 + (size_t)u * stride1;
          if (i < send && in_bounds(c, i < npacks)) r[u] = nvls_reduce<T>(R.mc_in + i * 16);
        }
      };
      auto store_batch = [&](size_t i0, uint4* r) {
#pragma unroll
        for (int u = 0; u < kNvlsUnroll; u++) {
          const size_t i = i0 + (size_t)u * stride1;
          if (i < send && in_bounds(c, i < npacks)) {
            if (a.scale != 1.f) {
              Acc acc[E];
              PK::unpack(r[u], acc);
#pragma unroll
              for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
              r[u] = PK::pack(acc);
            }
            multimem_st16(R.mc_in + i * 16, r[u]);
          }
        }
      };
      const size_t step = stride1 * kNvlsUnroll;
      uint4 ra[kNvlsUnroll], rb[kNvlsUnroll];
      size_t i0 = sbeg + first;
      if (i0 < send) load_batch(i0, ra);
      while (i0 < send) {
        const size_t i1 = i0 + step;
        if (i1 < send) load_batch(i1, rb);
        store_batch(i0, ra);
        if (i1 >= send) break;
        const size_t i2 = i1 + step;
        if (i2 < send) load_batch(i2, ra);
        store_batch(i1, rb);
        i0 = i2;
      }
    } else {
      reduce_range_any<T, OPT == OPT_RED>(R, P, sbeg, send, first, stride1, npacks, a.red, [&](size_t i, Acc* acc) {
#pragma unroll
        for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
        const uint4 r = PK::pack(acc);
#pragma unroll
        for (int p = 0; p < kMaxRanks; p++)
          if (p < P) st16(R.in[p] + i * 16, r);
      });
    }
    // The ragged tail (fewer elements than one pack) belongs to rank 0, block 0.
    if (me == 0 && blockIdx.x == 0) {
      for (size_t e = tail0 + threadIdx.x; e < a.count; e += blockDim.x) {
        typename Scalar<T>::Acc g = finish<typename Scalar<T>::Acc>(reduce_scalar<T>(R, P, e, a.red), a.scale, a.idiv);
        for (int p = 0; p < P; p++) Scalar<T>::st(reinterpret_cast<T*>(R.in[p]) + e, g);
      }
    }
    }   // in_p1
    stamp(a, 2);
    if (in_p1) {
      if (!peer_barrier(c, epoch)) { store_epoch(c, epoch); return; }
      store_epoch(c, epoch);
    }
    if (mixed && !local_barrier(c, c.local_base + gridDim.x + a.phase1_blocks, in_p1)) return;
    stamp(a, 3);

    // Phase 2: local epilogue. Block b reads, inside each slice, exactly the packs that block b
    // of the owning rank produced.
    const bool copy_needed = (OPT != OPT_NONE && OPT != OPT_RED) || (R.out != (void*)R.in[me]);
    if (copy_needed) {
      for (int q = 0; q < P; q++) {
        const size_t qb = npacks * (size_t)q / P, qe = npacks * (size_t)(q + 1) / P;
        if constexpr (OPT == OPT_NONE || OPT == OPT_RED) {
          // plain copy of the reduced buffer to a separate output
          if (in_bounds(c, qe <= npacks)) copy_packs(reinterpret_cast<char*>(R.out), R.in[me], qb, qe, first, stride);
        } else {
          for (size_t i = qb + first; i < qe; i += stride) {
            if (!in_bounds(c, i < npacks)) continue;
            Acc acc[E];
            PK::unpack(ld_local16(R.in[me] + i * 16), acc);
            epilogue_pack<T, OPT>(R, a, i, acc, me);
          }
        }
      }
      if (blockIdx.x == 0)
        for (size_t e = tail0 + threadIdx.x; e < a.count; e += blockDim.x)
          epilogue_scalar<T, OPT>(R, a, e, Scalar<T>::ld(reinterpret_cast<const T*>(R.in[me]) + e), me);
    }
    stamp(a, 4);
  }
}

__global__ void __launch_bounds__(512) copy_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src, size_t npacks,
                                                    char* dtail, const char* stail, int ntail) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < npacks; i += stride) dst[i] = src[i];
  if (blockIdx.x == 0 && (int)threadIdx.x < ntail) dtail[threadIdx.x] = stail[threadIdx.x];
}

template <typename T, int ALGO, int OPT>
cudaError_t launch_one(const ArArgs& a, const LaunchCfg& cfg, cudaStream_t s) {
  dim3 grid(cfg.blocks, a.nranks_here), block(cfg.threads);
  if (cfg.cooperative || a.nranks_here > 1) {
    void* params[] = {(void*)&a};
    return cudaLaunchCooperativeKernel((const void*)allreduce_kernel<T, ALGO, OPT>, grid, block, params, 0, s);
  }
  allreduce_kernel<T, ALGO, OPT><<<grid, block, 0, s>>>(a);
  return cudaGetLastError();
}

template <typename T>
cudaError_t dispatch_plain(const ArArgs& a, const LaunchCfg& cfg, cudaStream_t s) {
  if (a.red != 0) {
    switch (a.algo) {
      case ALGO_ONE: return launch_one<T, ALGO_ONE, OPT_RED>(a, cfg, s);
      case ALGO_TWO: return launch_one<T, ALGO_TWO, OPT_RED>(a, cfg, s);
    }
    return cudaErrorInvalidValue;
  }
  switch (a.algo) {
    case ALGO_ONE: return launch_one<T, ALGO_ONE, OPT_NONE>(a, cfg, s);
    case ALGO_TWO: return launch_one<T, ALGO_TWO, OPT_NONE>(a, cfg, s);
    case ALGO_NVLS:
      if constexpr (IsFloatGrad<T>::value) return launch_one<T, ALGO_NVLS, OPT_NONE>(a, cfg, s);
      return cudaErrorInvalidValue;
  }
  return cudaErrorInvalidValue;
}

template <typename T>
cudaError_t dispatch_fused(const ArArgs& a, const LaunchCfg& cfg, cudaStream_t s) {
  const bool nvls = a.algo == ALGO_NVLS;
  if (a.algo == ALGO_ONE) return cudaErrorInvalidValue;  // the fused update needs the two-phase structure
  switch (a.opt.kind) {
    case OPT_SGD: return nvls ? launch_one<T, ALGO_NVLS, OPT_SGD>(a, cfg, s) : launch_one<T, ALGO_TWO, OPT_SGD>(a, cfg, s);
    case OPT_ADAM: return nvls ? launch_one<T, ALGO_NVLS, OPT_ADAM>(a, cfg, s) : launch_one<T, ALGO_TWO, OPT_ADAM>(a, cfg, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace

cudaError_t launch_allreduce(const ArArgs& a, DType dtype, DType param_dtype, const LaunchCfg& cfg, cudaStream_t s) {
  if (cfg.blocks <= 0 || cfg.blocks > kMaxBlocks || cfg.threads < 32 || cfg.threads > 512) return cudaErrorInvalidConfiguration;
  if (a.opt.kind != OPT_NONE) {
    if (!(param_dtype == dtype)) return cudaErrorInvalidValue;
    if (dtype == DType::BF16 || dtype == DType::F16) {
      // the fp32 arrays that go with 16-bit gradients are accessed 32 bytes at a time
      for (int r = 0; r < a.nranks_here; r++)
        if ((((uintptr_t)a.r[r].master | (uintptr_t)a.r[r].state1 | (uintptr_t)a.r[r].state2) & 31) != 0) return cudaErrorMisalignedAddress;
    }
    switch (dtype) {
      case DType::F32: return dispatch_fused<float>(a, cfg, s);
      case DType::BF16: return dispatch_fused<__nv_bfloat16>(a, cfg, s);
      case DType::F16: return dispatch_fused<__half>(a, cfg, s);
      default: return cudaErrorInvalidValue;
    }
  }
  switch (dtype) {
    case DType::F32: return dispatch_plain<float>(a, cfg, s);
    case DType::BF16: return dispatch_plain<__nv_bfloat16>(a, cfg, s);
    case DType::F16: return dispatch_plain<__half>(a, cfg, s);
    case DType::I32: return dispatch_plain<int32_t>(a, cfg, s);
    case DType::I64: return dispatch_plain<int64_t>(a, cfg, s);
    case DType::F64: return dispatch_plain<double>(a, cfg, s);
    case DType::U8: return dispatch_plain<uint8_t>(a, cfg, s);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launch_copy(void* dst, const void* src, size_t bytes, cudaStream_t s) {
  if (bytes == 0) return cudaSuccess;
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) != 0) return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s);
  const size_t npacks = bytes / 16;
  const int ntail = (int)(bytes % 16);
  int blocks = (int)((npacks + 512 * 8 - 1) / (512 * 8));
  if (blocks < 1) blocks = 1;
  if (blocks > 592) blocks = 592;
  copy_kernel<<<blocks, 512, 0, s>>>((uint4*)dst, (const uint4*)src, npacks, (char*)dst + npacks * 16,
                                     (const char*)src + npacks * 16, ntail);
  return cudaGetLastError();
}

int max_emulated_blocks(int device, int nranks, int threads) {
  int per_sm = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)allreduce_kernel<float, ALGO_TWO, OPT_ADAM>, threads, 0) != cudaSuccess) return 1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 1;
  int total = per_sm * sms;
  int g = total / (nranks > 0 ? nranks : 1);
  if (g > kMaxBlocks) g = kMaxBlocks;
  return g < 1 ? 1 : g;
}

int choose_blocks(size_t bytes, int world, int algo, bool fused_opt, int sm_count, int cap_override, bool beside_compute) {
  // How much payload one block of 512 threads should have, and how many blocks pay at most.
  //   one-shot : every block loads all P copies of its packs, so the work per byte grows with P;
  //              the messages are small (latency-bound), one block per 32 KiB. (Two ranks use it
  //              for staged tensors of any size: up to one block per SM, as two-shot below.)
  //   two-shot : a rank reduces 1/P of the message but reads it from P places and stores it to
  //              P places over NVLink: one block per 32 KiB, up to 128 (64 SMs at two resident
  //              blocks each); with two ranks each rank owns half of the message, up to one
  //              block per SM.
  //   NVLS     : the switch does the reduction and the fan-out, a thread only issues one
  //              multimem load and one store per 16 bytes, and FEW blocks do that best: measured
  //              on 4 GPUs in place, 64 MiB runs at 618 GB/s bus bandwidth with 16 blocks, 607
  //              with 32, 589 with 64, 545 with 128 (16 MiB: 488 / 462 / 402 / 405), and only
  //              from 512 MiB on 32 blocks are ahead of 16 (682 against 679). One block per
  //              64 KiB, up to 16, and up to 32 above 256 MiB. On 8 GPUs a rank's share of the
  //              switch traffic is spread over more, shorter requests and 64 blocks measured
  //              best or within 2 % of it at every size (16 MiB: 300 GB/s with 32 blocks, 348
  //              with 64, 327-344 with 128; 256 MiB: 638 / 671 / 641-672; 512 MiB: 731 / 750 /
  //              738-753; fewer than 32 were not measured there): more than 4 ranks, up to 64.
  //   fused update: the second phase streams the parameters and the optimizer state through
  //              HBM (6 to 9 times the gradient bytes) and wants every SM: two blocks per SM.
  //   beside compute: gradient buckets that go out while backward runs share the GPU with
  //              compute kernels that may want most SMs for milliseconds: the persistent GRU
  //              layer is a cooperative launch of 128 blocks that each need an SM of their own,
  //              so it cannot start while more than sm_count - 128 SMs hold a block of another
  //              kernel. Blocks are spread one per SM while SMs are free; a grid of at most
  //              sm_count - 128 blocks (20 on B200) therefore never keeps such a layer waiting,
  //              whichever of the two kernels starts first, and all of its own blocks are
  //              resident together on every rank, so no barrier waits for a block that cannot
  //              start. Measured with 40 blocks on one GPU: every bucket launch delayed the next
  //              layer's kernel, 0.8 ms per step in total. At least 8.
  size_t per_block = 32u << 10;
  int cap = 128;
  if (algo == (int)Algo::NVLS) {
    per_block = 64u << 10;
    cap = world > 4 ? 64 : bytes <= (256u << 20) ? 16 : 32;
  } else if (world == 2) {
    cap = sm_count;
  }
  if (fused_opt) {
    per_block = 32u << 10;
    cap = 2 * sm_count;
  }
  if (beside_compute) {
    const int free_sms = sm_count - 128;
    cap = free_sms > 8 ? free_sms : 8;
  }
  if (cap_override > 0) cap = cap_override;
  if (cap > kMaxBlocks) cap = kMaxBlocks;
  size_t want = (bytes + per_block - 1) / per_block;
  if (want < 1) want = 1;
  return (int)(want > (size_t)cap ? (size_t)cap : want);
}

}  // namespace gpu
}  // namespace bc
