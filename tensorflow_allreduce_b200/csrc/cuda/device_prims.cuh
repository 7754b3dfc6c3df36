// Device-side building blocks for the peer-memory collectives (sm_100a).
//
// Every rank maps every peer's symmetric buffers and "signal pads" into its own address space
// (NVLink 5 through NVSwitch: each peer is one hop). A collective is ONE kernel per rank that
//   * meets its peers at a flag barrier (st.release.sys / ld.acquire.sys on the pads),
//   * loads peers' data with 16-byte ld.global, or lets the switch reduce it (multimem.ld_reduce),
//   * reduces in registers in a fixed rank order, so every rank gets bit-identical results,
//   * and runs its epilogue (scale, cast, optimizer update) on the reduced registers.
// This replaces the reference's N-1 host-driven MPI steps with a 32x256 accumulate launch and a
// stream synchronise after each (tensorflow/contrib/mpi_collectives/ring.cu.cc:41-69,
// ring.h:183-225).
//
// Every wait is bounded: when a peer does not show up within `timeout_ns` the block records a
// status word that the host can read and the kernel returns; nothing traps and nothing spins
// for ever.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "layout.h"

namespace bc {
namespace dev {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_timer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// 16-byte accesses to symmetric (possibly remote) memory. They are ordinary weak accesses: the
// flag barrier that precedes them (acquire at system scope by threads of this block, then
// bar.sync) makes the peers' earlier writes visible and drops stale L1 lines, and the barrier that
// follows them publishes the stores. Reads do not allocate in L1: every element is used once.
// Measured on B200 over NVLink 5, weak accesses stream a few percent faster than .relaxed.sys ones.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st16(void* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_local16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_local16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// 32-byte accesses (sm_100: 256-bit global loads and stores) for the fp32 arrays that go with a
// 16-byte pack of 16-bit gradients: eight floats per thread in ONE instruction. Two 16-byte
// accesses per thread instead make every warp-wide instruction touch only half of each 32-byte
// sector (the second instruction then hits L1: measured 54 % L1 hit rate and the load/store
// queue as a stall reason in the Adam epilogue). `p` must be 32-byte aligned.
__device__ __forceinline__ void ld_local32(const float* p, float* o) {
  asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=f"(o[0]), "=f"(o[1]), "=f"(o[2]), "=f"(o[3]), "=f"(o[4]), "=f"(o[5]), "=f"(o[6]), "=f"(o[7]) : "l"(p));
}
__device__ __forceinline__ void st_local32(float* p, const float* o) {
  asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(o[0]), "f"(o[1]), "f"(o[2]), "f"(o[3]),
               "f"(o[4]), "f"(o[5]), "f"(o[6]), "f"(o[7]) : "memory");
}

// NVLS: the switch sums the 16 bytes at this multicast address over all bound GPUs.
__device__ __forceinline__ uint4 multimem_ld_reduce_f32(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f16(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
// NVLS: the switch stores the 16 bytes into every bound GPU's copy.
__device__ __forceinline__ void multimem_st16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Flag barrier between block `blockIdx.x` of every rank on this channel.
//
// `epoch` is a per-thread copy of the block's epoch counter (identical in all threads); it is
// advanced here. Thread p < world publishes the new epoch into rank p's pad and then waits for
// rank p's epoch in its own pad. All data written by this block before the call is visible to
// the peers' blocks after they leave the barrier (bar.sync orders the block's writes before the
// system-scope release; the acquire plus bar.sync on the other side order the reads after it).
// Returns false (in every thread of the block) if a peer did not arrive in time.
__device__ __forceinline__ bool peer_barrier(const RankCtx& c, uint32_t& epoch) {
  __syncthreads();
  epoch += 1;
  int ok = 1;
  if ((int)threadIdx.x < c.world) {
    const int peer = threadIdx.x;
    st_release_sys(c.flags[peer] + (size_t)blockIdx.x * kMaxRanks + c.rank, epoch);
    const uint32_t* mine = c.flags[c.rank] + (size_t)blockIdx.x * kMaxRanks + peer;
    const unsigned long long t0 = global_timer();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (((++spins) & 0xff) == 0 && global_timer() - t0 > c.timeout_ns) {
        ok = 0;
        atomicOr(c.status, kStatusTimeout | (1u << peer) | ((uint32_t)c.rank << 8));
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// Barrier among the blocks of this rank's launch: blocks with `arrive` add one to the rank's
// counter, every block waits until the counter has reached `target` (arrivals are counted from
// RankCtx::local_base on, see there). All blocks of the launch must be able to be resident at
// the same time; the wait is bounded like every other. Returns false in every thread of the
// block when it ran out.
__device__ __forceinline__ bool local_barrier(const RankCtx& c, uint32_t target, bool arrive) {
  __syncthreads();
  int ok = 1;
  if (threadIdx.x == 0) {
    if (arrive) {
      __threadfence();
      atomicAdd(c.local_ctr, 1u);
    }
    const unsigned long long t0 = global_timer();
    uint32_t spins = 0, seen;
    do {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(c.local_ctr) : "memory");
      if ((int32_t)(seen - target) >= 0) break;
      if (((++spins) & 0xff) == 0 && global_timer() - t0 > c.timeout_ns) {
        ok = 0;
        atomicOr(c.status, kStatusTimeout | 0x80u | ((uint32_t)c.rank << 8));
        break;
      }
    } while (true);
  }
  return __syncthreads_and(ok) != 0;
}

// Bounds-checked builds (-DBC_DEBUG, `build.build(debug=True)` -> lib/libbcoll_debug.so, loaded
// when BC_DEBUG_KERNELS=1): every pack index and every allgather destination range is tested
// before the access; a violation sets kStatusBounds in the status word and the access is
// skipped. In normal builds the test folds to `true`.
__device__ __forceinline__ bool in_bounds(const RankCtx& c, bool ok) {
#ifdef BC_DEBUG
  if (!ok) atomicOr(c.status, kStatusBounds | ((uint32_t)c.rank << 8));
  return ok;
#else
  (void)c;
  (void)ok;
  return true;
#endif
}

__device__ __forceinline__ uint32_t load_epoch(const RankCtx& c) { return c.epochs[blockIdx.x]; }
__device__ __forceinline__ void store_epoch(const RankCtx& c, uint32_t epoch) {
  if (threadIdx.x == 0) c.epochs[blockIdx.x] = epoch;
}

// ---- 16-byte packs of each element type, accumulated in a wider/native type -----------------

template <typename T> struct Pack;  // kElems, Acc, load(uint4)->acc[], add, store(acc*scale)->uint4

template <> struct Pack<float> {
  static constexpr int kElems = 4;
  using Acc = float;
  __device__ static void unpack(uint4 v, Acc* a) {
    a[0] = __uint_as_float(v.x); a[1] = __uint_as_float(v.y); a[2] = __uint_as_float(v.z); a[3] = __uint_as_float(v.w);
  }
  __device__ static uint4 pack(const Acc* a) {
    return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
  }
};

template <> struct Pack<__nv_bfloat16> {
  static constexpr int kElems = 8;
  using Acc = float;
  __device__ static void unpack(uint4 v, Acc* a) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      a[2 * i] = __uint_as_float(w[i] << 16);
      a[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ static uint4 pack(const Acc* a) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <> struct Pack<__half> {
  static constexpr int kElems = 8;
  using Acc = float;
  __device__ static void unpack(uint4 v, Acc* a) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      float2 f = __half22float2(h);
      a[2 * i] = f.x; a[2 * i + 1] = f.y;
    }
  }
  __device__ static uint4 pack(const Acc* a) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2 h = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <> struct Pack<int32_t> {
  static constexpr int kElems = 4;
  using Acc = int32_t;
  __device__ static void unpack(uint4 v, Acc* a) { a[0] = (int)v.x; a[1] = (int)v.y; a[2] = (int)v.z; a[3] = (int)v.w; }
  __device__ static uint4 pack(const Acc* a) { return make_uint4((uint32_t)a[0], (uint32_t)a[1], (uint32_t)a[2], (uint32_t)a[3]); }
};

template <> struct Pack<int64_t> {
  static constexpr int kElems = 2;
  using Acc = long long;
  __device__ static void unpack(uint4 v, Acc* a) {
    a[0] = (long long)(((unsigned long long)v.y << 32) | v.x);
    a[1] = (long long)(((unsigned long long)v.w << 32) | v.z);
  }
  __device__ static uint4 pack(const Acc* a) {
    unsigned long long x = (unsigned long long)a[0], y = (unsigned long long)a[1];
    return make_uint4((uint32_t)x, (uint32_t)(x >> 32), (uint32_t)y, (uint32_t)(y >> 32));
  }
};

template <> struct Pack<double> {
  static constexpr int kElems = 2;
  using Acc = double;
  __device__ static void unpack(uint4 v, Acc* a) {
    a[0] = __longlong_as_double((long long)(((unsigned long long)v.y << 32) | v.x));
    a[1] = __longlong_as_double((long long)(((unsigned long long)v.w << 32) | v.z));
  }
  __device__ static uint4 pack(const Acc* a) {
    unsigned long long x = (unsigned long long)__double_as_longlong(a[0]), y = (unsigned long long)__double_as_longlong(a[1]);
    return make_uint4((uint32_t)x, (uint32_t)(x >> 32), (uint32_t)y, (uint32_t)(y >> 32));
  }
};

template <> struct Pack<uint8_t> {
  static constexpr int kElems = 16;
  using Acc = uint8_t;
  __device__ static void unpack(uint4 v, Acc* a) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 16; i++) a[i] = (uint8_t)(w[i >> 2] >> (8 * (i & 3)));
  }
  __device__ static uint4 pack(const Acc* a) {
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; i++) w[i >> 2] |= (uint32_t)a[i] << (8 * (i & 3));
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

// Sum after averaging: floating types multiply by `scale`; integer types divide by `idiv`
// (truncating), the behaviour of an integer tf.div in the reference
// (tensorflow/contrib/mpi_collectives/__init__.py:160-164).
template <typename Acc> __device__ __forceinline__ Acc finish(Acc v, float scale, int idiv);
template <> __device__ __forceinline__ float finish<float>(float v, float scale, int) { return v * scale; }
template <> __device__ __forceinline__ double finish<double>(double v, float scale, int) { return v * (double)scale; }
template <> __device__ __forceinline__ int32_t finish<int32_t>(int32_t v, float, int idiv) { return idiv > 1 ? v / idiv : v; }
template <> __device__ __forceinline__ long long finish<long long>(long long v, float, int idiv) { return idiv > 1 ? v / idiv : v; }
template <> __device__ __forceinline__ uint8_t finish<uint8_t>(uint8_t v, float, int idiv) { return idiv > 1 ? (uint8_t)(v / idiv) : v; }

}  // namespace dev
}  // namespace bc
