// Variable-length allgather over peer-mapped memory (sm_100a).
//
// Every rank owns a slab of `bytes` bytes (its rows of the gathered tensor; the first dimension
// may differ per rank, the other dimensions are equal). In ONE launch each rank
//   1. publishes (bytes, offset of its output inside its symmetric segment) into every peer's
//      signal pad and meets the peers at a flag barrier,
//   2. computes every displacement on the device as a prefix sum of the published sizes,
//   3. stores its slab into every rank's output at that displacement: with one multimem.st per
//      16 bytes when the outputs sit at the same segment offset on all ranks and the segment has
//      an NVLS multicast mapping (the slab then leaves this GPU once and the switch replicates
//      it), otherwise with P2P stores to each peer in turn (the local copy is one of them),
//   4. meets the peers again, after which the whole concatenation is present everywhere.
// The reference does this with a sizing allgather on the host followed by N-1 MPI_Sendrecv steps
// (tensorflow/contrib/mpi_collectives/mpi_ops.py:152-160, ring.h:236-301).
#include "collectives.h"
#include "device_prims.cuh"

namespace bc {
namespace gpu {

using namespace dev;

namespace {

// Copy `n` bytes from local `src` to (possibly remote) `dst`, spread over the whole grid.
// The widest access that both addresses allow is used for the body; ragged ends go bytewise.
__device__ __forceinline__ void push_slab(char* dst, const char* src, size_t n, size_t tid, size_t nthreads) {
  if (n == 0) return;
  const uintptr_t d = (uintptr_t)dst, s = (uintptr_t)src;
  const unsigned rel = (unsigned)((d - s) & 15);
  // Head: bytes until dst is 16-byte aligned (at most 15).
  size_t head = (16 - (d & 15)) & 15;
  if (head > n) head = n;
  if (tid < head) dst[tid] = src[tid];
  dst += head; src += head; n -= head;
  if (n == 0) return;
  size_t body = 0;
  if (rel == 0) {
    const size_t k = n / 16;
    // four independent 16-byte loads per thread before the first store
    size_t i = tid;
    for (; i + 3 * nthreads < k; i += 4 * nthreads) {
      const uint4 v0 = ld_local16(src + i * 16), v1 = ld_local16(src + (i + nthreads) * 16);
      const uint4 v2 = ld_local16(src + (i + 2 * nthreads) * 16), v3 = ld_local16(src + (i + 3 * nthreads) * 16);
      st16(dst + i * 16, v0);
      st16(dst + (i + nthreads) * 16, v1);
      st16(dst + (i + 2 * nthreads) * 16, v2);
      st16(dst + (i + 3 * nthreads) * 16, v3);
    }
    for (; i < k; i += nthreads) st16(dst + i * 16, ld_local16(src + i * 16));
    body = k * 16;
  } else if ((rel & 7) == 0) {
    const size_t k = n / 8;
    for (size_t i = tid; i < k; i += nthreads) reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(src)[i];
    body = k * 8;
  } else if ((rel & 3) == 0) {
    const size_t k = n / 4;
    for (size_t i = tid; i < k; i += nthreads) reinterpret_cast<uint32_t*>(dst)[i] = reinterpret_cast<const uint32_t*>(src)[i];
    body = k * 4;
  } else if ((rel & 1) == 0) {
    const size_t k = n / 2;
    for (size_t i = tid; i < k; i += nthreads) reinterpret_cast<uint16_t*>(dst)[i] = reinterpret_cast<const uint16_t*>(src)[i];
    body = k * 2;
  }
  for (size_t i = body + tid; i < n; i += nthreads) dst[i] = src[i];
}

// Multicast variant: `dst` is an address in the multicast mapping, so every store lands in every
// rank's segment. multimem stores are at least 4 bytes wide; the caller guarantees that dst, src
// and n are multiples of 4.
__device__ __forceinline__ void mc_st4(void* p, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void mc_st8(void* p, uint2 v) {
  unsigned long long w = ((unsigned long long)v.y << 32) | v.x;
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}

__device__ __forceinline__ void push_slab_mc(char* dst, const char* src, size_t n, size_t tid, size_t nthreads) {
  if (n == 0) return;
  const uintptr_t d = (uintptr_t)dst, s = (uintptr_t)src;
  const unsigned rel = (unsigned)((d - s) & 15);
  const unsigned width = rel == 0 ? 16 : ((rel & 7) == 0 ? 8 : 4);
  // Head: 4-byte words until dst is aligned to the body's access width.
  size_t head = (width - (d & (width - 1))) & (width - 1);
  if (head > n) head = n;
  if (tid < head / 4) mc_st4(dst + tid * 4, reinterpret_cast<const uint32_t*>(src)[tid]);
  dst += head; src += head; n -= head;
  if (n == 0) return;
  size_t body = 0;
  if (width == 16) {
    const size_t k = n / 16;
    size_t i = tid;
    for (; i + 3 * nthreads < k; i += 4 * nthreads) {
      const uint4 v0 = ld_local16(src + i * 16), v1 = ld_local16(src + (i + nthreads) * 16);
      const uint4 v2 = ld_local16(src + (i + 2 * nthreads) * 16), v3 = ld_local16(src + (i + 3 * nthreads) * 16);
      multimem_st16(dst + i * 16, v0);
      multimem_st16(dst + (i + nthreads) * 16, v1);
      multimem_st16(dst + (i + 2 * nthreads) * 16, v2);
      multimem_st16(dst + (i + 3 * nthreads) * 16, v3);
    }
    for (; i < k; i += nthreads) multimem_st16(dst + i * 16, ld_local16(src + i * 16));
    body = k * 16;
  } else if (width == 8) {
    const size_t k = n / 8;
    for (size_t i = tid; i < k; i += nthreads) mc_st8(dst + i * 8, reinterpret_cast<const uint2*>(src)[i]);
    body = k * 8;
  }
  const size_t words = (n - body) / 4;
  for (size_t i = tid; i < words; i += nthreads) mc_st4(dst + body + i * 4, reinterpret_cast<const uint32_t*>(src + body)[i]);
}

__global__ void __launch_bounds__(512) allgatherv_kernel(const __grid_constant__ AgArgs a) {
  const AgRank& R = a.r[blockIdx.y];
  const RankCtx& c = R.ctx;
  const int P = c.world, me = c.rank;
  __shared__ unsigned long long s_bytes[kMaxRanks];
  __shared__ unsigned long long s_off[kMaxRanks];

  uint32_t epoch = load_epoch(c);
  // Publish my size and output offset into slot [block][me] of every peer's metadata area.
  if ((int)threadIdx.x < P) {
    uint64_t* slot = c.meta[threadIdx.x] + ((size_t)blockIdx.x * kMaxRanks + me) * 2;
    slot[0] = R.bytes;
    slot[1] = R.out_off;
  }
  if (P > 1) {
    if (!peer_barrier(c, epoch)) { store_epoch(c, epoch); return; }
  } else {
    __syncthreads();
  }
  if ((int)threadIdx.x < P) {
    const volatile uint64_t* slot = c.meta[me] + ((size_t)blockIdx.x * kMaxRanks + threadIdx.x) * 2;
    s_bytes[threadIdx.x] = slot[0];
    s_off[threadIdx.x] = slot[1];
  }
  __syncthreads();
  unsigned long long disp = 0;
  for (int q = 0; q < me; q++) disp += s_bytes[q];
  if (R.sizes_out && blockIdx.x == 0 && (int)threadIdx.x < P) R.sizes_out[threadIdx.x] = s_bytes[threadIdx.x];

  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t nthreads = (size_t)gridDim.x * blockDim.x;
  {
    unsigned long long total = 0;
    for (int q = 0; q < P; q++) total += s_bytes[q];
    bool fits = true;
    for (int q = 0; q < P; q++) fits = fits && (R.capacity == 0 || s_off[q] + total <= R.capacity);
    if (!in_bounds(c, fits)) {   // bounds-checked builds: refuse to store past a segment
      if (P > 1) peer_barrier(c, epoch);
      store_epoch(c, epoch);
      return;
    }
  }
  bool multicast = R.mc_base != nullptr;
  for (int q = 1; q < P; q++) multicast = multicast && s_off[q] == s_off[0];
  multicast = multicast && ((((uintptr_t)R.in) | (s_off[0] + disp) | R.bytes) & 3) == 0;
  if (multicast) {
    // One store per 16 bytes; the switch delivers it to every rank, this one included.
    push_slab_mc(R.mc_base + s_off[0] + disp, R.in, (size_t)R.bytes, tid, nthreads);
  } else {
    // Start with the next rank so that at any moment the P ranks write to P different targets.
    for (int k = 0; k < P; k++) {
      const int p = (me + 1 + k) % P;
      push_slab(R.base[p] + s_off[p] + disp, R.in, (size_t)R.bytes, tid, nthreads);
    }
  }
  if (P > 1) peer_barrier(c, epoch);
  store_epoch(c, epoch);
}

struct ProbeArgs {
  int n;
  int absent;
  RankCtx c[kMaxRanks];
};

// Barrier only. The block of rank `absent` leaves at once, so the others exercise the bounded wait.
__global__ void barrier_probe_kernel(const __grid_constant__ ProbeArgs a) {
  if ((int)blockIdx.y == a.absent) return;
  const RankCtx& c = a.c[blockIdx.y];
  uint32_t epoch = load_epoch(c);
  peer_barrier(c, epoch);
  store_epoch(c, epoch);
}

}  // namespace

cudaError_t launch_barrier_probe(const RankCtx* ctxs, int nranks, int absent, cudaStream_t s) {
  ProbeArgs a;
  a.n = nranks;
  a.absent = absent;
  for (int r = 0; r < nranks; r++) a.c[r] = ctxs[r];
  dim3 grid(1, nranks), block(32);
  void* params[] = {(void*)&a};
  return cudaLaunchCooperativeKernel((const void*)barrier_probe_kernel, grid, block, params, 0, s);
}

cudaError_t launch_allgatherv(const AgArgs& a, const LaunchCfg& cfg, cudaStream_t s) {
  if (cfg.blocks <= 0 || cfg.blocks > kMetaBlocks || cfg.threads < 32 || cfg.threads > 512) return cudaErrorInvalidConfiguration;
  dim3 grid(cfg.blocks, a.nranks_here), block(cfg.threads);
  if (cfg.cooperative || a.nranks_here > 1) {
    void* params[] = {(void*)&a};
    return cudaLaunchCooperativeKernel((const void*)allgatherv_kernel, grid, block, params, 0, s);
  }
  allgatherv_kernel<<<grid, block, 0, s>>>(a);
  return cudaGetLastError();
}

}  // namespace gpu
}  // namespace bc
