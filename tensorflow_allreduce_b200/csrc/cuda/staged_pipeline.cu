// Allreduce of a tensor OUTSIDE symmetric memory in ONE launch whose blocks have roles: copier
// blocks bring the private input into this rank's staging buffer chunk by chunk and, a few
// chunks behind, copy finished chunks from the staging buffer to the private output; reducer
// blocks reduce chunk after chunk across the ranks as soon as every rank has staged it, in the
// switch (multimem.ld_reduce / multimem.st) or with peer loads and stores. The local copies
// (HBM-bound) therefore run beside the NVLink phase instead of before and after it, without the
// host launching anything per chunk.
//
// Reference path replaced: CopyTensorData + RingAllreduce on a tensor the framework owns
// (tensorflow/contrib/mpi_collectives/ring.h:136-228, ring.cu.cc:41-66): one D2D copy, then N-1
// send / receive / accumulate steps with a stream synchronise each.
//
// Synchronisation. Progress words live in every rank's signal pad, per peer q and group:
//   staged[q]  = chunks that rank q has copied into its staging buffer,
//   reduced[q] = chunks of which rank q has reduced its share,
// counted from `base` on (the host adds up what all launches of a channel contribute, so the
// words only grow and need no reset). The last copier block that finishes chunk c on a rank (a local
// arrival counter tells) publishes staged = base + c + 1 into every rank's pad with
// st.release.sys; reducers wait until all P staged words have reached their chunk; the last
// reducer block that finishes chunk c publishes reduced the same way; copiers wait for all P
// reduced words before they copy chunk c out. Nobody waits at a barrier: ranks and roles drift
// apart as far as the data allows. A rank's kernel ends only after its last copy-out, i.e.
// after every rank has reduced every chunk, so no peer reads this rank's staging buffer any
// more when the next launch overwrites it. Every wait is bounded (status word, early return).
#include "collectives.h"
#include "device_prims.cuh"

#include <type_traits>

namespace bc {
namespace gpu {

using namespace dev;

namespace {

__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu(uint32_t* p, uint32_t v) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}

// Threads q < world wait until word q of `words` (in this rank's own pad) has reached `target`.
// Returns false in every thread of the block if a wait ran out (`what`, bit 16 for a reducer's
// wait and bit 17 for a copier's, goes into the status word beside the peer and the rank).
__device__ __forceinline__ bool wait_words(const RankCtx& c, const uint32_t* words, uint32_t target, uint32_t what) {
  int ok = 1;
  if ((int)threadIdx.x < c.world) {
    const unsigned long long t0 = global_timer();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(words + threadIdx.x) - target) < 0) {
      if (((++spins) & 0xff) == 0 && global_timer() - t0 > c.timeout_ns) {
        ok = 0;
        atomicOr(c.status, kStatusTimeout | what | (1u << threadIdx.x) | ((uint32_t)c.rank << 8));
        break;
      }
    }
  }
  return __syncthreads_and(ok) != 0;
}

// The block has finished its part of a chunk: count it, and if it is the last of `nblocks`,
// tell every rank (this rank's word of the given kind in each pad).
// ONE system-scope fence, then plain stores: a st.release per peer waits for the previous
// peer's store to be acknowledged over NVLink before the next one leaves (measured on 4 GPUs,
// 1 GiB in 2 MiB chunks and four groups: 3.93 ms with a release per peer, 3.16 ms like this).
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void arrive_and_publish(const PipeRank& R, uint32_t* counter, int nblocks, int word, uint32_t value) {
  __syncthreads();
  if (threadIdx.x == 0) {
    // the release half of the atomic orders this block's stores (bar.sync above) before the count
    if (atom_add_acq_rel_gpu(counter, 1u) == (uint32_t)nblocks - 1) {
      __threadfence_system();
      for (int p = 0; p < R.ctx.world; p++) st_relaxed_sys(R.progress[p] + word * kMaxRanks + R.ctx.rank, value);
    }
  }
}

__device__ __forceinline__ void copy_run(char* dst, const char* src, size_t begin, size_t end, size_t first, size_t stride) {
  constexpr int U = 8;   // loads in flight per thread
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

template <typename T>
__device__ __forceinline__ uint4 switch_reduce(const char* mc) {
  if constexpr (sizeof(T) == 4) return multimem_ld_reduce_f32(mc);
  else if constexpr (std::is_same<T, __nv_bfloat16>::value) return multimem_ld_reduce_bf16(mc);
  else return multimem_ld_reduce_f16(mc);
}

template <typename T> struct SwitchAdds { static constexpr bool value = false; };
template <> struct SwitchAdds<float> { static constexpr bool value = true; };
template <> struct SwitchAdds<__nv_bfloat16> { static constexpr bool value = true; };
template <> struct SwitchAdds<__half> { static constexpr bool value = true; };


template <typename T, bool NVLS>
__global__ void __launch_bounds__(512, 1) staged_pipeline_kernel(const __grid_constant__ PipeArgs a) {
  using PK = Pack<T>;
  using Acc = typename PK::Acc;
  constexpr int E = PK::kElems;
  const PipeRank& R = a.r[blockIdx.y];
  const RankCtx& c = R.ctx;
  const int P = c.world, me = c.rank;
  const int NB = a.reducers, NC = (int)gridDim.x - NB;
  const int GR = a.rgroups, GC = a.cgroups;
  // what the ranks have told THIS rank: word (kind * kPipeMaxGroups + group) * kMaxRanks + rank
  const uint32_t* words = R.progress[me];

  if ((int)blockIdx.x < NB) {
    // ---- reducer of group blockIdx.x % GR ----
    const int grp = (int)blockIdx.x % GR, nb = NB / GR;
    const size_t first = (size_t)((int)blockIdx.x / GR) * blockDim.x + threadIdx.x, stride = (size_t)nb * blockDim.x;
    for (int ch = grp; ch < a.nchunks; ch += GR) {
      if (!wait_words(c, words + (ch % GC) * kMaxRanks, a.base + (uint32_t)(ch / GC) + 1, 0x10000u)) return;
      const size_t cb = (size_t)ch * a.chunk_packs, ce = cb + a.chunk_packs < a.npacks ? cb + a.chunk_packs : a.npacks;
      const size_t n = ce - cb;
      // this rank's share of the chunk, as pack offsets into the ring
      const size_t slot0 = (size_t)(ch % a.slots) * a.chunk_packs;
      const size_t sb = slot0 + n * (size_t)me / P, se = slot0 + n * (size_t)(me + 1) / P;
      if constexpr (NVLS && SwitchAdds<T>::value) {
        // batches of four packs, the loads of the next batch issued before the stores of this one
        constexpr int U = 4;
        auto load_batch = [&](size_t i0, uint4* r) {
#pragma unroll
          for (int u = 0; u < U; u++) {
            const size_t i = i0 + (size_t)u * stride;
            if (i < se) r[u] = switch_reduce<T>(R.mc_stage + i * 16);
          }
        };
        auto store_batch = [&](size_t i0, uint4* r) {
#pragma unroll
          for (int u = 0; u < U; u++) {
            const size_t i = i0 + (size_t)u * stride;
            if (i < se) {
              if (a.scale != 1.f) {
                Acc acc[E];
                PK::unpack(r[u], acc);
#pragma unroll
                for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
                r[u] = PK::pack(acc);
              }
              multimem_st16(R.mc_stage + i * 16, r[u]);
            }
          }
        };
        const size_t step = stride * U;
        uint4 ra[U], rb[U];
        size_t i0 = sb + first;
        if (i0 < se) load_batch(i0, ra);
        while (i0 < se) {
          const size_t i1 = i0 + step;
          if (i1 < se) load_batch(i1, rb);
          store_batch(i0, ra);
          if (i1 >= se) break;
          const size_t i2 = i1 + step;
          if (i2 < se) load_batch(i2, ra);
          store_batch(i1, rb);
          i0 = i2;
        }
      } else {
        // peer loads in rank order (bit-identical on all ranks), stores to every rank
        for (size_t i = sb + first; i < se; i += stride) {
          Acc acc[E];
          PK::unpack(ld_stream16(R.stage[0] + i * 16), acc);
          for (int p = 1; p < P; p++) {
            Acc tmp[E];
            PK::unpack(ld_stream16(R.stage[p] + i * 16), tmp);
#pragma unroll
            for (int e = 0; e < E; e++) acc[e] = acc[e] + tmp[e];
          }
#pragma unroll
          for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
          const uint4 r = PK::pack(acc);
          for (int p = 0; p < P; p++) st16(R.stage[p] + i * 16, r);
        }
      }
      arrive_and_publish(R, R.local + a.nchunks + ch, nb, kPipeMaxGroups + grp, a.base + (uint32_t)(ch / GR) + 1);
    }
    return;
  }

  // ---- copier of group (blockIdx.x - NB) % GC ----
  const int cid = (int)blockIdx.x - NB, grp = cid % GC, nc = NC / GC;
  const size_t first = (size_t)(cid / GC) * blockDim.x + threadIdx.x, stride = (size_t)nc * blockDim.x;
  for (int ch = grp; ch < a.nchunks + a.lag; ch += GC) {
    if (ch < a.nchunks) {
      const size_t cb = (size_t)ch * a.chunk_packs, ce = cb + a.chunk_packs < a.npacks ? cb + a.chunk_packs : a.npacks;
      copy_run(R.stage[me] + (size_t)(ch % a.slots) * a.chunk_packs * 16, R.src + cb * 16, 0, ce - cb, first, stride);
      arrive_and_publish(R, R.local + ch, nc, grp, a.base + (uint32_t)(ch / GC) + 1);
    }
    const int o = ch - a.lag;          // a chunk of this group as well: the lag is a multiple of GC
    if (o >= 0) {
      if (!wait_words(c, words + (kPipeMaxGroups + o % GR) * kMaxRanks, a.base + (uint32_t)(o / GR) + 1, 0x20000u)) return;
      const size_t ob = (size_t)o * a.chunk_packs, oe = ob + a.chunk_packs < a.npacks ? ob + a.chunk_packs : a.npacks;
      copy_run(R.out + ob * 16, R.stage[me] + (size_t)(o % a.slots) * a.chunk_packs * 16, 0, oe - ob, first, stride);
    }
  }
}

template <typename T>
cudaError_t launch_typed(const PipeArgs& a, bool nvls, const LaunchCfg& cfg, cudaStream_t s) {
  dim3 grid(cfg.blocks, a.nranks_here), block(cfg.threads);
  const void* fn = nvls ? (const void*)staged_pipeline_kernel<T, true> : (const void*)staged_pipeline_kernel<T, false>;
  void* params[] = {(void*)&a};
  if (cfg.cooperative || a.nranks_here > 1) return cudaLaunchCooperativeKernel(fn, grid, block, params, 0, s);
  return cudaLaunchKernel(fn, grid, block, params, 0, s);
}

}  // namespace

cudaError_t launch_staged_pipeline(const PipeArgs& a, DType dtype, bool nvls, const LaunchCfg& cfg, cudaStream_t s) {
  if (a.nchunks < 1 || a.nchunks > kPipeMaxChunks || a.reducers < 1 || cfg.blocks <= a.reducers || cfg.threads != 512) return cudaErrorInvalidConfiguration;
  if (a.rgroups < 1 || a.rgroups > kPipeMaxGroups || a.cgroups < 1 || a.cgroups > kPipeMaxGroups) return cudaErrorInvalidConfiguration;
  if (a.reducers % a.rgroups || (cfg.blocks - a.reducers) % a.cgroups) return cudaErrorInvalidConfiguration;
  if (a.chunk_packs == 0 || (size_t)a.nchunks * a.chunk_packs < a.npacks || a.slots < 1 || a.lag < 0 || a.lag % a.cgroups) return cudaErrorInvalidValue;
  // a ring that wraps: the copy-out stays fewer chunks behind than the ring holds, and a slot keeps its group
  if (a.nchunks > a.slots && (a.lag >= a.slots || a.slots % a.cgroups)) return cudaErrorInvalidValue;
  switch (dtype) {
    case DType::F32: return launch_typed<float>(a, nvls, cfg, s);
    case DType::BF16: return launch_typed<__nv_bfloat16>(a, nvls, cfg, s);
    case DType::F16: return launch_typed<__half>(a, nvls, cfg, s);
    case DType::I32: return launch_typed<int32_t>(a, false, cfg, s);
    case DType::I64: return launch_typed<int64_t>(a, false, cfg, s);
    case DType::F64: return launch_typed<double>(a, false, cfg, s);
    case DType::U8: return launch_typed<uint8_t>(a, false, cfg, s);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace gpu
}  // namespace bc
