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
// Synchronisation. Progress words live in every rank's signal pad, per peer q and group of blocks:
//   staged[q]  = chunks that rank q has copied into its staging buffer,
//   reduced[q] = chunks of which rank q has reduced its share,
// counted from `base` on (the host adds up what all launches of a channel contribute, so the
// words only grow and need no reset). The last copier block that finishes chunk c on a rank (a
// local arrival counter tells) publishes "staged" into every rank's pad: one system-scope fence,
// then a plain store per peer. Reducers wait until all P staged words have reached their chunk;
// the last reducer block that finishes chunk c publishes "reduced" the same way; copiers wait for
// all P reduced words before they copy chunk c out. Nobody waits at a barrier: ranks and roles
// drift apart as far as the data allows. A rank's kernel ends only after its last copy-out, i.e.
// after every rank has reduced every chunk, so no peer reads this rank's staging buffer any
// more when the next launch overwrites it. Every wait is bounded (status word, early return).
//
// The staging buffer is a ring of `slots` chunks: chunk c lives in slot c % slots, so one launch
// takes a tensor of any size through a staging area of a few tens of MiB. A copier thread
// handles the same offsets of a slot for every chunk (`slots` and the lag of the copy-out are
// multiples of `cgroups`, so a slot always belongs to the same group of copiers), copies chunk c
// out before it copies chunk c + slots in (the copy-out trails the copy-in by fewer chunks than
// the ring has slots), and has by then seen every rank's "reduced" word for chunk c: nothing in
// a slot is overwritten while anybody still needs it.
//
// Groups. The copier blocks form `cgroups` groups; group g takes the chunks c with
// c % cgroups == g, so that several chunks are on their way at once and the pause of one group
// between two chunks (publish, wait) is covered by the others. Reducer blocks come in two kinds:
// draining ones (`streaming` = 0: wait, reduce, publish chunk by chunk, in `rgroups` groups that
// hide one another's pauses; 4 GPUs, 1 GiB fp32 in 2 MiB chunks: 6.74 ms with one group of 16
// blocks, 2.74 ms with eight groups of 4) and streaming ones (below: a block never pauses;
// 2.45 ms), which the library uses.
//
// All blocks of a launch must be resident at once (reducers and copiers wait for one another),
// one block per SM (`__launch_bounds__(544, 1)`); the host sizes the grid accordingly.
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



// ---- streaming reducer ---------------------------------------------------------------------------
// A reducer block that waits for a chunk, reduces it and publishes it drains twice per chunk: its
// last stores must be acknowledged before it may tell the peers, and the first loads of the next
// chunk start from an empty pipeline. Here the block splits the work by warp instead. All warps
// but the last move data and never wait for memory they do not need: a warp walks through the batches
// of all its chunks in ONE software pipeline (the loads of the next batch, which may belong to
// the next chunk, are issued before the stores of the current one), reads "chunks staged so
// far" from shared memory before it enters a chunk, and adds one to a counter in shared memory
// when it has issued its last store of a chunk. The last warp does the waiting: it polls the progress
// words of the copiers (ld.acquire.sys) and raises the shared "staged" count, and when all data
// warps have counted a chunk it fences, counts the block in (the global arrival counter of the
// chunk) and, as the last block, publishes the chunk to every rank. The counters in shared
// memory are written with release and read with acquire semantics at CTA scope, so the fence of
// the last warp covers the data warps' stores (the same chain as bar.sync + fence in a plain block).
// Every wait is a bounded poll; a warp that gives up raises the shared error word, which ends
// all warps of the block.
constexpr int kDoneRing = 8;   // chunks that the data warps may be ahead of the publisher

struct StreamShared {
  uint32_t staged;             // chunks ch < staged are staged on every rank
  uint32_t published;          // how many of this block's chunks the last warp has retired
  uint32_t error;
  uint32_t done[kDoneRing];    // data warps that have finished chunk number k (slot k % kDoneRing)
};

__device__ __forceinline__ uint32_t ld_acquire_cta_shared(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"((uint32_t)__cvta_generic_to_shared(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_cta_shared(uint32_t* p, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_cta_shared_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.cta.shared.add.u32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(p)), "r"(v) : "memory");
}

// Polls shared memory until pred() holds; false when the block has failed or the wait ran out.
template <typename Pred>
__device__ __forceinline__ bool poll_shared(StreamShared& sh, const RankCtx& c, uint32_t what, Pred pred) {
  if (pred()) return true;
  const unsigned long long t0 = global_timer();
  uint32_t spins = 0;
  while (true) {
    if (pred()) return true;
    if (ld_acquire_cta_shared(&sh.error)) return false;
    if (((++spins) & 0x3ff) == 0 && global_timer() - t0 > c.timeout_ns) {
      atomicOr(c.status, kStatusTimeout | what | ((uint32_t)c.rank << 8));
      st_release_cta_shared(&sh.error, 1u);
      return false;
    }
  }
}

template <typename T, bool NVLS>
__device__ void reduce_streaming(const PipeArgs& a, const PipeRank& R, StreamShared& sh) {
  using PK = Pack<T>;
  using Acc = typename PK::Acc;
  constexpr int E = PK::kElems;
  constexpr bool kSwitch = NVLS && SwitchAdds<T>::value;
  constexpr int U = kSwitch ? 4 : 2;   // packs per batch (peer variant: P loads per pack)
  const RankCtx& c = R.ctx;
  const int P = c.world, me = c.rank;
  const int GR = a.rgroups, GC = a.cgroups;
  const int grp = (int)blockIdx.x % GR, nb = a.reducers / GR;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kDataWarps = (int)(blockDim.x >> 5) - 1;   // 16 in a launch of 544 threads, 15 in one of 512
  const uint32_t* words = R.progress[me];
  const int mine = a.nchunks > grp ? (a.nchunks - grp + GR - 1) / GR : 0;   // chunks of this block's group

  if (threadIdx.x == 0) {
    sh.staged = 0;
    sh.published = 0;
    sh.error = 0;
    for (int i = 0; i < kDoneRing; i++) sh.done[i] = 0;
  }
  __syncthreads();

  if (warp == kDataWarps) {
    // ---- the warp that waits ----
    uint32_t staged = 0;       // chunks [0, staged) are staged everywhere
    int retired = 0;           // chunks of this group that are published
    unsigned long long t_progress = global_timer();
    while (retired < mine) {
      bool moved = false;
      // (a) has every rank staged the next chunk?
      if ((int)staged < a.nchunks) {
        int ok = 1;
        if (lane < P) ok = (int32_t)(ld_acquire_sys(words + ((int)staged % GC) * kMaxRanks + lane) - (a.base + staged / GC + 1)) >= 0;
        if (__all_sync(0xffffffffu, ok)) {
          staged++;
          if (lane == 0) st_release_cta_shared(&sh.staged, staged);
          moved = true;
        }
      }
      // (b) have all data warps issued the last store of the oldest unpublished chunk?
      uint32_t cnt = 0;
      if (lane == 0) cnt = ld_acquire_cta_shared(&sh.done[retired % kDoneRing]);
      cnt = __shfl_sync(0xffffffffu, cnt, 0);
      if (cnt == (uint32_t)kDataWarps) {
        const int ch = grp + retired * GR;
        if (lane == 0) {
          sh.done[retired % kDoneRing] = 0;
          // acq_rel: the data warps' stores (acquired above) are ordered before the count
          if (atom_add_acq_rel_gpu(R.local + a.nchunks + ch, 1u) == (uint32_t)nb - 1) {
            __threadfence_system();
            for (int p = 0; p < P; p++) st_relaxed_sys(R.progress[p] + (kPipeMaxGroups + grp) * kMaxRanks + me, a.base + (uint32_t)(ch / GR) + 1);
          }
          st_release_cta_shared(&sh.published, (uint32_t)retired + 1);
        }
        retired++;
        moved = true;
      }
      if (moved) {
        t_progress = global_timer();
      } else {
        int bad = ld_acquire_cta_shared(&sh.error) != 0;
        if (!bad && global_timer() - t_progress > c.timeout_ns) {
          bad = 1;
          if (lane == 0) {
            atomicOr(c.status, kStatusTimeout | 0x10000u | ((uint32_t)c.rank << 8));
            st_release_cta_shared(&sh.error, 1u);
          }
        }
        if (__any_sync(0xffffffffu, bad)) return;
      }
    }
    return;
  }

  // ---- data warps ----
  const size_t tid = (size_t)((int)blockIdx.x / GR) * (kDataWarps * 32) + threadIdx.x;
  const size_t stride = (size_t)nb * (kDataWarps * 32), step = stride * U;
  // position of a batch: chunk number k of this group (chunk grp + k * GR), first pack i0, end of the share
  struct Pos { int k; size_t i0, se; };
  auto enter = [&](int k, Pos& p) {   // first batch of chunk k of this thread (may be empty: i0 >= se)
    const int ch = grp + k * GR;
    const size_t cb = (size_t)ch * a.chunk_packs, ce = cb + a.chunk_packs < a.npacks ? cb + a.chunk_packs : a.npacks;
    const size_t n = ce - cb, slot0 = (size_t)(ch % a.slots) * a.chunk_packs;
    p.k = k;
    p.i0 = slot0 + n * (size_t)me / P + tid;
    p.se = slot0 + n * (size_t)(me + 1) / P;
  };
  // May the warp touch chunk k? (staged everywhere, and its slot of the done ring is free)
  // Lane 0 polls for the warp, so that all lanes get the same answer.
  auto admit = [&](int k) {
    const uint32_t ch = (uint32_t)(grp + k * GR);
    int ok = 1;
    if (lane == 0)
      ok = poll_shared(sh, c, 0x40000u, [&] {
        return ld_acquire_cta_shared(&sh.staged) > ch && (uint32_t)k - ld_acquire_cta_shared(&sh.published) < (uint32_t)kDoneRing;
      });
    ok = __shfl_sync(0xffffffffu, ok, 0);
    __syncwarp();
    return ok != 0;
  };
  auto load_batch = [&](const Pos& p, uint4* r) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const size_t i = p.i0 + (size_t)u * stride;
      if (i < p.se) {
        if constexpr (kSwitch) {
          r[u] = switch_reduce<T>(R.mc_stage + i * 16);
        } else {
          Acc acc[E];
          PK::unpack(ld_stream16(R.stage[0] + i * 16), acc);
          for (int q = 1; q < P; q++) {
            Acc tmp[E];
            PK::unpack(ld_stream16(R.stage[q] + i * 16), tmp);
#pragma unroll
            for (int e = 0; e < E; e++) acc[e] = acc[e] + tmp[e];
          }
#pragma unroll
          for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
          r[u] = PK::pack(acc);
        }
      }
    }
  };
  auto store_batch = [&](const Pos& p, uint4* r) {
#pragma unroll
    for (int u = 0; u < U; u++) {
      const size_t i = p.i0 + (size_t)u * stride;
      if (i < p.se) {
        if constexpr (kSwitch) {
          if (a.scale != 1.f) {
            Acc acc[E];
            PK::unpack(r[u], acc);
#pragma unroll
            for (int e = 0; e < E; e++) acc[e] = finish<Acc>(acc[e], a.scale, a.idiv);
            r[u] = PK::pack(acc);
          }
          multimem_st16(R.mc_stage + i * 16, r[u]);
        } else {
          for (int q = 0; q < P; q++) st16(R.stage[q] + i * 16, r[u]);
        }
      }
    }
  };
  if (mine == 0) return;
  // Where is the batch after `cur`? The next one of the same chunk, or the first one of the
  // group's next chunk if the warp may enter it already (kNext: its loads go out before the
  // stores of `cur`, across the chunk boundary). If that chunk is not staged yet (kWait) the warp
  // first finishes `cur`, so that nobody waits for this chunk longer than necessary, and then
  // waits. The lanes of a warp cross chunk boundaries together: lane 0, which holds the warp's
  // lowest pack, decides.
  enum { kNext, kEnd, kWait };
  auto advance = [&](const Pos& cur, Pos& nx, bool& last_of_chunk) {
    last_of_chunk = false;
    nx = cur;
    const size_t lane0_next = __shfl_sync(0xffffffffu, cur.i0, 0) + step;
    if (lane0_next < cur.se) {
      nx.i0 = cur.i0 + step;
      return (int)kNext;
    }
    last_of_chunk = true;
    if (cur.k + 1 >= mine) return (int)kEnd;
    int open = 0;
    if (lane == 0) {
      const uint32_t ch = (uint32_t)(grp + (cur.k + 1) * GR);
      open = ld_acquire_cta_shared(&sh.staged) > ch && (uint32_t)(cur.k + 1) - ld_acquire_cta_shared(&sh.published) < (uint32_t)kDoneRing;
    }
    open = __shfl_sync(0xffffffffu, open, 0);
    __syncwarp();
    if (!open) return (int)kWait;
    enter(cur.k + 1, nx);
    return (int)kNext;
  };
  auto chunk_done = [&](int k) {
    __syncwarp();
    if (lane == 0) red_release_cta_shared_add(&sh.done[k % kDoneRing], 1u);
  };
  Pos cur, nx;
  bool last_of_chunk;
  uint4 ra[U], rb[U];
  if (!admit(0)) return;
  enter(0, cur);
  load_batch(cur, ra);
  while (true) {
    int st = advance(cur, nx, last_of_chunk);
    if (st == kNext) load_batch(nx, rb);
    store_batch(cur, ra);
    if (last_of_chunk) chunk_done(cur.k);
    if (st == kEnd) break;
    if (st == kWait) {
      if (!admit(cur.k + 1)) return;
      enter(cur.k + 1, nx);
      load_batch(nx, rb);
    }
    cur = nx;
    st = advance(cur, nx, last_of_chunk);
    if (st == kNext) load_batch(nx, ra);
    store_batch(cur, rb);
    if (last_of_chunk) chunk_done(cur.k);
    if (st == kEnd) break;
    if (st == kWait) {
      if (!admit(cur.k + 1)) return;
      enter(cur.k + 1, nx);
      load_batch(nx, ra);
    }
    cur = nx;
  }
}

template <typename T, bool NVLS>
__global__ void __launch_bounds__(544, 1) staged_pipeline_kernel(const __grid_constant__ PipeArgs a) {
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

  __shared__ StreamShared sh;
  if ((int)blockIdx.x < NB && a.streaming) {
    reduce_streaming<T, NVLS>(a, R, sh);
    return;
  }
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
  if (a.nchunks < 1 || a.nchunks > kPipeMaxChunks || a.reducers < 1 || cfg.blocks <= a.reducers || (cfg.threads != 512 && cfg.threads != 544)) return cudaErrorInvalidConfiguration;
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
