#include "comm.h"

#include <string.h>

#include <algorithm>

namespace bc {
namespace gpu {

using namespace dev;

#define CUDA_RT(expr)                                                                            \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess) throw ::bc::Error(std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

namespace {
size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
constexpr size_t kMaxLaunchBytes = 512u << 20;
constexpr size_t kGuardBytes = 4096;   // before and after every buffer of an emulated group
constexpr int kGuardPattern = 0xA5;
unsigned long long to_ns(double s) { return (unsigned long long)(s * 1e9); }
}  // namespace

Comm::Comm(int rank, int world, int device, uint64_t job_id, const CommConfig& cfg, const HostAllgather& ag, double host_timeout_s)
    : rank_(rank), world_(world), device_(device), cfg_(cfg) {
  CUDA_RT(cudaSetDevice(device));
  CUDA_RT(cudaDeviceGetAttribute(&sm_count_, cudaDevAttrMultiProcessorCount, device));
  int lo = 0, hi = 0;
  CUDA_RT(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  // Streams that carry collective kernels (the channels and their second lanes) get the highest
  // priority, the streams of the local staging copies the lowest: where a reduction and a copy
  // become runnable together, the reduction's blocks are placed first and the copy fills what
  // is left.
  for (int c = 0; c < kChannels; c++)
    CUDA_RT(cudaStreamCreateWithPriority(&streams_[c], cudaStreamNonBlocking, c < 2 * kUserChannels ? hi : lo));
  for (int c = 0; c < kUserChannels; c++) {
    CUDA_RT(cudaEventCreateWithFlags(&fork_[c], cudaEventDisableTiming));
    for (int h = 0; h < 2; h++) CUDA_RT(cudaEventCreateWithFlags(&join_[c][h], cudaEventDisableTiming));
    for (int h = 0; h < kStageBuffers; h++) {
      CUDA_RT(cudaEventCreateWithFlags(&in_done_[c][h], cudaEventDisableTiming));
      CUDA_RT(cudaEventCreateWithFlags(&red_done_[c][h], cudaEventDisableTiming));
    }
  }
  alloc_.reset(new SymmAllocator(rank, world, device, job_id, cfg.symm_mode, cfg.use_nvls, host_timeout_s));
  pad_off_ = 0;
  staging_off_ = align_up(kPadBytes, 1u << 20);
  // one slice per user channel, each cut into kStageBuffers parts: keep all of them on 512 KiB boundaries
  cfg_.staging_bytes = align_up(std::max<size_t>(cfg_.staging_bytes, 8u << 20), (size_t)kUserChannels * kStageBuffers * (512u << 10));
  heap_off_ = staging_off_ + cfg_.staging_bytes;
  cfg_.heap_bytes = align_up(cfg_.heap_bytes, 1u << 20);
  seg0_ = alloc_->alloc(heap_off_ + cfg_.heap_bytes, ag);
  CUDA_RT(cudaMalloc(&epochs_, sizeof(uint32_t) * kChannels * (kMaxBlocks + 1)));
  CUDA_RT(cudaMemset(epochs_, 0, sizeof(uint32_t) * kChannels * (kMaxBlocks + 1)));
  CUDA_RT(cudaMalloc(&pipe_local_, sizeof(uint32_t) * kUserChannels * 2 * kPipeMaxChunks));
  CUDA_RT(cudaHostAlloc(&status_host_, 64, cudaHostAllocMapped));
  memset(status_host_, 0, 64);
  CUDA_RT(cudaHostGetDevicePointer((void**)&status_dev_, status_host_, 0));
  CUDA_RT(cudaDeviceSynchronize());
  ag(std::string());
}

Comm::~Comm() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  alloc_.reset();
  if (epochs_) cudaFree(epochs_);
  if (pipe_local_) cudaFree(pipe_local_);
  if (status_host_) cudaFreeHost(status_host_);
  for (int c = 0; c < kChannels; c++)
    if (streams_[c]) cudaStreamDestroy(streams_[c]);
  for (int c = 0; c < kUserChannels; c++) {
    if (fork_[c]) cudaEventDestroy(fork_[c]);
    for (int h = 0; h < 2; h++)
      if (join_[c][h]) cudaEventDestroy(join_[c][h]);
    for (int h = 0; h < kStageBuffers; h++) {
      if (in_done_[c][h]) cudaEventDestroy(in_done_[c][h]);
      if (red_done_[c][h]) cudaEventDestroy(red_done_[c][h]);
    }
  }
}

RankCtx Comm::make_ctx(int channel) const {
  RankCtx c;
  memset(&c, 0, sizeof(c));
  c.rank = rank_;
  c.world = world_;
  for (int p = 0; p < world_; p++) {
    char* pad = seg0_->peer[p] + pad_off_ + (size_t)channel * kChannelBytes;
    c.flags[p] = (uint32_t*)pad;
    c.meta[p] = (uint64_t*)(pad + kFlagBytes);
  }
  c.epochs = epochs_ + (size_t)channel * kMaxBlocks;
  c.local_ctr = epochs_ + (size_t)kChannels * kMaxBlocks + channel;
  c.local_base = local_arrivals_[channel];
  c.status = status_dev_;
  c.timeout_ns = to_ns(cfg_.device_timeout_s);
  return c;
}

size_t plan_gather_rounds(const unsigned long long* all_bytes, int world, size_t staging_bytes, std::vector<size_t>* piece) {
  size_t total = 0;
  for (int p = 0; p < world; p++) total += (size_t)all_bytes[p];
  BC_CHECK(staging_bytes > 32 * (size_t)world, "the staging area is too small for a gather in rounds");
  // Pieces are rounded up to 16 bytes, which can add up to 16 bytes per rank to a round.
  const size_t room = staging_bytes - 16 * (size_t)world;
  const size_t rounds = std::max<size_t>(1, (total + room - 1) / room);
  piece->assign(world, 0);
  for (int p = 0; p < world; p++) (*piece)[p] = align_up(((size_t)all_bytes[p] + rounds - 1) / rounds, 16);
  return rounds;
}

Algo select_algo(const CommConfig& cfg, int world, size_t bytes, DType dtype, bool in_place_or_fused, bool has_mc) {
  const bool is_float = dtype == DType::F32 || dtype == DType::BF16 || dtype == DType::F16;
  Algo forced = (Algo)cfg.force_algo;
  if (forced == Algo::ONE_SHOT && !in_place_or_fused) return forced;
  if (forced == Algo::TWO_SHOT) return forced;
  if (forced == Algo::NVLS && has_mc && is_float) return forced;
  if (forced != Algo::AUTO) return Algo::TWO_SHOT;
  if (!in_place_or_fused && bytes <= cfg.one_shot_max_bytes) return Algo::ONE_SHOT;
  // Two ranks, separate output: one-shot moves as many bytes over NVLink as two-shot does (each
  // rank reads the other's copy once), needs one pass instead of three over the local buffers
  // and no second exchange: measured 30 % faster for staged tensors of 64 MiB and more.
  if (!in_place_or_fused && world == 2) return Algo::ONE_SHOT;
  // With two ranks the switch-side reduction saves no traffic (each GPU moves N/2 either way)
  // and measured slower than plain peer loads and stores; it pays from four ranks on.
  if (has_mc && cfg.use_nvls && is_float && world >= 4 && bytes >= cfg.nvls_min_bytes) return Algo::NVLS;
  return Algo::TWO_SHOT;
}

PipePlan plan_pipeline(const CommConfig& cfg, size_t bytes, size_t slice_bytes, size_t unit_bytes) {
  PipePlan p;
  const size_t unit = unit_bytes ? unit_bytes : 4096;
  const int gc = std::min(std::max(cfg.pipeline_cgroups, 1), (int)kPipeMaxGroups);
  const int slots = std::max(2 * gc, cfg.pipeline_slots / gc * gc);
  // Chunks are multiples of the unit (at least one), `slots` of them inside the slice.
  // Draining reducers: at least eight chunks of at most 4 MiB. Streaming reducers (their unit is
  // one step of all ranks' reducer blocks): a 64th of the tensor, at most pipeline_chunk_bytes
  // (larger chunks lengthen the fill and the drain of the pipeline: 7.5 MiB chunks ran 64 MiB at
  // 475 GB/s, but 1 GiB at 654 against 540), but at least two steps (with one, the warp that
  // publishes cannot keep up: 64 MiB on 4 GPUs ran at 440 GB/s against 509).
  size_t chunk = unit_bytes ? std::max<size_t>(std::min(cfg.pipeline_chunk_bytes, bytes / 64), 2 * unit)
                            : std::min(std::min<size_t>(cfg.pipeline_chunk_bytes, 4u << 20), std::max<size_t>(bytes / 8, 64u << 10));
  chunk = std::min(chunk, slice_bytes / (size_t)slots);
  chunk = std::max<size_t>(chunk / unit * unit, unit);
  p.chunk_bytes = chunk;
  const size_t n = (bytes + chunk - 1) / chunk;
  p.nchunks = (int)std::min<size_t>(n, (size_t)kPipeMaxChunks);   // the caller launches again for the rest
  p.slots = std::min(slots, p.nchunks);   // fewer chunks than slots: the ring does not wrap
  p.lag = std::max(gc, slots / 2 / gc * gc);
  // A slice too small for the ring (one unit per slot can be megabytes): no plan, the caller
  // takes another path.
  if ((size_t)p.slots * chunk > slice_bytes) p.nchunks = 0;
  return p;
}

bool Comm::launch_pipeline(int channel, const char* in, char* out, size_t packs, DType dtype, float scale, int idiv, bool nvls) {
  cudaStream_t s = streams_[channel];
  const bool streaming = cfg_.pipeline_streaming;
  const int rgroups = streaming ? 1 : std::min(std::max(cfg_.pipeline_rgroups, 1), (int)kPipeMaxGroups);
  // Streaming reducers where the switch reduces: 16 blocks at every size (4 GPUs: 32 blocks ran
  // 128 MiB at 498 GB/s against 577). Larger groups have not been measured with this kernel;
  // they use the same 16, which keeps a chunk (two steps of all ranks' reducers) at 8 MiB for 8 ranks.
  int reducers = cfg_.pipeline_reducers > 0 ? cfg_.pipeline_reducers
                 : !streaming               ? (nvls ? 32 : 48)
                 : nvls                     ? 16
                                            : 32;
  reducers = (reducers + rgroups - 1) / rgroups * rgroups;
  // Every block of the launch needs an SM of its own, and all of them at once. By default the
  // launch takes at most half of the SMs, so that two such launches, or one beside another
  // collective kernel whose blocks must all be resident (a mixed grid: at most one block per SM at
  // two blocks per SM), fit on the GPU together in whichever order the ranks happened to launch
  // them (collectives on different channels, issued by different host threads, have no common
  // order). A program that never has two collectives in flight can ask for more copiers
  // (measured on 4 GPUs: 128 copiers 553 GB/s at 64 MiB and 603 at 128 MiB, 64 copiers 506 / 575).
  const int cgroups = std::min(std::max(cfg_.pipeline_cgroups, 1), (int)kPipeMaxGroups);
  const int room = cfg_.pipeline_copiers > 0 ? sm_count_ - reducers : sm_count_ / 2 - reducers;
  int copiers = std::min(cfg_.pipeline_copiers > 0 ? cfg_.pipeline_copiers : room, room) / cgroups * cgroups;
  BC_CHECK(copiers >= cgroups, "the staged pipeline kernel needs more SMs than the device has");
  // streaming: one step of a rank's reducers is blocks x 512 data threads x batch packs; a chunk is a
  // whole number of steps of every rank
  const size_t unit = streaming ? (size_t)world_ * (reducers / rgroups) * kPipeDataThreads * (nvls ? kPipeSwitchBatch : kPipePeerBatch) * 16 : 0;
  const PipePlan plan = plan_pipeline(cfg_, packs * 16, staging_slice_bytes(), unit);
  if (plan.nchunks == 0) return false;
  const size_t chunk_packs = plan.chunk_bytes / 16;
  for (size_t done = 0; done < packs;) {
    const size_t n = std::min(packs - done, chunk_packs * (size_t)kPipeMaxChunks);
    PipeArgs a;
    memset(&a, 0, sizeof(a));
    a.nranks_here = 1;
    a.npacks = n;
    a.chunk_packs = chunk_packs;
    a.nchunks = (int)((n + chunk_packs - 1) / chunk_packs);
    a.slots = std::min(plan.slots, a.nchunks);
    a.lag = plan.lag;
    a.base = pipe_base_[channel];
    a.scale = scale;
    a.idiv = idiv;
    a.rgroups = rgroups;
    a.cgroups = cgroups;
    a.reducers = reducers;
    a.streaming = streaming ? 1 : 0;
    PipeRank& r = a.r[0];
    r.ctx = make_ctx(channel);
    for (int p = 0; p < world_; p++) {
      r.stage[p] = seg0_->peer[p] + staging_offset(channel);
      r.progress[p] = (uint32_t*)(seg0_->peer[p] + pad_off_ + (size_t)channel * kChannelBytes + kFlagBytes + kMetaBytes);
    }
    r.mc_stage = seg0_->mc ? seg0_->mc + staging_offset(channel) : nullptr;
    r.src = in + done * 16;
    r.out = out + done * 16;
    r.local = pipe_local_ + (size_t)channel * 2 * kPipeMaxChunks;
    CUDA_RT(cudaMemsetAsync(r.local, 0, sizeof(uint32_t) * 2 * (size_t)a.nchunks, s));
    LaunchCfg cfg;
    if (streaming) cfg.threads = kPipeStreamingThreads;
    cfg.blocks = a.reducers + copiers;
    CUDA_RT(launch_staged_pipeline(a, dtype, nvls, cfg, s));
    pipe_base_[channel] += (uint32_t)a.nchunks;
    last_blocks = cfg.blocks;
    last_launches++;
    done += n;
  }
  return true;
}

Algo Comm::choose_algo(size_t bytes, DType dtype, bool in_place_or_fused, bool has_mc) const {
  return select_algo(cfg_, world_, bytes, dtype, in_place_or_fused, has_mc);
}

void Comm::fill_ar_rank(ArRank* r, int channel, Segment* seg, size_t off) const {
  memset(r, 0, sizeof(*r));
  r->ctx = make_ctx(channel);
  for (int p = 0; p < world_; p++) r->in[p] = seg->peer[p] + off;
  r->mc_in = seg->mc ? seg->mc + off : nullptr;
}

Algo Comm::allreduce(int channel, const void* in, void* out, size_t count, DType dtype, float scale, int idiv,
                     bool zero_copy_agreed, ReduceOp red, bool check_place) {
  CUDA_RT(cudaSetDevice(device_));
  BC_CHECK(channel >= 0 && channel < kUserChannels, "bad channel");
  cudaStream_t s = streams_[channel];
  const size_t es = dtype_size(dtype);
  const size_t bytes = count * es;
  last_launches = 0;
  if (count == 0) return Algo::ONE_SHOT;
  BC_CHECK((((uintptr_t)in | (uintptr_t)out) & 15) == 0, "allreduce: device pointers must be 16-byte aligned");
  ArArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = 1;
  a.scale = scale;
  a.idiv = idiv;
  a.red = (int)red;
  a.prof = prof_;
  LaunchCfg cfg;
  // The switch only adds; other reductions use the peer-load kernels.
  auto pick = [&](size_t nbytes, bool in_place, bool has_mc) {
    Algo g = choose_algo(nbytes, dtype, in_place, has_mc);
    return (red != ReduceOp::SUM && g == Algo::NVLS) ? Algo::TWO_SHOT : g;
  };

  if (world_ == 1) {
    if (in == out && scale == 1.f && idiv <= 1) return Algo::ONE_SHOT;
    a.algo = (int)Algo::ONE_SHOT;
    a.count = count;
    a.r[0].ctx = make_ctx(channel);
    a.r[0].in[0] = (char*)in;
    a.r[0].out = out;
    cfg.blocks = choose_blocks(bytes, 1, a.algo, true, sm_count_, cfg_.max_blocks);
    CUDA_RT(launch_allreduce(a, dtype, dtype, cfg, s));
    last_blocks = cfg.blocks;
    last_launches = 1;
    return Algo::ONE_SHOT;
  }

  Segment* seg = zero_copy_agreed ? alloc_->find(in, bytes) : nullptr;
  if (seg && in == out) {
    // In place on symmetric memory: no staging at all.
    const size_t off = (const char*)in - seg->local;
    Algo algo = pick(bytes, true, seg->mc != nullptr);
    a.algo = (int)algo;
    // Very large tensors go in pieces of kMaxLaunchBytes: measured on 8 GPUs, one 1 GiB launch
    // ran at 630 GB/s bus bandwidth where 512 MiB launches reach 790.
    for (size_t done = 0; done < bytes; done += kMaxLaunchBytes) {
      const size_t nb = std::min(kMaxLaunchBytes, bytes - done);
      fill_ar_rank(&a.r[0], channel, seg, off + done);
      a.r[0].out = (char*)out + done;
      if (check_place) a.r[0].place = 1 + (((unsigned long long)seg->id << 48) | (unsigned long long)(off + done));
      a.count = nb / es;
      cfg.blocks = choose_blocks(nb, world_, a.algo, false, sm_count_, cfg_.max_blocks);
      CUDA_RT(launch_allreduce(a, dtype, dtype, cfg, s));
      last_launches++;
    }
    last_blocks = cfg.blocks;
    return algo;
  }
  if (seg && bytes <= cfg_.one_shot_max_bytes && (Algo)cfg_.force_algo != Algo::TWO_SHOT && (Algo)cfg_.force_algo != Algo::NVLS) {
    // Small registered input, separate output: one-shot reads the peers' tensors where they are.
    const size_t off = (const char*)in - seg->local;
    fill_ar_rank(&a.r[0], channel, seg, off);
    a.r[0].out = out;
    a.algo = (int)Algo::ONE_SHOT;
    a.count = count;
    cfg.blocks = choose_blocks(bytes, world_, a.algo, false, sm_count_, cfg_.max_blocks);
    CUDA_RT(launch_allreduce(a, dtype, dtype, cfg, s));
    last_blocks = cfg.blocks;
    last_launches = 1;
    return Algo::ONE_SHOT;
  }

  // Staged, large enough for the pipeline kernel: copier blocks and reducer blocks of ONE launch
  // work on different chunks of a ring inside the channel's slice (staged_pipeline.cu).
  if (cfg_.staged_pipeline > 0 && red == ReduceOp::SUM && bytes >= cfg_.pipeline_min_bytes && bytes >= 16) {
    const Algo inplace = pick(bytes, true, seg0_->mc != nullptr);
    const bool nvls = inplace == Algo::NVLS;
    const size_t packs = bytes / 16;
    if ((nvls || cfg_.staged_pipeline > 1) && launch_pipeline(channel, (const char*)in, (char*)out, packs, dtype, scale, idiv, nvls)) {
      const size_t head = packs * (16 / es);
      if (head < count) {
        // the last few elements (less than one pack) take the small-tensor path
        const int launches = last_launches, blocks = last_blocks;
        allreduce(channel, (const char*)in + head * es, (char*)out + head * es, count - head, dtype, scale, idiv, false, red, false);
        last_launches += launches;
        last_blocks = blocks;
      }
      return nvls ? Algo::NVLS : Algo::TWO_SHOT;
    }
  }

  // Staged. A tensor of at most one part (a quarter) of the channel's slice: ONE kernel copies
  // the input into the staging area (ArRank::src), reduces there and writes the result to `out`.
  const size_t part = staging_slice_bytes() / kStageBuffers;
  const size_t part_elems = (part / 16) * (16 / es);
  if (count <= part_elems) {
    Algo algo = pick(bytes, false, seg0_->mc != nullptr);
    fill_ar_rank(&a.r[0], channel, seg0_, staging_offset(channel));
    a.r[0].src = (const char*)in;
    a.r[0].out = out;
    a.algo = (int)algo;
    a.count = count;
    cfg.blocks = choose_blocks(bytes, world_, a.algo, false, sm_count_, cfg_.max_blocks);
    // The copy phases of this kernel want many blocks, its NVLS phase few: a mixed grid, in which
    // all blocks copy and the first few alone drive the switch (64 MiB on 4 GPUs with one grid for
    // all phases: 445 GB/s with 64 blocks, 290 with 16, 456 with 128).
    if (algo == Algo::NVLS && cfg_.max_blocks <= 0) {
      const int p1 = cfg.blocks;
      cfg.blocks = choose_blocks(bytes, world_, (int)Algo::TWO_SHOT, false, sm_count_, 0);
      if (cfg.blocks > p1) {
        a.phase1_blocks = p1;
        a.r[0].ctx.local_base = claim_local_barrier(channel, cfg.blocks, p1);
      }
    }
    CUDA_RT(launch_allreduce(a, dtype, dtype, cfg, s));
    last_blocks = cfg.blocks;
    last_launches = 1;
    return algo;
  }
  // Chunks of the pipeline below: equal shares of at most one part, in multiples of 256 bytes,
  // and at least four of them (with two, nothing is copied while something else is reduced).
  const size_t nchunks = std::max<size_t>(4, (count + part_elems - 1) / part_elems);
  const size_t chunk_elems = align_up((count + nchunks - 1) / nchunks, 256 / es);
  // A larger tensor goes in chunks of one part through a pipeline on three streams: the
  // reductions (NVLink-bound) alternate between the channel's stream and its second lane, so
  // that two are in flight and the fixed costs of one (barriers, ramp-up, drain: about 35 us)
  // hide behind the data phase of the other; the copies in and out (local, HBM-bound) run on a
  // third stream of low priority beside them. (Each chunk costs the host about ten CUDA calls,
  // so chunks far below the size of a part would make the pipeline launch-bound: 8 MiB chunks
  // measured slower than the single fused kernel.) Chunk k lives in part k % 4 of the slice. The NVLS
  // reductions run on 16 blocks each (choose_blocks), which also leaves the SMs to the copies:
  // with 64 blocks per lane 1 GiB took 2.80 ms on 4 GPUs, with 16 it takes 2.41 (in place: 2.37).
  //   copies : in(0) in(1) in(2) out(0) in(3) out(1) in(4) out(2) ...    (out(k) waits for red(k))
  //   lane 0 :   red(0)      red(2)      red(4) ...                      (red(k) waits for in(k))
  //   lane 1 :      red(1)      red(3)      red(5) ...
  // in(k + 4) follows out(k) in stream order, and a reduction ends only after all peers have
  // finished reading this rank's part (last barrier), so a part is never overwritten early.
  // Measured on 4 GPUs, 1 GiB: one fused kernel per chunk on two lanes 3.16 ms (the lanes fall
  // into step: both copy, then both reduce), copies on a stream of their own beside ONE lane of
  // reductions 3.31 ms (the copies hide, but 64 MiB launches run at 544 GB/s where 512 MiB ones
  // reach 673), in place on symmetric memory 2.39 ms.
  // Two ranks reduce one-shot straight into `out`, which needs no copy-out; all others reduce in
  // place on their part of the staging area.
  cudaStream_t lane[2] = {s, streams_[channel + kUserChannels]};
  cudaStream_t cpy = streams_[channel + 2 * kUserChannels];
  const Algo first_algo = pick(std::min(chunk_elems, count) * es, false, seg0_->mc != nullptr);
  const bool to_out = first_algo == Algo::ONE_SHOT;
  CUDA_RT(cudaEventRecord(fork_[channel], s));
  CUDA_RT(cudaStreamWaitEvent(lane[1], fork_[channel], 0));
  CUDA_RT(cudaStreamWaitEvent(cpy, fork_[channel], 0));
  Algo used = Algo::TWO_SHOT;
  struct Chunk { size_t done, n; };
  std::vector<Chunk> chunks;
  for (size_t done = 0; done < count; done += chunk_elems) chunks.push_back({done, std::min(chunk_elems, count - done)});
  auto part_of = [&](size_t k) { return seg0_->local + staging_offset(channel) + (k % kStageBuffers) * part; };
  auto copy_out = [&](size_t k) {
    const Chunk& c = chunks[k];
    CUDA_RT(cudaStreamWaitEvent(cpy, red_done_[channel][k % kStageBuffers], 0));
    if (!to_out) CUDA_RT(launch_copy((char*)out + c.done * es, part_of(k), c.n * es, cpy));
  };
  for (size_t k = 0; k < chunks.size(); k++) {
    const Chunk& c = chunks[k];
    const int b = (int)(k % kStageBuffers), l = (int)(k & 1);
    const size_t nb = c.n * es;
    // one-shot has no copy-out to order in(k) behind: the part is free once red(k - 4) has ended
    if (to_out && k >= (size_t)kStageBuffers) CUDA_RT(cudaStreamWaitEvent(cpy, red_done_[channel][b], 0));
    CUDA_RT(launch_copy(part_of(k), (const char*)in + c.done * es, nb, cpy));
    CUDA_RT(cudaEventRecord(in_done_[channel][b], cpy));
    if (k >= 2 && !to_out) copy_out(k - 2);
    CUDA_RT(cudaStreamWaitEvent(lane[l], in_done_[channel][b], 0));
    Algo algo = to_out ? Algo::ONE_SHOT : pick(nb, true, seg0_->mc != nullptr);
    fill_ar_rank(&a.r[0], channel + l * kUserChannels, seg0_, (size_t)(part_of(k) - seg0_->local));
    a.r[0].out = to_out ? (void*)((char*)out + c.done * es) : (void*)part_of(k);
    a.algo = (int)algo;
    a.count = c.n;
    cfg.blocks = choose_blocks(nb, world_, a.algo, false, sm_count_, cfg_.max_blocks);
    // two reductions side by side: kernels whose blocks do the loads and stores themselves share the SMs
    if (a.algo != (int)Algo::NVLS && cfg.blocks > 74 && cfg_.max_blocks <= 0) cfg.blocks = 74;
    CUDA_RT(launch_allreduce(a, dtype, dtype, cfg, lane[l]));
    CUDA_RT(cudaEventRecord(red_done_[channel][b], lane[l]));
    last_blocks = cfg.blocks;
    last_launches++;
    if (k == 0) used = algo;
  }
  if (!to_out) {
    if (chunks.size() >= 2) copy_out(chunks.size() - 2);
    copy_out(chunks.size() - 1);
  }
  CUDA_RT(cudaEventRecord(join_[channel][0], cpy));
  CUDA_RT(cudaEventRecord(join_[channel][1], lane[1]));
  CUDA_RT(cudaStreamWaitEvent(s, join_[channel][0], 0));
  CUDA_RT(cudaStreamWaitEvent(s, join_[channel][1], 0));
  return used;
}

void Comm::allgatherv(int channel, const void* in, size_t bytes, void* out_symm, void* out_private, size_t total_bytes,
                      unsigned long long* sizes_out, const unsigned long long* all_bytes) {
  CUDA_RT(cudaSetDevice(device_));
  BC_CHECK(channel >= 0 && channel < kUserChannels, "bad channel");
  cudaStream_t s = streams_[channel];
  if (total_bytes == 0) return;
  const size_t slice = staging_slice_bytes(), slice_off = staging_offset(channel);
  AgArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = 1;
  AgRank& r = a.r[0];
  r.ctx = make_ctx(channel);
  r.sizes_out = sizes_out;
  for (int p = 0; p < world_; p++) r.base[p] = seg0_->peer[p];
  r.capacity = seg0_->size;
  // With two ranks the multicast store saves nothing (one peer either way).
  r.mc_base = (cfg_.use_nvls && seg0_->mc && world_ >= 3) ? seg0_->mc : nullptr;
  LaunchCfg cfg;
  auto launch = [&](const void* src, size_t n, size_t off, size_t grid_bytes) {
    r.in = (const char*)src;
    r.bytes = n;
    r.out_off = off;
    // The grid must be the same on every rank, so it is derived from the total, not from this
    // rank's slab.
    size_t want = (grid_bytes / world_ + (32u << 10) - 1) / (32u << 10);
    const size_t cap = cfg_.max_blocks > 0 ? std::min<size_t>(cfg_.max_blocks, kMetaBlocks) : 48;
    cfg.blocks = (int)std::min<size_t>(std::max<size_t>(want, 1), cap);
    CUDA_RT(launch_allgatherv(a, cfg, s));
    last_blocks = cfg.blocks;
  };
  if (out_symm) {
    BC_CHECK((char*)out_symm >= seg0_->local && (char*)out_symm + total_bytes <= seg0_->local + seg0_->size,
             "allgatherv: symmetric output lies outside segment 0");
    launch(in, bytes, (char*)out_symm - seg0_->local, total_bytes);
    return;
  }
  if (total_bytes <= slice) {
    launch(in, bytes, slice_off, total_bytes);
    if (out_private) CUDA_RT(launch_copy(out_private, staging(channel), total_bytes, s));
    return;
  }
  // The result is larger than the staging area and lies in private memory: gather it in rounds.
  // In round j every rank contributes piece j of its slab; the pieces land back to back in the
  // channel's slice of the staging area and are copied from there to their places in the result. Every rank derives the
  // same piece sizes from the slab sizes agreed during negotiation.
  BC_CHECK(all_bytes && out_private, "allgatherv: a result of " << total_bytes << " bytes fits neither the symmetric heap nor the "
           "staging area and the slab sizes are not known on the host; raise BC_HEAP_MB or BC_STAGING_MB");
  std::vector<size_t> piece;
  const size_t rounds = plan_gather_rounds(all_bytes, world_, slice, &piece);
  std::vector<size_t> disp(world_);
  size_t acc = 0;
  for (int p = 0; p < world_; p++) {
    disp[p] = acc;
    acc += (size_t)all_bytes[p];
  }
  for (size_t j = 0; j < rounds; j++) {
    size_t round_total = 0;
    std::vector<size_t> len(world_);
    for (int p = 0; p < world_; p++) {
      const size_t done = std::min<size_t>(j * piece[p], (size_t)all_bytes[p]);
      len[p] = std::min<size_t>(piece[p], (size_t)all_bytes[p] - done);
      round_total += len[p];
    }
    if (round_total == 0) break;
    launch((const char*)in + std::min<size_t>(j * piece[rank_], bytes), len[rank_], slice_off, round_total);
    size_t src_off = 0;
    for (int p = 0; p < world_; p++) {
      if (len[p]) CUDA_RT(launch_copy((char*)out_private + disp[p] + j * piece[p], staging(channel) + src_off, len[p], s));
      src_off += len[p];
    }
  }
}

Algo Comm::fused_step(int channel, void* grad, size_t count, DType dtype, void* param, float* master, float* s1, float* s2,
                      const OptHyper& h, float scale, cudaStream_t stream_override, bool beside_compute) {
  CUDA_RT(cudaSetDevice(device_));
  cudaStream_t s = stream_override ? stream_override : streams_[channel];
  const size_t bytes = count * dtype_size(dtype);
  if (count == 0) return Algo::TWO_SHOT;
  ArArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = 1;
  a.scale = scale;
  a.idiv = 1;
  a.count = count;
  a.opt = h;
  a.prof = prof_;
  Algo algo = Algo::TWO_SHOT;
  if (world_ == 1) {
    a.r[0].ctx = make_ctx(channel);
    a.r[0].in[0] = (char*)grad;
  } else {
    Segment* seg = alloc_->find(grad, bytes);
    BC_CHECK(seg, "fused_step: the gradient bucket must live in symmetric memory");
    fill_ar_rank(&a.r[0], channel, seg, (char*)grad - seg->local);
    algo = choose_algo(bytes, dtype, true, seg->mc != nullptr);
  }
  a.algo = (int)algo;
  a.r[0].out = grad;
  a.r[0].param = param;
  a.r[0].master = master;
  a.r[0].state1 = s1;
  a.r[0].state2 = s2;
  LaunchCfg cfg;
  cfg.blocks = choose_blocks(bytes, world_, a.algo, true, sm_count_, beside_compute && cfg_.overlap_blocks > 0 ? cfg_.overlap_blocks : cfg_.max_blocks,
                             beside_compute);
  if (algo == Algo::NVLS && !beside_compute && cfg_.max_blocks <= 0) {
    // Nothing else is expected on the GPU: the update phase gets one block per SM (all of them
    // can be resident whatever else still drains), the switch phase the few blocks that suit it.
    const int p1 = choose_blocks(bytes, world_, a.algo, false, sm_count_, 0);
    if (cfg.blocks > sm_count_) cfg.blocks = sm_count_;
    if (cfg.blocks > p1) {
      a.phase1_blocks = p1;
      a.r[0].ctx.local_base = claim_local_barrier(channel, cfg.blocks, p1);
    }
  }
  CUDA_RT(launch_allreduce(a, dtype, dtype, cfg, s));
  last_blocks = cfg.blocks;
  return algo;
}

// ---------------------------------------------------------------------------------------------

EmuGroup::EmuGroup(int device, int nranks, size_t bytes_per_rank) : device_(device), n_(nranks), bytes_(align_up(bytes_per_rank, 256)) {
  BC_CHECK(nranks >= 1 && nranks <= kMaxRanks, "emulated group size must be 1.." << kMaxRanks);
  CUDA_RT(cudaSetDevice(device));
  bufs_.assign(n_, nullptr);
  pads_.assign(n_, nullptr);
  for (int r = 0; r < n_; r++) {
    char* raw = nullptr;
    CUDA_RT(cudaMalloc(&raw, bytes_ + 2 * kGuardBytes));
    CUDA_RT(cudaMemset(raw, kGuardPattern, bytes_ + 2 * kGuardBytes));
    bufs_[r] = raw + kGuardBytes;
    CUDA_RT(cudaMalloc(&raw, kPadBytes + 2 * kGuardBytes));
    CUDA_RT(cudaMemset(raw, kGuardPattern, kPadBytes + 2 * kGuardBytes));
    pads_[r] = raw + kGuardBytes;
    CUDA_RT(cudaMemset(pads_[r], 0, kPadBytes));
  }
  CUDA_RT(cudaMalloc(&epochs_, sizeof(uint32_t) * (n_ * kChannels * kMaxBlocks + n_)));
  CUDA_RT(cudaMemset(epochs_, 0, sizeof(uint32_t) * (n_ * kChannels * kMaxBlocks + n_)));
  CUDA_RT(cudaMalloc(&pipe_local_, sizeof(uint32_t) * n_ * 2 * kPipeMaxChunks));
  CUDA_RT(cudaHostAlloc(&status_host_, 64, cudaHostAllocMapped));
  memset(status_host_, 0, 64);
  CUDA_RT(cudaHostGetDevicePointer((void**)&status_dev_, status_host_, 0));
  CUDA_RT(cudaDeviceSynchronize());
}

EmuGroup::~EmuGroup() {
  cudaSetDevice(device_);
  cudaDeviceSynchronize();
  for (char* p : bufs_) if (p) cudaFree(p - kGuardBytes);
  for (char* p : pads_) if (p) cudaFree(p - kGuardBytes);
  if (epochs_) cudaFree(epochs_);
  if (pipe_local_) cudaFree(pipe_local_);
  if (status_host_) cudaFreeHost(status_host_);
}

size_t EmuGroup::damaged_guard_bytes() {
  CUDA_RT(cudaSetDevice(device_));
  CUDA_RT(cudaDeviceSynchronize());
  std::vector<unsigned char> host(kGuardBytes);
  size_t bad = 0;
  auto check = [&](const char* dev) {
    CUDA_RT(cudaMemcpy(host.data(), dev, kGuardBytes, cudaMemcpyDeviceToHost));
    for (unsigned char c : host) bad += c != (unsigned char)kGuardPattern;
  };
  for (int r = 0; r < n_; r++) {
    check(bufs_[r] - kGuardBytes);
    check(bufs_[r] + bytes_);
    check(pads_[r] - kGuardBytes);
    check(pads_[r] + kPadBytes);
  }
  return bad;
}

RankCtx EmuGroup::ctx(int r, int channel) const {
  RankCtx c;
  memset(&c, 0, sizeof(c));
  c.rank = r;
  c.world = n_;
  for (int p = 0; p < n_; p++) {
    char* pad = pads_[p] + (size_t)channel * kChannelBytes;
    c.flags[p] = (uint32_t*)pad;
    c.meta[p] = (uint64_t*)(pad + kFlagBytes);
  }
  c.epochs = epochs_ + ((size_t)r * kChannels + channel) * kMaxBlocks;
  c.local_ctr = epochs_ + (size_t)n_ * kChannels * kMaxBlocks + r;
  c.local_base = local_arrivals_;
  c.status = status_dev_;
  c.timeout_ns = to_ns(timeout_s_);
  return c;
}

cudaError_t EmuGroup::allreduce(size_t off, void* const* outs, size_t count, DType dtype, Algo algo, float scale, int idiv,
                                int blocks, cudaStream_t s, ReduceOp red, const void* const* srcs, const unsigned long long* places,
                                unsigned long long* prof, int phase1_blocks) {
  ArArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = n_;
  a.algo = (int)algo;
  a.count = count;
  a.scale = scale;
  a.idiv = idiv;
  a.red = (int)red;
  a.prof = prof;
  for (int r = 0; r < n_; r++) {
    a.r[r].ctx = ctx(r, 0);
    for (int p = 0; p < n_; p++) a.r[r].in[p] = bufs_[p] + off;
    a.r[r].out = outs[r];
    a.r[r].src = srcs ? (const char*)srcs[r] : nullptr;
    a.r[r].place = places ? places[r] : 0;
  }
  LaunchCfg cfg;
  cfg.cooperative = true;
  cfg.blocks = std::min(blocks > 0 ? blocks : 4, max_emulated_blocks(device_, n_, cfg.threads));
  if (phase1_blocks > 0 && phase1_blocks < cfg.blocks && algo != Algo::ONE_SHOT) {
    a.phase1_blocks = phase1_blocks;
    local_arrivals_ += (uint32_t)(cfg.blocks + phase1_blocks);     // every rank's counter advances alike
  }
  return launch_allreduce(a, dtype, dtype, cfg, s);
}

cudaError_t EmuGroup::fused_step(size_t off, size_t count, DType dtype, void* const* params, float* const* masters,
                                 float* const* s1, float* const* s2, const OptHyper& h, float scale, int blocks, cudaStream_t s,
                                 int phase1_blocks) {
  ArArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = n_;
  a.algo = (int)Algo::TWO_SHOT;
  a.count = count;
  a.scale = scale;
  a.idiv = 1;
  a.opt = h;
  for (int r = 0; r < n_; r++) {
    a.r[r].ctx = ctx(r, 0);
    for (int p = 0; p < n_; p++) a.r[r].in[p] = bufs_[p] + off;
    a.r[r].out = bufs_[r] + off;
    a.r[r].param = params[r];
    a.r[r].master = masters ? masters[r] : nullptr;
    a.r[r].state1 = s1 ? s1[r] : nullptr;
    a.r[r].state2 = s2 ? s2[r] : nullptr;
  }
  LaunchCfg cfg;
  cfg.cooperative = true;
  cfg.blocks = std::min(blocks > 0 ? blocks : 4, max_emulated_blocks(device_, n_, cfg.threads));
  if (phase1_blocks > 0 && phase1_blocks < cfg.blocks) {
    a.phase1_blocks = phase1_blocks;
    local_arrivals_ += (uint32_t)(cfg.blocks + phase1_blocks);
  }
  return launch_allreduce(a, dtype, dtype, cfg, s);
}

cudaError_t EmuGroup::allgatherv(const void* const* ins, const unsigned long long* bytes, const unsigned long long* out_offs,
                                 int blocks, cudaStream_t s) {
  AgArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = n_;
  for (int r = 0; r < n_; r++) {
    a.r[r].ctx = ctx(r, 1);
    a.r[r].in = (const char*)ins[r];
    a.r[r].bytes = bytes[r];
    a.r[r].out_off = out_offs[r];
    a.r[r].capacity = bytes_;
    for (int p = 0; p < n_; p++) a.r[r].base[p] = bufs_[p];
  }
  LaunchCfg cfg;
  cfg.cooperative = true;
  cfg.blocks = std::min(std::min(blocks > 0 ? blocks : 2, (int)kMetaBlocks), max_emulated_blocks(device_, n_, cfg.threads));
  return launch_allgatherv(a, cfg, s);
}

cudaError_t EmuGroup::staged_pipeline(size_t off, const void* const* srcs, void* const* outs, size_t count, DType dtype,
                                      float scale, int idiv, size_t chunk_bytes, int slots, int lag, int reducers, int copiers,
                                      int rgroups, int cgroups, bool streaming, cudaStream_t s) {
  const size_t bytes = count * dtype_size(dtype);
  if (bytes == 0 || bytes % 16 || chunk_bytes == 0 || chunk_bytes % 16 || slots < 1 || reducers < 1 || copiers < 1)
    return cudaErrorInvalidValue;
  if (off + (size_t)slots * chunk_bytes > bytes_) return cudaErrorInvalidValue;
  PipeArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = n_;
  a.npacks = bytes / 16;
  a.chunk_packs = chunk_bytes / 16;
  const size_t nchunks = (a.npacks + a.chunk_packs - 1) / a.chunk_packs;
  if (nchunks > (size_t)kPipeMaxChunks) return cudaErrorInvalidValue;
  a.nchunks = (int)nchunks;
  a.slots = std::min(slots, a.nchunks);
  a.lag = lag;
  a.reducers = reducers;
  a.rgroups = rgroups;
  a.cgroups = cgroups;
  a.streaming = streaming ? 1 : 0;
  a.base = pipe_base_;
  a.scale = scale;
  a.idiv = idiv;
  for (int r = 0; r < n_; r++) {
    PipeRank& R = a.r[r];
    R.ctx = ctx(r, 3);
    for (int p = 0; p < n_; p++) {
      R.stage[p] = bufs_[p] + off;
      R.progress[p] = (uint32_t*)(pads_[p] + 3 * kChannelBytes + kFlagBytes + kMetaBytes);
    }
    R.src = (const char*)srcs[r];
    R.out = (char*)outs[r];
    R.local = pipe_local_ + (size_t)r * 2 * kPipeMaxChunks;
  }
  cudaError_t e = cudaMemsetAsync(pipe_local_, 0, sizeof(uint32_t) * n_ * 2 * kPipeMaxChunks, s);
  if (e != cudaSuccess) return e;
  LaunchCfg cfg;
  cfg.cooperative = true;
  cfg.blocks = reducers + copiers;
  if (cfg.blocks > max_emulated_blocks(device_, n_, cfg.threads)) return cudaErrorInvalidConfiguration;
  e = launch_staged_pipeline(a, dtype, false, cfg, s);
  if (e == cudaSuccess) pipe_base_ += (uint32_t)a.nchunks;
  return e;
}

cudaError_t EmuGroup::barrier_probe(int absent, double timeout_s, cudaStream_t s) {
  std::vector<RankCtx> c(n_);
  for (int r = 0; r < n_; r++) {
    c[r] = ctx(r, 2);
    c[r].timeout_ns = to_ns(timeout_s);
  }
  return launch_barrier_probe(c.data(), n_, absent, s);
}

}  // namespace gpu
}  // namespace bc
