// GPU communicator of one rank: symmetric segments, signal pads, private streams, the
// algorithm selector, and the launch paths used by the runtime (negotiated collectives), by the
// gradient-bucket fast path (ordered launches without negotiation) and by single-GPU emulation.
//
// Reference counterpart: the private CUDA stream plus RingAllreduce<GPU>/RingAllgather<GPU>
// dispatch of the background thread (tensorflow/contrib/mpi_collectives/mpi_ops.cc:213-230,
// 435-515, 873).
#pragma once

#include <atomic>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "collectives.h"
#include "symm.h"

namespace bc {
namespace gpu {

struct CommConfig {
  size_t staging_bytes = 1024u << 20;   // staging area for tensors outside symmetric memory, cut into one slice per user channel
  size_t heap_bytes = 256u << 20;       // general symmetric heap inside segment 0 (allgather outputs, user tensors)
  double device_timeout_s = 30.0;       // bound of every device-side wait
  int force_algo = 0;                   // Algo, 0 = pick from the table
  size_t one_shot_max_bytes = 256u << 10;
  size_t nvls_min_bytes = 512u << 10;
  bool use_nvls = true;
  int max_blocks = 0;                   // 0 = heuristic
  int overlap_blocks = 0;               // grid cap of launches that run beside the backward pass (0 = one per SM that a
                                        // 128-SM persistent kernel leaves free, at least 8)
  // Tensors outside symmetric memory in one launch whose blocks have roles (staged_pipeline.cu):
  // 0 = off, 1 = where the switch reduces (NVLS), 2 = also with peer loads and stores.
  int staged_pipeline = 1;
  size_t pipeline_min_bytes = 96u << 20;
  size_t pipeline_chunk_bytes = 8u << 20;   // upper bound of a chunk (see plan_pipeline)
  int pipeline_slots = 16;                  // chunks that the staging ring holds
  int pipeline_copiers = 0;                 // blocks that copy in and out; 0 = what half of the SMs leaves beside the reducers
  int pipeline_reducers = 0;                // blocks that reduce; 0 = 16 where the switch reduces, else 32 (draining: 32 / 48)
  int pipeline_rgroups = 8;                 // groups of reducer blocks (one chunk each at a time); streaming: 1
  bool pipeline_streaming = true;           // reducer blocks that never drain between chunks (staged_pipeline.cu)
  int pipeline_cgroups = 4;                 // groups of copier blocks
  SymmAllocator::Mode symm_mode = SymmAllocator::Mode::AUTO;
};

// How the staged pipeline kernel cuts a tensor of `bytes` bytes whose staging slice has
// `slice_bytes`: a pure function, the same on every rank.
struct PipePlan {
  size_t chunk_bytes;
  int nchunks, slots, lag;   // slots and lag are multiples of the number of copier groups when the ring wraps;
                             // nchunks == 0: the slice cannot hold the ring
};
// `unit_bytes` (0 = 4 KiB): chunks are multiples of it.
PipePlan plan_pipeline(const CommConfig& cfg, size_t bytes, size_t slice_bytes, size_t unit_bytes = 0);

// The algorithm for a reduction of `bytes` bytes in a group of `world` ranks: a pure function of
// its arguments, so every rank computes the same answer (and it can be checked without a GPU).
Algo select_algo(const CommConfig& cfg, int world, size_t bytes, DType dtype, bool in_place_or_fused, bool has_mc);

// A gathered result that is larger than the staging area goes through it in rounds: in round j
// rank p contributes bytes [j * piece[p], (j + 1) * piece[p]) of its slab. Returns the number of
// rounds; every round's pieces fit the staging area together, and the pieces are multiples of 16.
size_t plan_gather_rounds(const unsigned long long* all_bytes, int world, size_t staging_bytes, std::vector<size_t>* piece);

struct OpTiming {
  cudaEvent_t start = nullptr, stop = nullptr;
};

class Comm {
 public:
  Comm(int rank, int world, int device, uint64_t job_id, const CommConfig& cfg, const HostAllgather& ag, double host_timeout_s);
  ~Comm();

  int rank() const { return rank_; }
  int world() const { return world_; }
  int device() const { return device_; }
  cudaStream_t stream(int channel) const { return streams_[channel]; }
  const CommConfig& config() const { return cfg_; }
  SymmAllocator& allocator() { return *alloc_; }

  // Status word written by kernels whose wait ran out; 0 while healthy.
  uint32_t device_status() const { return status_host_ ? *(volatile uint32_t*)status_host_ : 0; }
  void set_device_timeout(double s) { cfg_.device_timeout_s = s; }
  void set_overlap_blocks(int n) { cfg_.overlap_blocks = n; }
  CommConfig& mutable_config() { return cfg_; }

  // Algorithm for a reduction of `bytes` bytes (all ranks compute the same answer).
  Algo choose_algo(size_t bytes, DType dtype, bool in_place_or_fused, bool has_mc) const;

  // Sum-allreduce of `count` elements, launched on stream(channel). `in` may be anywhere on the
  // device; data outside symmetric memory is staged. `scale`/`idiv` implement averaging.
  // `zero_copy_agreed`: every rank passes the same tensor of symmetric memory (in == out) and
  // has said so; `check_place` then lets the kernel compare the offsets of all ranks (for callers
  // that could not agree beforehand). Returns the algorithm used.
  Algo allreduce(int channel, const void* in, void* out, size_t count, DType dtype, float scale, int idiv,
                 bool zero_copy_agreed, ReduceOp red = ReduceOp::SUM, bool check_place = false);
  // Variable allgather: `in` = this rank's slab, `out_symm` must lie in segment 0's heap or be null
  // (then the staging area is the landing zone and `out_private` receives a copy; a result larger
  // than the staging area is gathered in rounds, for which `all_bytes` = every rank's slab size
  // must be given).
  void allgatherv(int channel, const void* in, size_t bytes, void* out_symm, void* out_private, size_t total_bytes,
                  unsigned long long* sizes_out = nullptr, const unsigned long long* all_bytes = nullptr);

  // Fused reduce + optimizer update on a gradient bucket that lives in symmetric memory.
  // `beside_compute`: the launch shares the GPU with the backward pass; its grid is capped so
  // that all of its blocks can be resident together (see choose_blocks).
  Algo fused_step(int channel, void* grad, size_t count, DType dtype, void* param, float* master, float* s1, float* s2,
                  const OptHyper& h, float scale, cudaStream_t stream_override, bool beside_compute = false);

  // Device array of kProfStamps time stamps that the next reduction launches fill in (null: off).
  void set_profile(unsigned long long* stamps) { prof_ = stamps; }

  // Segment-0 layout: every user channel owns one slice of the staging area, so staged
  // collectives on different channels (different streams) never share bytes.
  size_t staging_slice_bytes() const { return cfg_.staging_bytes / dev::kUserChannels; }
  size_t staging_offset(int channel) const { return staging_off_ + (size_t)(channel % dev::kUserChannels) * staging_slice_bytes(); }
  char* staging(int channel) const { return seg0_->local + staging_offset(channel); }
  size_t staging_bytes() const { return cfg_.staging_bytes; }
  char* heap_base() const { return seg0_->local + heap_off_; }
  size_t heap_bytes() const { return cfg_.heap_bytes; }
  Segment* seg0() const { return seg0_; }
  Segment* new_segment(size_t bytes, const HostAllgather& ag) { return alloc_->alloc(bytes, ag); }

  dev::RankCtx make_ctx(int channel) const;
  int sm_count() const { return sm_count_; }

  // last launch info (for stats)
  int last_blocks = 0;
  int last_launches = 0;   // kernel launches of the last allreduce() call

 private:
  void fill_ar_rank(ArRank* r, int channel, Segment* seg, size_t off) const;

  int rank_, world_, device_;
  CommConfig cfg_;
  std::unique_ptr<SymmAllocator> alloc_;
  Segment* seg0_ = nullptr;
  size_t pad_off_ = 0, staging_off_ = 0, heap_off_ = 0;
  uint32_t* epochs_ = nullptr;        // device-local epoch counters [kChannels][kMaxBlocks], then one arrival counter
                                      // per channel for the barriers among the blocks of a launch (mixed grids)
  mutable uint32_t local_arrivals_[dev::kChannels] = {0};   // what those counters will hold once the queued launches have run
  // Marks the next launch on `channel` as one with a mixed grid of `blocks` blocks of which
  // `phase1_blocks` talk to the peers: returns the counter value it starts from.
  uint32_t claim_local_barrier(int channel, int blocks, int phase1_blocks) const {
    const uint32_t base = local_arrivals_[channel];
    local_arrivals_[channel] += (uint32_t)(blocks + phase1_blocks);
    return base;
  }
  uint32_t* status_host_ = nullptr;   // pinned, mapped
  uint32_t* status_dev_ = nullptr;
  // Staged pipeline kernel: arrival counters per user channel ([2][kPipeMaxChunks], zeroed on the
  // stream before each launch) and the value that the channel's progress words hold once the
  // queued launches have run.
  uint32_t* pipe_local_ = nullptr;
  uint32_t pipe_base_[dev::kUserChannels] = {0};
  // Reduces the first `packs` 16-byte packs of a private tensor with the staged pipeline kernel;
  // false (nothing launched) when the channel's staging slice is too small for its ring.
  bool launch_pipeline(int channel, const char* in, char* out, size_t packs, DType dtype, float scale, int idiv, bool nvls);
  cudaStream_t streams_[dev::kChannels] = {nullptr};
  // Events of the pipeline that carries a large staged tensor (Comm::allreduce).
  static constexpr int kStageBuffers = 4;                      // parts of a channel's staging slice in rotation
  cudaEvent_t fork_[dev::kUserChannels] = {nullptr};           // the helper streams start behind the channel's stream ...
  cudaEvent_t join_[dev::kUserChannels][2] = {{nullptr}};      // ... and the channel's stream continues behind them
  cudaEvent_t in_done_[dev::kUserChannels][kStageBuffers] = {{nullptr}};    // chunk copied into part b of the slice
  cudaEvent_t red_done_[dev::kUserChannels][kStageBuffers] = {{nullptr}};   // chunk in part b reduced
  unsigned long long* prof_ = nullptr;
  int sm_count_ = 148;
};

// ---------------------------------------------------------------------------------------------
// Single-GPU emulation of an N-rank group: all ranks' buffers and pads live on one device and a
// collective is ONE cooperative launch (blockIdx.y = rank). Used to test the multi-rank protocol
// where only one GPU is available.
class EmuGroup {
 public:
  EmuGroup(int device, int nranks, size_t bytes_per_rank);
  ~EmuGroup();
  int nranks() const { return n_; }
  char* buffer(int r) const { return bufs_[r]; }
  size_t bytes_per_rank() const { return bytes_; }
  uint32_t status() const { return *(volatile uint32_t*)status_host_; }
  void clear_status() { *(volatile uint32_t*)status_host_ = 0; }
  // Every buffer and signal pad sits between two guard regions filled with a byte pattern.
  // Returns the number of guard bytes that no longer hold the pattern (0 = nothing wrote out of
  // bounds). Synchronises the device.
  size_t damaged_guard_bytes();

  // In-place-capable allreduce over ranks' buffers at `off`; outs[r] may equal the input.
  // `srcs` (optional): private inputs that the kernel copies into the ranks' buffers first, as the
  // staged path does. `places` (optional): the offsets the ranks claim to have passed (the kernel
  // compares them and sets kStatusLayout on a mismatch).
  // `phase1_blocks` > 0: mixed grid, only that many blocks of every rank run the cross-rank phase.
  cudaError_t allreduce(size_t off, void* const* outs, size_t count, DType dtype, Algo algo, float scale, int idiv,
                        int blocks, cudaStream_t s, ReduceOp red = ReduceOp::SUM, const void* const* srcs = nullptr,
                        const unsigned long long* places = nullptr, unsigned long long* prof = nullptr, int phase1_blocks = 0);
  cudaError_t fused_step(size_t off, size_t count, DType dtype, void* const* params, float* const* masters,
                         float* const* s1, float* const* s2, const OptHyper& h, float scale, int blocks, cudaStream_t s,
                         int phase1_blocks = 0);
  cudaError_t allgatherv(const void* const* ins, const unsigned long long* bytes, const unsigned long long* out_offs,
                         int blocks, cudaStream_t s);
  // The staged pipeline kernel (peer loads and stores) on private tensors srcs[r] -> outs[r] of
  // `count` elements (a multiple of 16 bytes), through rings of `slots` chunks of `chunk_bytes`
  // at `off` of the ranks' buffers; `reducers` + `copiers` blocks per rank.
  cudaError_t staged_pipeline(size_t off, const void* const* srcs, void* const* outs, size_t count, DType dtype, float scale,
                              int idiv, size_t chunk_bytes, int slots, int lag, int reducers, int copiers, int rgroups,
                              int cgroups, bool streaming, cudaStream_t s);
  // A barrier-only launch in which rank `absent` (if >= 0) does not take part, so that the
  // others run into the bounded wait. `timeout_s` bounds it.
  cudaError_t barrier_probe(int absent, double timeout_s, cudaStream_t s);

 private:
  dev::RankCtx ctx(int r, int channel) const;
  int device_, n_;
  size_t bytes_;
  std::vector<char*> bufs_;   // user-visible starts (allocation start + kGuardBytes)
  std::vector<char*> pads_;
  uint32_t* epochs_ = nullptr;  // [n][kChannels][kMaxBlocks], then one arrival counter per rank (mixed grids)
  uint32_t local_arrivals_ = 0; // what each rank's counter will hold once the queued launches have run
  uint32_t* pipe_local_ = nullptr;  // [n][2][kPipeMaxChunks] arrival counters of the staged pipeline kernel
  uint32_t pipe_base_ = 0;          // what the progress words hold once the queued launches have run
  uint32_t* status_host_ = nullptr;
  uint32_t* status_dev_ = nullptr;
  double timeout_s_ = 20.0;
};

cudaError_t launch_barrier_probe(const dev::RankCtx* ctxs, int nranks, int absent, cudaStream_t s);

}  // namespace gpu
}  // namespace bc
