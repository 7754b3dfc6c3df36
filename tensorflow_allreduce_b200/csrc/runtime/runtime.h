// Process-wide runtime: global state, the background coordinator thread, the tensor table and
// the dispatch of negotiated collectives to the CPU ring or the GPU kernels.
//
// Same responsibilities as MPIGlobalState / BackgroundThreadLoop / EnqueueTensorCollective /
// PerformCollectiveOp in the reference (tensorflow/contrib/mpi_collectives/mpi_ops.cc:170-244,
// 435-515, 572-868), with these differences by design:
//   * the thread sleeps in poll() on its sockets and an eventfd and wakes on demand; there is no
//     1 ms tick;
//   * every wait has a deadline and a lost peer fails all pending operations on every rank;
//   * a GPU collective is enqueued on a private stream behind an event recorded by the producer,
//     and completion is an event the consumer's stream waits on: the host never synchronises
//     with the device on this path;
//   * names that are still in flight are rejected instead of being dropped silently.
#pragma once

#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "../common.h"
#include "../control/bootstrap.h"
#include "../control/node_group.h"
#include "../control/wire.h"
#include "../cpu/shm_group.h"

namespace bc {

namespace gpu { class Comm; }

// Called on the background thread when an allgather's total first dimension is known; returns
// the output buffer (and, for GPU tensors, whether it lies in the symmetric heap).
typedef void* (*AllocFn)(int64_t handle, int64_t total_rows, void* user, int* is_symmetric);

struct OpRecord {
  int64_t id = 0;
  std::string name;
  OpType op = OpType::ALLREDUCE;
  DType dtype = DType::F32;
  DeviceKind device = DeviceKind::CPU;
  std::vector<int64_t> shape;
  const void* in = nullptr;
  void* out = nullptr;
  bool average = false;
  ReduceOp red = ReduceOp::SUM;
  bool zero_copy = false;        // GPU: input and output are the same symmetric tensor on every rank
  void* ready_event = nullptr;   // cudaEvent_t recorded by the producer stream, or null
  void* done_event = nullptr;    // cudaEvent_t recorded on the private stream after the launch
  AllocFn alloc = nullptr;
  void* alloc_user = nullptr;
  std::string blob;
  // results
  std::vector<int64_t> dim0;
  std::vector<std::string> blobs;
  int algo = 0;
  enum State { PENDING, DONE, FAILED } state = PENDING;
  std::string error;
  double t_enqueue = 0, t_negotiated = 0, t_done = 0;
  double two_level_s[3] = {0, 0, 0};   // allreduce in two levels: inside the host, over the rail, back inside the host
  void* timed_start = nullptr;         // timing events around the kernels of a GPU collective while device timing is on
  void* timed_stop = nullptr;
};

struct RuntimeOptions {
  int rank = 0, size = 1;
  int local_rank_override = -1;
  std::string addr = "127.0.0.1";
  int port = 29500;
  int device = -1;                // CUDA device ordinal, -1 = CPU only
  double timeout_s = 300.0;       // host-side deadline for negotiation and ring steps
  double device_timeout_s = 30.0;
  size_t staging_bytes = 1024u << 20;
  size_t heap_bytes = 256u << 20;
  int force_algo = 0;
  size_t one_shot_max_bytes = 256u << 10;
  size_t nvls_min_bytes = 512u << 10;
  bool use_nvls = true;
  int max_blocks = 0;
  int symm_mode = 0;              // 0 auto, 1 vmm, 2 ipc
  std::string fault;              // fault-injection spec (host side only)
  std::string hostname;           // host name to report (empty: BC_HOSTNAME, else the machine's)
};

struct FaultSpec {
  enum Kind { NONE, DROP_REQUEST, DELAY_MS, EXIT_BEFORE, CLOSE_CTRL, EXIT_IN_COLLECTIVE } kind = NONE;
  int rank = -1;           // -1 = any rank
  std::string name;        // empty = any name
  int ms = 0;
  static FaultSpec parse(const std::string& s);
  bool matches(int r, const std::string& n) const {
    return kind != NONE && (rank < 0 || rank == r) && (name.empty() || name == n);
  }
};

struct StatEntry {
  std::string name;
  int op = 0, algo = 0, device = 0, blocks = 0;
  int64_t bytes = 0;
  double t_enqueue = 0, t_negotiated = 0, t_done = 0;
  double two_level_s[3] = {0, 0, 0};
  double device_us = -1;    // time of the kernels on the device (CUDA events), where it was sampled
  int channel = -1;         // private stream of an ordered launch
};

// An ordered launch whose device time is being measured: two timing events around it on its
// stream. The record joins the statistics once the stop event has completed.
struct TimedLaunch {
  StatEntry entry;
  void* start = nullptr;    // cudaEvent_t
  void* stop = nullptr;
};

class Runtime {
 public:
  explicit Runtime(const RuntimeOptions& o);
  ~Runtime();

  int rank() const { return t_.rank; }
  int size() const { return t_.size; }
  int local_rank() const { return local_rank_; }
  int local_size() const { return t_.local_size; }
  bool on_gpu() const { return comm_ != nullptr; }
  gpu::Comm* comm() const { return comm_.get(); }
  // Hosts of a GPU group that spans several of them (then `comm()` covers the ranks of this host
  // only and collectives run in two levels); 1 otherwise.
  int n_nodes() const { return node_ ? node_->n_nodes : 1; }
  NodeGroup* node_group() const { return node_.get(); }
  const RuntimeOptions& options() const { return opt_; }

  // Queue a collective; returns its handle. Throws if the name is already in flight or the
  // communicator is broken.
  int64_t enqueue(std::unique_ptr<OpRecord> rec);
  // Block until the operation has been performed (CPU) or launched (GPU). Throws on failure.
  void wait(int64_t handle, double timeout_s);
  bool poll(int64_t handle);
  std::shared_ptr<OpRecord> get(int64_t handle);
  void release(int64_t handle);

  // Convenience: host allgather of small blobs through the negotiated path.
  std::vector<std::string> blob_gather(const std::string& name, const std::string& mine);

  void shutdown();
  bool broken() const { return broken_.load(); }
  std::string broken_reason();
  void set_fault(const std::string& spec);

  std::string stats_json();
  void clear_stats();

  // Device timing of ordered launches (gradient buckets): while switched on, the entry points
  // bracket every launch with two timing events (`timed_begin` before, `timed_end` after).
  void set_device_timing(bool on) { device_timing_.store(on); }
  bool device_timing() const { return device_timing_.load(); }
  TimedLaunch timed_begin(void* stream);
  void timed_end(TimedLaunch t, void* stream, const char* name, int algo, int blocks, int64_t bytes, int channel);

 private:
  void setup_node_group();      // constructor steps, collective over all ranks
  void setup_shared_memory();
  void loop();
  void loop_body();
  void drain_local_queue();
  void coordinator_handle(const Request& req);
  void coordinator_check_deadlines();
  void send_request(const OpRecord& rec);
  void perform(const Response& resp);
  void perform_allreduce(OpRecord& r);
  void perform_allgather(OpRecord& r, const Response& resp);
  void two_level_allreduce(OpRecord& r, size_t count, double scale, int64_t idiv);
  void two_level_allgather(OpRecord& r, size_t row_bytes, size_t total_bytes);
  void* pinned(size_t bytes);
  void* device_scratch(size_t bytes);
  void finish(const std::shared_ptr<OpRecord>& r, bool ok, const std::string& err);
  void fail_everything(const std::string& why);
  void wake();

  RuntimeOptions opt_;
  Transport t_;
  int local_rank_ = 0;
  std::unique_ptr<gpu::Comm> comm_;
  std::unique_ptr<NodeGroup> node_;   // set when the ranks span several hosts (see build_node_group)
  std::unique_ptr<ShmGroup> shm_;     // CPU tensors among the ranks of this host: the whole job, or with node_ this
                                      // host's level of a two-level allreduce (BC_SHM=0: sockets only)
  std::vector<char> cpu_staging_;     // this rank's slice on its way over the rail (background thread only)
  void* pinned_ = nullptr;            // host staging of the two-level path (background thread only)
  size_t pinned_bytes_ = 0;
  void* scratch_ = nullptr;           // device staging of the two-level path
  size_t scratch_bytes_ = 0;

  std::thread thread_;
  double spin_s_ = 100e-6;            // how long the thread keeps polling after an event before it sleeps (BC_SPIN_US)
  size_t two_level_chunk_bytes_ = 2u << 20;   // CPU tensors over several hosts: chunk of the pipelined allreduce, used from
                                              // four chunks on (BC_TWO_LEVEL_CHUNK_KB; 0 = one piece, nothing overlaps)
  double last_event_s_ = 0;
  int wake_fd_ = -1;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<std::shared_ptr<OpRecord>> queue_;                       // enqueued, not yet seen by the thread
  std::unordered_map<std::string, std::shared_ptr<OpRecord>> table_;  // in flight, by name
  std::unordered_map<int64_t, std::shared_ptr<OpRecord>> handles_;
  int64_t next_id_ = 1;
  std::atomic<bool> broken_{false};
  std::atomic<bool> stop_{false};
  bool shutdown_done_ = false;
  std::string broken_reason_;
  FaultSpec fault_;

  // coordinator (rank 0 only)
  struct Pending {
    std::vector<Request> reqs;
    std::vector<bool> have;
    int count = 0;
    double first_seen = 0;
  };
  std::unordered_map<std::string, Pending> pending_;

  std::mutex stats_mu_;
  std::deque<StatEntry> stats_;
  std::atomic<bool> device_timing_{false};
  std::deque<TimedLaunch> timed_;          // launched, stop event not yet seen complete
  std::vector<void*> event_pool_;          // timing events ready for reuse
  void collect_timed_locked();             // moves completed launches into stats_ (stats_mu_ held)
};

}  // namespace bc
