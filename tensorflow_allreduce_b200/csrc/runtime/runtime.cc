#include "runtime.h"

#include <cuda_runtime.h>
#include <poll.h>
#include <stdarg.h>
#include <string.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>

#include "../cpu/ring.h"
#include "../cuda/comm.h"
#include "two_level.h"

namespace bc {

namespace {
inline void cpu_pause() {
#if defined(__x86_64__) || defined(__i386__)
  __builtin_ia32_pause();
#endif
}
}  // namespace

// ---- logging -------------------------------------------------------------------------------

int log_level() {
  static int lvl = [] {
    const char* e = getenv("BC_LOG_LEVEL");
    return e ? atoi(e) : 0;
  }();
  return lvl;
}

void log_line(int level, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  const char* rank = getenv("RANK");
  fprintf(stderr, "[bcoll %s r%s] %s\n", level <= 0 ? "E" : level == 1 ? "I" : "D", rank ? rank : "?", buf);
}

// ---- fault injection (host side only) --------------------------------------------------------

FaultSpec FaultSpec::parse(const std::string& s) {
  FaultSpec f;
  if (s.empty()) return f;
  size_t pos = 0;
  bool first = true;
  while (pos <= s.size()) {
    size_t next = s.find(':', pos);
    std::string tok = s.substr(pos, next == std::string::npos ? std::string::npos : next - pos);
    if (first) {
      first = false;
      std::string kind = tok;
      size_t eq = tok.find('=');
      if (eq != std::string::npos) kind = tok.substr(0, eq);
      if (kind == "drop_request") f.kind = DROP_REQUEST;
      else if (kind == "delay_ms") { f.kind = DELAY_MS; if (eq != std::string::npos) f.ms = atoi(tok.c_str() + eq + 1); }
      else if (kind == "exit_before") f.kind = EXIT_BEFORE;
      else if (kind == "close_ctrl") f.kind = CLOSE_CTRL;
      else if (kind == "exit_in_collective") f.kind = EXIT_IN_COLLECTIVE;
      else throw Error("unknown fault kind '" + kind + "'");
    } else {
      size_t eq = tok.find('=');
      if (eq != std::string::npos) {
        std::string k = tok.substr(0, eq), v = tok.substr(eq + 1);
        if (k == "rank") f.rank = atoi(v.c_str());
        else if (k == "name") f.name = v;
        else if (k == "ms") f.ms = atoi(v.c_str());
      }
    }
    if (next == std::string::npos) break;
    pos = next + 1;
  }
  return f;
}

// ---- construction / teardown ---------------------------------------------------------------

Runtime::Runtime(const RuntimeOptions& o) : opt_(o) {
  t_ = bootstrap(o.rank, o.size, o.addr, o.port, o.timeout_s, o.hostname);
  local_rank_ = o.local_rank_override >= 0 ? o.local_rank_override : t_.local_rank;
  fault_ = FaultSpec::parse(o.fault);
  setup_node_group();
  if (o.device >= 0) {
    gpu::CommConfig cc;
    cc.staging_bytes = o.staging_bytes;
    cc.heap_bytes = o.heap_bytes;
    cc.device_timeout_s = o.device_timeout_s;
    cc.force_algo = o.force_algo;
    cc.one_shot_max_bytes = o.one_shot_max_bytes;
    cc.nvls_min_bytes = o.nvls_min_bytes;
    cc.use_nvls = o.use_nvls;
    cc.max_blocks = o.max_blocks;
    cc.symm_mode = o.symm_mode == 1 ? gpu::SymmAllocator::Mode::VMM
                 : o.symm_mode == 2 ? gpu::SymmAllocator::Mode::IPC : gpu::SymmAllocator::Mode::AUTO;
    const double dl = o.timeout_s;
    if (node_) {
      // The communicator covers the ranks of this host; its set-up talks over the node's star.
      NodeGroup* ng = node_.get();
      gpu::HostAllgather ag = [ng, dl](const std::string& mine) { return ng->allgather(mine, now_s() + dl); };
      const uint64_t node_job = t_.job_id ^ (0x9E3779B97F4A7C15ull * (uint64_t)(node_->node_index + 1));
      comm_.reset(new gpu::Comm(node_->local_rank, node_->local_size, o.device, node_job, cc, ag, o.timeout_s));
    } else {
      Transport* tp = &t_;
      gpu::HostAllgather ag = [tp, dl](const std::string& mine) { return tp->allgather(mine, now_s() + dl); };
      comm_.reset(new gpu::Comm(t_.rank, t_.size, o.device, t_.job_id, cc, ag, o.timeout_s));
    }
  }
  setup_shared_memory();
  // Polling instead of sleeping pays while every thread has a core of its own (a caller and a
  // background thread per rank); on a machine with fewer cores it only takes time from the peers.
  if (const char* us = getenv("BC_SPIN_US")) spin_s_ = std::max(0, atoi(us)) * 1e-6;
  if (const char* kb = getenv("BC_TWO_LEVEL_CHUNK_KB")) two_level_chunk_bytes_ = (size_t)std::max(0, atoi(kb)) << 10;
  else if (std::thread::hardware_concurrency() < 2u * (unsigned)std::max(1, t_.local_size)) spin_s_ = 0;
  wake_fd_ = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  BC_CHECK(wake_fd_ >= 0, "eventfd failed");
  thread_ = std::thread([this] { loop(); });
}

void Runtime::setup_node_group() {
  // Ranks on several hosts: collectives run in two levels (inside a host the NVLink kernels for
  // GPU tensors and shared memory for CPU tensors, rings of sockets between hosts). A GPU job
  // always gets the node groups for that, a CPU job when its hosts run several ranks each;
  // BC_NODE_GROUPS=1 / 0 forces / forbids them for a CPU job.
  const char* groups_env = getenv("BC_NODE_GROUPS");
  const int want_groups = groups_env ? atoi(groups_env) : -1;
  if (t_.local_size != t_.size) {
    std::string why;
    const bool uniform = hosts_are_uniform(t_, &why);
    if (opt_.device >= 0 || want_groups > 0)
      BC_CHECK(uniform, "collectives in two levels need the same number of ranks on every host (" << why << ")");
    if (opt_.device >= 0 || want_groups > 0 || (want_groups != 0 && uniform && t_.local_size > 1))
      node_.reset(new NodeGroup(build_node_group(t_, now_s() + opt_.timeout_s)));
  }
}

void Runtime::setup_shared_memory() {
  // CPU tensors among the ranks of one host go through a shared-memory segment: the whole job when
  // it runs on one host, else the level inside a host of a job with node groups. BC_SHM=0 keeps
  // the sockets, BC_SHM_SLOT_KB sets the chunk per rank.
  const char* shm_env = getenv("BC_SHM");
  const bool one_host = t_.size > 1 && t_.local_size == t_.size;
  const bool host_level = node_ && node_->local_size > 1;
  if ((one_host || host_level) && !(shm_env && atoi(shm_env) == 0)) {
    const char* kb = getenv("BC_SHM_SLOT_KB");
    const size_t slot = (size_t)std::max(4, kb ? atoi(kb) : 512) << 10;
    char name[96];
    snprintf(name, sizeof(name), "bcoll-%016llx-shm-%d", (unsigned long long)t_.job_id, host_level ? node_->node_index : 0);
    Transport* tp = &t_;
    NodeGroup* ng = node_.get();
    const double dl = opt_.timeout_s;
    const int my = host_level ? ng->local_rank : t_.rank, n = host_level ? ng->local_size : t_.size;
    ShmGroup::Allgather ag = [tp, ng, host_level, dl](const std::string& mine) {
      return host_level ? ng->allgather(mine, now_s() + dl) : tp->allgather(mine, now_s() + dl);
    };
    try {
      // A rank waiting in shared memory looks at the ring's sockets now and then: end-of-file on
      // one of them means that the neighbour's process has ended (the kernel closes its sockets
      // even before the process is reaped). Data that is waiting there is left alone.
      auto peer_lost = [tp]() -> std::string {
        const Socket* socks[2] = {&tp->ring_prev, &tp->ring_next};
        for (const Socket* s : socks) {
          char c;
          if (s->valid() && ::recv(s->fd(), &c, 1, MSG_PEEK | MSG_DONTWAIT) == 0)
            return std::string("the process of ring neighbour ") + (s == socks[0] ? "before" : "after") + " this rank has ended";
        }
        return std::string();
      };
      shm_.reset(new ShmGroup(my, n, name, slot, ag, peer_lost));
    } catch (const CommLost&) {
      throw;
    } catch (const Error& e) {
      // Every rank of the host learns of a failed set-up in the same exchange.
      BC_LOG(1, "%s; CPU tensors use the socket ring", e.what());
    }
    if (host_level) {
      // All hosts must take the same path: one host without shared memory puts every host on the ring.
      bool all = true;
      for (const std::string& ok : t_.allgather(shm_ ? "1" : "0", now_s() + dl)) all = all && ok == "1";
      if (!all) shm_.reset();
    }
  }
}

Runtime::~Runtime() {
  try {
    shutdown();
  } catch (...) {
  }
  if (wake_fd_ >= 0) ::close(wake_fd_);
}

void Runtime::wake() {
  uint64_t one = 1;
  ssize_t k = ::write(wake_fd_, &one, 8);
  (void)k;
}

void Runtime::shutdown() {
  if (shutdown_done_) return;
  shutdown_done_ = true;
  if (!broken_.load() && thread_.joinable()) {
    try {
      std::unique_ptr<OpRecord> rec(new OpRecord());
      rec->name = "__shutdown__";
      rec->op = OpType::SHUTDOWN;
      int64_t h = enqueue(std::move(rec));
      wait(h, std::min(opt_.timeout_s, 30.0));
      release(h);
    } catch (const std::exception& e) {
      BC_LOG(1, "shutdown handshake failed: %s", e.what());
    }
  }
  stop_.store(true);
  wake();
  if (thread_.joinable()) thread_.join();
  if (comm_) {
    cudaSetDevice(opt_.device);
    cudaDeviceSynchronize();
    if (!broken_.load()) {
      try {
        t_.barrier(now_s() + std::min(opt_.timeout_s, 30.0));
      } catch (...) {
      }
    }
    {
      std::lock_guard<std::mutex> g(stats_mu_);
      collect_timed_locked();
      for (auto& t : timed_) {
        cudaEventDestroy((cudaEvent_t)t.start);
        cudaEventDestroy((cudaEvent_t)t.stop);
      }
      timed_.clear();
      for (void* e : event_pool_) cudaEventDestroy((cudaEvent_t)e);
      event_pool_.clear();
    }
    if (pinned_) cudaFreeHost(pinned_);
    if (scratch_) cudaFree(scratch_);
    pinned_ = scratch_ = nullptr;
    comm_.reset();
  }
}

std::string Runtime::broken_reason() {
  std::lock_guard<std::mutex> g(mu_);
  return broken_reason_;
}

void Runtime::set_fault(const std::string& spec) {
  std::lock_guard<std::mutex> g(mu_);
  fault_ = FaultSpec::parse(spec);
}

// ---- user-thread side ----------------------------------------------------------------------

int64_t Runtime::enqueue(std::unique_ptr<OpRecord> rec_in) {
  std::shared_ptr<OpRecord> rec(rec_in.release());
  {
    std::lock_guard<std::mutex> g(mu_);
    if (broken_.load()) throw CommLost("communicator is broken: " + broken_reason_);
    BC_CHECK(!stop_.load(), "the runtime has been shut down");
    BC_CHECK(table_.find(rec->name) == table_.end(),
             "a collective named '" << rec->name << "' is already in flight on this rank");
    if (rec->device == DeviceKind::GPU) {
      BC_CHECK(comm_ != nullptr, "GPU tensor passed, but init() ran without a GPU device");
      cudaEvent_t ev = nullptr;
      cudaSetDevice(opt_.device);
      cudaError_t e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
      BC_CHECK(e == cudaSuccess, "cudaEventCreate: " << cudaGetErrorString(e));
      rec->done_event = ev;
    }
    rec->id = next_id_++;
    rec->t_enqueue = now_s();
    handles_[rec->id] = rec;
    table_[rec->name] = rec;
    queue_.push_back(rec);
  }
  wake();
  return rec->id;
}

std::shared_ptr<OpRecord> Runtime::get(int64_t handle) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = handles_.find(handle);
  BC_CHECK(it != handles_.end(), "unknown handle " << handle);
  return it->second;
}

bool Runtime::poll(int64_t handle) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = handles_.find(handle);
  BC_CHECK(it != handles_.end(), "unknown handle " << handle);
  return it->second->state != OpRecord::PENDING;
}

void Runtime::wait(int64_t handle, double timeout_s) {
  std::unique_lock<std::mutex> lk(mu_);
  auto it = handles_.find(handle);
  BC_CHECK(it != handles_.end(), "unknown handle " << handle);
  std::shared_ptr<OpRecord> rec = it->second;
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::duration<double>(timeout_s);
  // Most collectives finish within tens of microseconds: look a few times before sleeping.
  for (const double spin_until = now_s() + spin_s_; rec->state == OpRecord::PENDING && now_s() < spin_until;) {
    lk.unlock();
    for (int i = 0; i < 32; i++) cpu_pause();
    lk.lock();
  }
  while (rec->state == OpRecord::PENDING) {
    if (cv_.wait_until(lk, deadline) == std::cv_status::timeout && rec->state == OpRecord::PENDING)
      throw Error("timed out waiting for collective '" + rec->name + "'");
  }
  if (rec->state == OpRecord::FAILED) throw Error(rec->error);
}

void Runtime::release(int64_t handle) {
  std::shared_ptr<OpRecord> rec;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = handles_.find(handle);
    if (it == handles_.end()) return;
    rec = it->second;
    handles_.erase(it);
  }
  if (rec->done_event) {
    cudaEventDestroy((cudaEvent_t)rec->done_event);
    rec->done_event = nullptr;
  }
}

std::vector<std::string> Runtime::blob_gather(const std::string& name, const std::string& mine) {
  std::unique_ptr<OpRecord> rec(new OpRecord());
  rec->name = name;
  rec->op = OpType::BLOB_GATHER;
  rec->dtype = DType::U8;
  rec->blob = mine;
  int64_t h = enqueue(std::move(rec));
  wait(h, opt_.timeout_s + 5.0);
  std::vector<std::string> out = get(h)->blobs;
  release(h);
  return out;
}

// ---- background thread ---------------------------------------------------------------------

void Runtime::finish(const std::shared_ptr<OpRecord>& r, bool ok, const std::string& err) {
  r->t_done = now_s();
  {
    std::lock_guard<std::mutex> g(stats_mu_);
    StatEntry e;
    e.name = r->name;
    e.op = (int)r->op;
    e.algo = r->algo;
    e.device = (int)r->device;
    e.blocks = (comm_ && r->device == DeviceKind::GPU) ? comm_->last_blocks : 0;
    int64_t n = 1;
    for (int64_t d : r->shape) n *= d;
    e.bytes = n * (int64_t)dtype_size(r->dtype);
    e.t_enqueue = r->t_enqueue;
    e.t_negotiated = r->t_negotiated;
    e.t_done = r->t_done;
    for (int i = 0; i < 3; i++) e.two_level_s[i] = r->two_level_s[i];
    if (r->timed_stop) {
      // the device time is known once the stop event has completed: the record waits for it
      TimedLaunch t;
      t.entry = e;
      t.entry.channel = 0;
      t.start = r->timed_start;
      t.stop = r->timed_stop;
      r->timed_start = r->timed_stop = nullptr;
      timed_.push_back(t);
    } else {
      stats_.push_back(e);
      if (stats_.size() > 4096) stats_.pop_front();
    }
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    r->error = err;
    r->state = ok ? OpRecord::DONE : OpRecord::FAILED;
  }
  cv_.notify_all();
}

void Runtime::fail_everything(const std::string& why) {
  std::vector<std::shared_ptr<OpRecord>> victims;
  {
    std::lock_guard<std::mutex> g(mu_);
    broken_.store(true);
    broken_reason_ = why;
    for (auto& kv : table_) victims.push_back(kv.second);
    table_.clear();
    queue_.clear();
  }
  BC_LOG(0, "communicator failed: %s", why.c_str());
  if (t_.rank == 0) {
    Response abort_msg;
    abort_msg.type = ResponseType::ABORT;
    abort_msg.error = why;
    const std::string frame = encode(abort_msg);
    for (int r = 1; r < t_.size; r++) {
      if (!t_.ctrl[r].valid()) continue;
      try {
        t_.ctrl[r].send_frame(frame, now_s() + 1.0);
      } catch (...) {
      }
    }
  }
  for (auto& r : victims)
    if (r->state == OpRecord::PENDING) finish(r, false, "collective '" + r->name + "' failed: " + why);
}

void Runtime::loop() {
  if (comm_) cudaSetDevice(opt_.device);
  try {
    while (!stop_.load()) loop_body();
  } catch (const std::exception& e) {
    fail_everything(e.what());
  }
}

void Runtime::send_request(const OpRecord& rec) {
  Request q;
  q.rank = t_.rank;
  q.op = rec.op;
  q.dtype = rec.dtype;
  q.device = rec.device;
  q.name = rec.name;
  q.shape = rec.shape;
  q.blob = rec.blob;
  q.symm_off = -1;
  q.red = rec.red;
  if (rec.zero_copy && comm_ && !node_) {
    int64_t n = 1;
    for (int64_t d : rec.shape) n *= d;
    gpu::Segment* seg = comm_->allocator().find(rec.in, (size_t)n * dtype_size(rec.dtype));
    if (seg && rec.in == rec.out) q.symm_off = ((int64_t)seg->id << 48) | (int64_t)((const char*)rec.in - seg->local);
  }
  FaultSpec f;
  {
    std::lock_guard<std::mutex> g(mu_);
    f = fault_;
  }
  if (f.matches(t_.rank, rec.name)) {
    switch (f.kind) {
      case FaultSpec::DROP_REQUEST:
        BC_LOG(1, "fault injection: dropping request for '%s'", rec.name.c_str());
        return;
      case FaultSpec::DELAY_MS:
        std::this_thread::sleep_for(std::chrono::milliseconds(f.ms));
        break;
      case FaultSpec::EXIT_BEFORE:
        fprintf(stderr, "[bcoll] fault injection: exiting before '%s'\n", rec.name.c_str());
        fflush(stderr);
        _exit(41);
      case FaultSpec::CLOSE_CTRL:
        for (auto& s : t_.ctrl) s.close();
        throw CommLost("fault injection: control connection closed");
      default:
        break;
    }
  }
  if (t_.rank == 0) {
    coordinator_handle(q);
  } else {
    t_.ctrl[0].send_frame(encode(q), now_s() + opt_.timeout_s);
  }
}

void Runtime::drain_local_queue() {
  std::deque<std::shared_ptr<OpRecord>> local;
  {
    std::lock_guard<std::mutex> g(mu_);
    local.swap(queue_);
  }
  for (auto& rec : local) {
    BC_LOG(2, "request '%s'", rec->name.c_str());
    send_request(*rec);
  }
}

void Runtime::coordinator_handle(const Request& q) {
  BC_CHECK(q.rank >= 0 && q.rank < t_.size, "request from out-of-range rank " << q.rank);
  Pending& p = pending_[q.name];
  if (p.reqs.empty()) {
    p.reqs.resize(t_.size);
    p.have.assign(t_.size, false);
    p.first_seen = now_s();
  }
  if (p.have[q.rank]) {
    BC_LOG(0, "rank %d asked twice for '%s' before it completed; ignoring the second request", q.rank, q.name.c_str());
    return;
  }
  p.have[q.rank] = true;
  p.reqs[q.rank] = q;
  p.count++;
  if (p.count < t_.size) return;
  Response resp = build_response(q.name, p.reqs);
  pending_.erase(q.name);
  const std::string frame = encode(resp);
  for (int r = 1; r < t_.size; r++) t_.ctrl[r].send_frame(frame, now_s() + opt_.timeout_s);
  perform(resp);
}

void Runtime::coordinator_check_deadlines() {
  if (pending_.empty()) return;
  const double now = now_s();
  std::vector<std::string> late;
  for (auto& kv : pending_)
    if (now - kv.second.first_seen > opt_.timeout_s) late.push_back(kv.first);
  for (const auto& name : late) {
    Pending& p = pending_[name];
    std::string missing;
    for (int r = 0; r < t_.size; r++)
      if (!p.have[r]) missing += (missing.empty() ? "" : ",") + std::to_string(r);
    Response resp;
    resp.type = ResponseType::ERROR;
    resp.name = name;
    resp.error = "Timed out after " + std::to_string((int)opt_.timeout_s) + " s waiting for rank(s) " + missing +
                 " to request collective '" + name + "'.";
    pending_.erase(name);
    const std::string frame = encode(resp);
    for (int r = 1; r < t_.size; r++) t_.ctrl[r].send_frame(frame, now_s() + opt_.timeout_s);
    perform(resp);
  }
}

void Runtime::loop_body() {
  std::vector<struct pollfd> fds;
  std::vector<int> who;
  fds.push_back({wake_fd_, POLLIN, 0});
  who.push_back(-1);
  if (t_.size > 1) {
    if (t_.rank == 0) {
      for (int r = 1; r < t_.size; r++) {
        fds.push_back({t_.ctrl[r].fd(), POLLIN, 0});
        who.push_back(r);
      }
    } else {
      fds.push_back({t_.ctrl[0].fd(), POLLIN, 0});
      who.push_back(0);
    }
  }
  const int timeout_ms = (t_.rank == 0 && !pending_.empty()) ? 50 : 500;
  // Collectives come in bursts (one per gradient, one per step): for a short while after the last
  // event the thread polls without sleeping, which saves a wake-up per message; then it blocks.
  int rc = 0;
  if (spin_s_ > 0 && now_s() - last_event_s_ < spin_s_) {
    do {
      rc = ::poll(fds.data(), fds.size(), 0);
      if (rc != 0) break;
      for (int i = 0; i < 32; i++) cpu_pause();
    } while (now_s() - last_event_s_ < spin_s_);
  }
  if (rc == 0) rc = ::poll(fds.data(), fds.size(), timeout_ms);
  if (rc < 0) {
    if (errno == EINTR) return;
    throw CommLost(std::string("poll failed: ") + strerror(errno));
  }
  if (rc > 0) last_event_s_ = now_s();
  if (fds[0].revents & POLLIN) {
    uint64_t v;
    while (::read(wake_fd_, &v, 8) == 8) {
    }
    drain_local_queue();
  }
  for (size_t i = 1; i < fds.size(); i++) {
    if (!(fds[i].revents & (POLLIN | POLLHUP | POLLERR))) continue;
    if (stop_.load()) break;
    const int r = who[i];
    std::string frame;
    try {
      frame = t_.ctrl[r].recv_frame(now_s() + opt_.timeout_s);
    } catch (const CommLost& e) {
      throw CommLost("lost the control connection to rank " + std::to_string(r) + " (" + e.what() + ")");
    }
    if (t_.rank == 0) {
      coordinator_handle(decode_request(frame));
    } else {
      perform(decode_response(frame));
    }
  }
  if (t_.rank == 0) coordinator_check_deadlines();
}

void Runtime::perform(const Response& resp) {
  if (resp.type == ResponseType::ABORT) throw CommLost(resp.error.empty() ? "aborted by rank 0" : resp.error);
  std::shared_ptr<OpRecord> rec;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = table_.find(resp.name);
    if (it != table_.end()) {
      rec = it->second;
      table_.erase(it);
    }
  }
  if (!rec) {
    if (resp.type == ResponseType::ERROR) {
      BC_LOG(1, "error for a collective this rank has not requested ('%s'): %s", resp.name.c_str(), resp.error.c_str());
      return;
    }
    throw Error("received a go-ahead for unknown collective '" + resp.name + "'");
  }
  rec->t_negotiated = now_s();
  BC_LOG(2, "perform '%s' type=%d", rec->name.c_str(), (int)resp.type);
  {
    FaultSpec f;
    {
      std::lock_guard<std::mutex> g(mu_);
      f = fault_;
    }
    if (f.kind == FaultSpec::EXIT_IN_COLLECTIVE && f.matches(t_.rank, rec->name)) {
      // The go-ahead has arrived and the peers are entering the data phase: leave now.
      fprintf(stderr, "[bcoll] fault injection: exiting inside '%s'\n", rec->name.c_str());
      fflush(stderr);
      _exit(42);
    }
  }
  NvtxRange range(resp.type == ResponseType::ALLGATHER ? "bcoll.allgather" : resp.type == ResponseType::ALLREDUCE ? "bcoll.allreduce" : "bcoll.control");
  try {
    switch (resp.type) {
      case ResponseType::ERROR:
        finish(rec, false, resp.error);
        return;
      case ResponseType::ALLREDUCE:
        rec->zero_copy = rec->zero_copy && (resp.flags & kFlagZeroCopy);
        perform_allreduce(*rec);
        break;
      case ResponseType::ALLGATHER:
        perform_allgather(*rec, resp);
        break;
      case ResponseType::BLOB_GATHER:
        rec->blobs = resp.blobs;
        break;
      case ResponseType::SHUTDOWN:
        stop_.store(true);
        break;
      default:
        throw Error("unexpected response type");
    }
    finish(rec, true, "");
    BC_LOG(2, "performed '%s'", rec->name.c_str());
  } catch (const CommLost&) {
    finish(rec, false, "collective '" + rec->name + "' failed: connection lost");
    throw;
  } catch (const std::exception& e) {
    finish(rec, false, e.what());
  }
}

void Runtime::perform_allreduce(OpRecord& r) {
  size_t count = 1;
  for (int64_t d : r.shape) count *= (size_t)d;
  BC_CHECK(!(r.average && r.red != ReduceOp::SUM), "allreduce: averaging goes with the sum only");
  const double scale = r.average ? 1.0 / t_.size : 1.0;
  const int64_t idiv = r.average ? t_.size : 1;
  if (r.device == DeviceKind::CPU) {
    const double deadline = now_s() + opt_.timeout_s;
    if (shm_ && !node_) {
      // reads the input where it is and writes the result where it belongs: no copy in between
      shm_->allreduce(r.in, r.out, count, r.dtype, scale, idiv, r.red, deadline);
      r.algo = 4;
      return;
    }
    if (r.in != r.out && count) memcpy(r.out, r.in, count * dtype_size(r.dtype));
    if (shm_ && node_) {
      // several hosts with several ranks each: shared memory inside the host, rails between hosts
      const size_t es = dtype_size(r.dtype);
      const size_t chunk_elems = two_level_chunk_bytes_ / es;
      if (chunk_elems > 0 && count >= 4 * chunk_elems) {
        // large tensors: chunk by chunk, the step between the hosts on a helper thread beside the steps inside the host
        cpu_staging_.resize(2 * slice_len(chunk_elems, node_->local_size, 0) * es + 16);
        bc::two_level_allreduce_pipelined(*node_, *shm_, r.out, cpu_staging_.data(), count, chunk_elems, r.dtype, scale, idiv, r.red,
                                          deadline, r.two_level_s);
      } else {
        ShmLocalLevel local(*shm_, r.out, deadline);
        cpu_staging_.resize(slice_len(count, node_->local_size, 0) * es + 16);
        bc::two_level_allreduce(*node_, local, cpu_staging_.data(), count, r.dtype, scale, idiv, r.red, deadline, r.two_level_s);
      }
    } else {
      cpu_ring_allreduce(t_, r.out, count, r.dtype, scale, idiv, deadline, r.red);
    }
    r.algo = shm_ ? 4 : 0;
    return;
  }
  BC_CHECK(comm_, "GPU collective without a GPU communicator");
  BC_CHECK(comm_->device_status() == 0, "an earlier device-side wait timed out (status 0x" << std::hex << comm_->device_status()
           << "); the communicator cannot be used any more");
  cudaStream_t s = comm_->stream(0);
  if (r.ready_event) {
    cudaError_t e = cudaStreamWaitEvent(s, (cudaEvent_t)r.ready_event, 0);
    BC_CHECK(e == cudaSuccess, "cudaStreamWaitEvent: " << cudaGetErrorString(e));
  }
  TimedLaunch timed;
  if (device_timing()) timed = timed_begin(s);
  if (node_)
    two_level_allreduce(r, count, scale, idiv);
  else
    r.algo = (int)comm_->allreduce(0, r.in, r.out, count, r.dtype, (float)scale, (int)idiv, r.zero_copy, r.red);
  if (timed.stop) {
    cudaError_t te = cudaEventRecord((cudaEvent_t)timed.stop, s);
    BC_CHECK(te == cudaSuccess, "cudaEventRecord: " << cudaGetErrorString(te));
    r.timed_start = timed.start;
    r.timed_stop = timed.stop;
  }
  cudaError_t e = cudaEventRecord((cudaEvent_t)r.done_event, s);
  BC_CHECK(e == cudaSuccess, "cudaEventRecord: " << cudaGetErrorString(e));
}

void Runtime::perform_allgather(OpRecord& r, const Response& resp) {
  BC_CHECK((int)resp.dim0.size() == t_.size, "allgather response lacks the per-rank sizes");
  r.dim0 = resp.dim0;
  int64_t total_rows = 0;
  for (int64_t d : r.dim0) total_rows += d;
  size_t row_bytes = dtype_size(r.dtype);
  for (size_t i = 1; i < r.shape.size(); i++) row_bytes *= (size_t)r.shape[i];
  int is_symm = 0;
  BC_CHECK(r.alloc, "allgather needs an output allocator");
  BC_LOG(2, "allgather '%s': asking for %lld rows", r.name.c_str(), (long long)total_rows);
  r.out = r.alloc(r.id, total_rows, r.alloc_user, &is_symm);
  BC_LOG(2, "allgather '%s': output %p symmetric=%d", r.name.c_str(), r.out, is_symm);
  const size_t total_bytes = (size_t)total_rows * row_bytes;
  BC_CHECK(r.out || total_bytes == 0, "the output allocator returned no buffer");
  if (r.device == DeviceKind::CPU) {
    if (shm_ && !node_)
      shm_->allgatherv(r.in, r.out, r.dim0, row_bytes, now_s() + opt_.timeout_s);
    else
      cpu_ring_allgatherv(t_, r.in, r.out, r.dim0, row_bytes, now_s() + opt_.timeout_s);
    r.algo = (shm_ && !node_) ? 4 : 0;
    return;
  }
  BC_CHECK(comm_, "GPU collective without a GPU communicator");
  BC_CHECK(comm_->device_status() == 0, "an earlier device-side wait timed out; the communicator cannot be used any more");
  cudaStream_t s = comm_->stream(0);
  if (r.ready_event) {
    cudaError_t e = cudaStreamWaitEvent(s, (cudaEvent_t)r.ready_event, 0);
    BC_CHECK(e == cudaSuccess, "cudaStreamWaitEvent: " << cudaGetErrorString(e));
  }
  if (node_) {
    two_level_allgather(r, row_bytes, total_bytes);
  } else {
    std::vector<unsigned long long> slab_bytes(r.dim0.size());
    for (size_t i = 0; i < r.dim0.size(); i++) slab_bytes[i] = (unsigned long long)r.dim0[i] * row_bytes;
    comm_->allgatherv(0, r.in, (size_t)r.shape[0] * row_bytes, is_symm ? r.out : nullptr, is_symm ? nullptr : r.out, total_bytes,
                      nullptr, slab_bytes.data());
  }
  r.algo = 0;
  cudaError_t e = cudaEventRecord((cudaEvent_t)r.done_event, s);
  BC_CHECK(e == cudaSuccess, "cudaEventRecord: " << cudaGetErrorString(e));
}

// ---- GPU groups over several hosts -----------------------------------------------------------

void* Runtime::pinned(size_t bytes) {
  if (bytes > pinned_bytes_) {
    if (pinned_) cudaFreeHost(pinned_);
    pinned_ = nullptr;
    pinned_bytes_ = 0;
    const size_t want = std::max<size_t>(bytes + bytes / 4, 1u << 20);
    cudaError_t e = cudaMallocHost(&pinned_, want);
    BC_CHECK(e == cudaSuccess, "cudaMallocHost(" << want << "): " << cudaGetErrorString(e));
    pinned_bytes_ = want;
  }
  return pinned_;
}

void* Runtime::device_scratch(size_t bytes) {
  if (bytes > scratch_bytes_) {
    cudaStream_t s = comm_->stream(0);
    cudaStreamSynchronize(s);          // an earlier gather may still read the old scratch
    if (scratch_) cudaFree(scratch_);
    scratch_ = nullptr;
    scratch_bytes_ = 0;
    const size_t want = std::max<size_t>(bytes + bytes / 4, 1u << 20);
    cudaError_t e = cudaMalloc(&scratch_, want);
    BC_CHECK(e == cudaSuccess, "cudaMalloc(" << want << "): " << cudaGetErrorString(e));
    scratch_bytes_ = want;
  }
  return scratch_;
}

namespace {

void check(cudaError_t e, const char* what) { BC_CHECK(e == cudaSuccess, what << ": " << cudaGetErrorString(e)); }

// The levels inside a host on GPUs: the NVLink kernels of the host's communicator, and copies
// between the device and pinned host memory on the communicator's stream.
class GpuLocalLevel : public LocalLevel {
 public:
  GpuLocalLevel(gpu::Comm& c, const void* in, void* out, std::function<void*(size_t)> scratch)
      : c_(c), in_(in), out_((char*)out), scratch_(std::move(scratch)), s_(c.stream(0)) {}

  void reduce_in_node(size_t count, DType dtype, ReduceOp red) override {
    if (c_.world() > 1)
      c_.allreduce(0, in_, out_, count, dtype, 1.f, 1, false, red);
    else if (in_ != out_ && count)
      check(cudaMemcpyAsync(out_, in_, count * dtype_size(dtype), cudaMemcpyDeviceToDevice, s_), "cudaMemcpyAsync");
  }

  void fetch(void* dst, size_t begin, size_t len, DType dtype) override {
    const size_t e = dtype_size(dtype);
    if (len) check(cudaMemcpyAsync(dst, out_ + begin * e, len * e, cudaMemcpyDeviceToHost, s_), "cudaMemcpyAsync (to host)");
    check(cudaStreamSynchronize(s_), "cudaStreamSynchronize");
  }

  void finish(const void* src, size_t begin, size_t len, const std::vector<size_t>& lens, DType dtype) override {
    const size_t e = dtype_size(dtype);
    if (c_.world() == 1) {
      if (len) check(cudaMemcpyAsync(out_ + begin * e, src, len * e, cudaMemcpyHostToDevice, s_), "cudaMemcpyAsync (to device)");
      return;
    }
    // The gather's input must not alias its output: the slice goes to scratch memory first.
    void* mine = scratch_(len * e);
    if (len) check(cudaMemcpyAsync(mine, src, len * e, cudaMemcpyHostToDevice, s_), "cudaMemcpyAsync (to device)");
    std::vector<unsigned long long> slab(lens.size());
    size_t total = 0;
    for (size_t i = 0; i < lens.size(); i++) {
      slab[i] = (unsigned long long)(lens[i] * e);
      total += lens[i] * e;
    }
    c_.allgatherv(0, mine, len * e, nullptr, out_, total, nullptr, slab.data());
  }

 private:
  gpu::Comm& c_;
  const void* in_;
  char* out_;
  std::function<void*(size_t)> scratch_;
  cudaStream_t s_;
};

}  // namespace

void Runtime::two_level_allreduce(OpRecord& r, size_t count, double scale, int64_t idiv) {
  const size_t e = dtype_size(r.dtype);
  void* staging = pinned(slice_len(count, node_->local_size, 0) * e);
  GpuLocalLevel local(*comm_, r.in, r.out, [this](size_t b) { return device_scratch(b); });
  bc::two_level_allreduce(*node_, local, staging, count, r.dtype, scale, idiv, r.red, now_s() + opt_.timeout_s, r.two_level_s);
  // The pinned slice is read by a copy that is still queued; the next operation reuses it.
  check(cudaStreamSynchronize(comm_->stream(0)), "cudaStreamSynchronize");
  r.algo = 0;
}

void Runtime::two_level_allgather(OpRecord& r, size_t row_bytes, size_t total_bytes) {
  // Slabs travel through host memory over the ring of all ranks, as with the reference's MPI
  // ring on a build without GPU-aware MPI; gathers carry little data (sparse gradients, shapes).
  cudaStream_t s = comm_->stream(0);
  char* host = (char*)pinned(total_bytes);
  size_t my_off = 0;
  for (int i = 0; i < t_.rank; i++) my_off += (size_t)r.dim0[i] * row_bytes;
  const size_t my_bytes = (size_t)r.dim0[t_.rank] * row_bytes;
  if (my_bytes) check(cudaMemcpyAsync(host + my_off, r.in, my_bytes, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync (to host)");
  check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  cpu_ring_allgatherv(t_, host + my_off, host, r.dim0, row_bytes, now_s() + opt_.timeout_s);   // own slab already in place
  if (total_bytes) check(cudaMemcpyAsync(r.out, host, total_bytes, cudaMemcpyHostToDevice, s), "cudaMemcpyAsync (to device)");
  check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
}

// ---- stats ---------------------------------------------------------------------------------

TimedLaunch Runtime::timed_begin(void* stream) {
  TimedLaunch t;
  {
    std::lock_guard<std::mutex> g(stats_mu_);
    for (void** e : {&t.start, &t.stop}) {
      if (!event_pool_.empty()) {
        *e = event_pool_.back();
        event_pool_.pop_back();
      }
    }
  }
  for (void** e : {&t.start, &t.stop}) {
    if (!*e) {
      cudaEvent_t ev = nullptr;
      cudaError_t rc = cudaEventCreate(&ev);
      BC_CHECK(rc == cudaSuccess, "cudaEventCreate: " << cudaGetErrorString(rc));
      *e = ev;
    }
  }
  t.entry.t_enqueue = now_s();
  cudaError_t rc = cudaEventRecord((cudaEvent_t)t.start, (cudaStream_t)stream);
  BC_CHECK(rc == cudaSuccess, "cudaEventRecord: " << cudaGetErrorString(rc));
  return t;
}

void Runtime::timed_end(TimedLaunch t, void* stream, const char* name, int algo, int blocks, int64_t bytes, int channel) {
  cudaError_t rc = cudaEventRecord((cudaEvent_t)t.stop, (cudaStream_t)stream);
  BC_CHECK(rc == cudaSuccess, "cudaEventRecord: " << cudaGetErrorString(rc));
  t.entry.name = name;
  t.entry.op = (int)OpType::ALLREDUCE;
  t.entry.algo = algo;
  t.entry.device = (int)DeviceKind::GPU;
  t.entry.blocks = blocks;
  t.entry.bytes = bytes;
  t.entry.channel = channel;
  t.entry.t_negotiated = t.entry.t_enqueue;     // an ordered launch is not negotiated
  t.entry.t_done = now_s();
  std::lock_guard<std::mutex> g(stats_mu_);
  timed_.push_back(t);
  if (timed_.size() > 1024) collect_timed_locked();
}

void Runtime::collect_timed_locked() {
  while (!timed_.empty()) {
    TimedLaunch& t = timed_.front();
    if (cudaEventQuery((cudaEvent_t)t.stop) != cudaSuccess) {
      cudaGetLastError();      // "not ready" is not an error to keep
      break;
    }
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, (cudaEvent_t)t.start, (cudaEvent_t)t.stop) == cudaSuccess) t.entry.device_us = (double)ms * 1e3;
    stats_.push_back(t.entry);
    if (stats_.size() > 4096) stats_.pop_front();
    event_pool_.push_back(t.start);
    event_pool_.push_back(t.stop);
    timed_.pop_front();
  }
}

std::string Runtime::stats_json() {
  std::lock_guard<std::mutex> g(stats_mu_);
  collect_timed_locked();
  std::ostringstream os;
  os << "[";
  bool first = true;
  for (const auto& e : stats_) {
    if (!first) os << ",";
    first = false;
    os << "{\"name\":\"";
    for (char ch : e.name) {
      if (ch == '"' || ch == '\\') os << '\\';
      os << ch;
    }
    os.precision(9);
    os << "\",\"op\":" << e.op << ",\"algo\":" << e.algo << ",\"device\":" << e.device << ",\"blocks\":" << e.blocks
       << ",\"bytes\":" << e.bytes << std::fixed << ",\"t_enqueue\":" << e.t_enqueue << ",\"t_negotiated\":" << e.t_negotiated
       << ",\"t_done\":" << e.t_done;
    if (e.two_level_s[0] > 0 || e.two_level_s[1] > 0 || e.two_level_s[2] > 0)
      os << ",\"two_level_s\":[" << e.two_level_s[0] << "," << e.two_level_s[1] << "," << e.two_level_s[2] << "]";
    if (e.device_us >= 0) os << ",\"device_us\":" << e.device_us;
    if (e.channel >= 0) os << ",\"channel\":" << e.channel;
    os << "}";
  }
  os << "]";
  return os.str();
}

void Runtime::clear_stats() {
  std::lock_guard<std::mutex> g(stats_mu_);
  stats_.clear();
}

}  // namespace bc
