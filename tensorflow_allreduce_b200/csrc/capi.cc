// C ABI of the native library (loaded from Python with ctypes; declarations in bcoll.h).
//
// This is the analogue of the reference's op registrations (MPIInit / MPISize / MPIRank /
// MPILocalRank / MPIAllreduce / MPIAllgather, tensorflow/contrib/mpi_collectives/mpi_ops.cc:878-1270):
// thin entry points over the runtime. Every function returns 0 / a non-negative value on success
// and -1 on failure; bc_last_error() then holds the message for the calling thread.
#include "bcoll.h"

#include <cuda_runtime.h>
#include <string.h>

#include <memory>
#include <mutex>

#include "cuda/comm.h"
#include "cuda/bn_clip.h"
#include "cuda/gru_persistent.h"
#include "runtime/runtime.h"
#include "runtime/two_level.h"

using namespace bc;

namespace {

std::unique_ptr<Runtime> g_rt;
std::mutex g_mu;
thread_local std::string t_err;
thread_local std::string t_str;
int64_t g_segment_seq = 0;

Runtime& rt() {
  if (!g_rt) throw Error("MPI has not been initialized; use Session or init() first.");
  return *g_rt;
}

gpu::Comm& comm() {
  Runtime& r = rt();
  if (!r.comm()) throw Error("init() ran without a GPU device; GPU collectives are unavailable");
  return *r.comm();
}

#define API_BEGIN try {
#define API_END(fail)                      \
  }                                        \
  catch (const std::exception& e) {        \
    t_err = e.what();                      \
    return fail;                           \
  }                                        \
  catch (...) {                            \
    t_err = "unknown native error";        \
    return fail;                           \
  }

void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw Error(std::string(what) + ": " + cudaGetErrorString(e));
}

}  // namespace

extern "C" {

const char* bc_last_error() { return t_err.c_str(); }

int bc_init(int rank, int size, int local_rank, const char* addr, int port, int device, double timeout_s,
            double device_timeout_s, long long staging_bytes, long long heap_bytes, int force_algo,
            long long one_shot_max_bytes, long long nvls_min_bytes, int use_nvls, int max_blocks, int symm_mode,
            const char* fault) {
  API_BEGIN
  std::lock_guard<std::mutex> g(g_mu);
  if (g_rt) throw Error("init() was already called in this process");
  RuntimeOptions o;
  o.rank = rank;
  o.size = size;
  o.local_rank_override = local_rank;
  o.addr = addr ? addr : "127.0.0.1";
  o.port = port;
  o.device = device;
  o.timeout_s = timeout_s;
  o.device_timeout_s = device_timeout_s;
  if (staging_bytes > 0) o.staging_bytes = (size_t)staging_bytes;
  if (heap_bytes >= 0) o.heap_bytes = (size_t)heap_bytes;
  o.force_algo = force_algo;
  if (one_shot_max_bytes >= 0) o.one_shot_max_bytes = (size_t)one_shot_max_bytes;
  if (nvls_min_bytes >= 0) o.nvls_min_bytes = (size_t)nvls_min_bytes;
  o.use_nvls = use_nvls != 0;
  o.max_blocks = max_blocks;
  o.symm_mode = symm_mode;
  o.fault = fault ? fault : "";
  g_rt.reset(new Runtime(o));
  return 0;
  API_END(-1)
}

int bc_initialized() { return g_rt ? 1 : 0; }

int bc_shutdown() {
  API_BEGIN
  std::lock_guard<std::mutex> g(g_mu);
  if (g_rt) {
    g_rt->shutdown();
    g_rt.reset();
  }
  return 0;
  API_END(-1)
}

int bc_rank() { API_BEGIN return rt().rank(); API_END(-1) }
int bc_size() { API_BEGIN return rt().size(); API_END(-1) }
int bc_local_rank() { API_BEGIN return rt().local_rank(); API_END(-1) }
int bc_local_size() { API_BEGIN return rt().local_size(); API_END(-1) }
int bc_on_gpu() { API_BEGIN return rt().on_gpu() ? 1 : 0; API_END(-1) }
int bc_broken() { API_BEGIN return rt().broken() ? 1 : 0; API_END(-1) }
int bc_n_nodes() { API_BEGIN return rt().n_nodes(); API_END(-1) }
int bc_node_index() { API_BEGIN return rt().node_group() ? rt().node_group()->node_index : 0; API_END(-1) }

int bc_two_level_allreduce_host(void* data, long long count, int dtype, int average, int reduce_op) {
  API_BEGIN
  Runtime& r = rt();
  NodeGroup* g = r.node_group();
  if (!g) throw Error("no node groups: the ranks are on one host, or this CPU job was started without BC_NODE_GROUPS=1");
  if (reduce_op < 0 || reduce_op > (int)ReduceOp::MAX) throw Error("unknown reduction");
  if (average && reduce_op != (int)ReduceOp::SUM) throw Error("averaging goes with the sum only");
  const double deadline = now_s() + r.options().timeout_s;
  HostLocalLevel local(*g, data, deadline);
  std::vector<char> staging(slice_len((size_t)count, g->local_size, 0) * dtype_size((DType)dtype) + 16);
  two_level_allreduce(*g, local, staging.data(), (size_t)count, (DType)dtype, average ? 1.0 / r.size() : 1.0,
                      average ? r.size() : 1, (ReduceOp)reduce_op, deadline);
  return 0;
  API_END(-1)
}

int bc_select_algo(int world, long long bytes, int dtype, int in_place_or_fused, int has_multicast, int force_algo,
                   long long one_shot_max_bytes, long long nvls_min_bytes, int use_nvls) {
  API_BEGIN
  gpu::CommConfig cfg;
  cfg.force_algo = force_algo;
  if (one_shot_max_bytes >= 0) cfg.one_shot_max_bytes = (size_t)one_shot_max_bytes;
  if (nvls_min_bytes >= 0) cfg.nvls_min_bytes = (size_t)nvls_min_bytes;
  cfg.use_nvls = use_nvls != 0;
  return (int)gpu::select_algo(cfg, world, (size_t)bytes, (DType)dtype, in_place_or_fused != 0, has_multicast != 0);
  API_END(-1)
}

int bc_plan_pipeline(long long bytes, long long slice_bytes, long long chunk_bytes, int slots, int cgroups, long long unit_bytes,
                     long long* out4) {
  API_BEGIN
  gpu::CommConfig cfg;
  if (cgroups > 0) cfg.pipeline_cgroups = cgroups;
  if (chunk_bytes > 0) cfg.pipeline_chunk_bytes = (size_t)chunk_bytes;
  if (slots > 0) cfg.pipeline_slots = slots;
  const gpu::PipePlan p = gpu::plan_pipeline(cfg, (size_t)bytes, (size_t)slice_bytes, (size_t)std::max<long long>(unit_bytes, 0));
  out4[0] = (long long)p.chunk_bytes;
  out4[1] = p.nchunks;
  out4[2] = p.slots;
  out4[3] = p.lag;
  return 0;
  API_END(-1)
}

long long bc_plan_gather_rounds(int world, const unsigned long long* all_bytes, long long staging_bytes, unsigned long long* pieces_out) {
  API_BEGIN
  std::vector<size_t> piece;
  const size_t rounds = gpu::plan_gather_rounds(all_bytes, world, (size_t)staging_bytes, &piece);
  for (int p = 0; p < world; p++) pieces_out[p] = piece[p];
  return (long long)rounds;
  API_END(-1)
}

int bc_choose_blocks(long long bytes, int world, int algo, int fused_update, int sm_count, int cap_override, int beside_compute) {
  API_BEGIN
  return gpu::choose_blocks((size_t)bytes, world, algo, fused_update != 0, sm_count, cap_override, beside_compute != 0);
  API_END(-1)
}

static void require_healthy(gpu::Comm& c) {
  const unsigned st = c.device_status();
  if (st == 0) return;
  if (st & dev::kStatusLayout)
    throw Error("an in-place reduction found its tensor at different offsets of symmetric memory on different ranks; its result "
                "is wrong and the communicator cannot be used any more");
  throw Error("an earlier device-side wait timed out; the communicator cannot be used any more");
}

static void check_channel(int channel) {
  if (channel < 0 || channel >= dev::kUserChannels) throw Error("bad channel (0.." + std::to_string(dev::kUserChannels - 1) + ")");
}

// Entry points that address the communicator directly assume that it spans the whole job.
static void require_one_host(const char* what) {
  if (rt().n_nodes() > 1)
    throw Error(std::string(what) + " is not available while the GPU ranks span several hosts; use the negotiated collectives");
}

long long bc_allreduce_async(const char* name, const void* in, void* out, int dtype, int ndim, const long long* shape,
                             int device_kind, int average, int zero_copy, void* ready_event, int reduce_op) {
  API_BEGIN
  std::unique_ptr<OpRecord> r(new OpRecord());
  r->name = name;
  r->op = OpType::ALLREDUCE;
  r->dtype = (DType)dtype;
  r->device = (DeviceKind)device_kind;
  r->shape.assign(shape, shape + ndim);
  r->in = in;
  r->out = out;
  r->average = average != 0;
  if (reduce_op < 0 || reduce_op > (int)ReduceOp::MAX) throw Error("allreduce: unknown reduction");
  r->red = (ReduceOp)reduce_op;
  r->zero_copy = zero_copy != 0;
  r->ready_event = ready_event;
  return rt().enqueue(std::move(r));
  API_END(-1)
}

long long bc_allgather_async(const char* name, const void* in, int dtype, int ndim, const long long* shape, int device_kind,
                             bc_alloc_fn alloc, void* user, void* ready_event) {
  API_BEGIN
  std::unique_ptr<OpRecord> r(new OpRecord());
  r->name = name;
  r->op = OpType::ALLGATHER;
  r->dtype = (DType)dtype;
  r->device = (DeviceKind)device_kind;
  r->shape.assign(shape, shape + ndim);
  r->in = in;
  r->alloc = (AllocFn)alloc;
  r->alloc_user = user;
  r->ready_event = ready_event;
  return rt().enqueue(std::move(r));
  API_END(-1)
}

int bc_wait(long long handle, double timeout_s) {
  API_BEGIN
  rt().wait(handle, timeout_s);
  return 0;
  API_END(-1)
}

int bc_poll(long long handle) { API_BEGIN return rt().poll(handle) ? 1 : 0; API_END(-1) }

void* bc_done_event(long long handle) { API_BEGIN return rt().get(handle)->done_event; API_END(nullptr) }

int bc_result_algo(long long handle) { API_BEGIN return rt().get(handle)->algo; API_END(-1) }

int bc_result_dim0(long long handle, long long* out, int n) {
  API_BEGIN
  auto r = rt().get(handle);
  if ((int)r->dim0.size() != n) throw Error("bc_result_dim0: size mismatch");
  for (int i = 0; i < n; i++) out[i] = r->dim0[i];
  return 0;
  API_END(-1)
}

int bc_release(long long handle) { API_BEGIN rt().release(handle); return 0; API_END(-1) }

int bc_blob_gather(const char* name, const void* data, int len, void* out, long long out_cap, int* lens) {
  API_BEGIN
  std::vector<std::string> all = rt().blob_gather(name, std::string((const char*)data, (size_t)len));
  long long pos = 0;
  for (size_t r = 0; r < all.size(); r++) {
    if (pos + (long long)all[r].size() > out_cap) throw Error("bc_blob_gather: output buffer too small");
    memcpy((char*)out + pos, all[r].data(), all[r].size());
    lens[r] = (int)all[r].size();
    pos += (long long)all[r].size();
  }
  return 0;
  API_END(-1)
}

int bc_set_fault(const char* spec) { API_BEGIN rt().set_fault(spec ? spec : ""); return 0; API_END(-1) }

const char* bc_stats_json() {
  API_BEGIN
  t_str = rt().stats_json();
  return t_str.c_str();
  API_END(nullptr)
}

int bc_clear_stats() { API_BEGIN rt().clear_stats(); return 0; API_END(-1) }

unsigned bc_device_status() { API_BEGIN return rt().comm() ? rt().comm()->device_status() : 0u; API_END(0u) }

int bc_set_device_timeout(double s) { API_BEGIN comm().set_device_timeout(s); return 0; API_END(-1) }

// ---- symmetric memory -------------------------------------------------------------------------

void* bc_symm_heap(long long* bytes) {
  API_BEGIN
  if (bytes) *bytes = (long long)comm().heap_bytes();
  return comm().heap_base();
  API_END(nullptr)
}

void* bc_symm_new_segment(long long bytes, int* seg_id, int* has_multicast) {
  API_BEGIN
  require_one_host("a user segment of symmetric memory");
  Runtime& r = rt();
  gpu::Comm& c = comm();
  const int64_t seq = g_segment_seq++;
  int64_t step = 0;
  gpu::HostAllgather ag = [&](const std::string& mine) {
    return r.blob_gather("__symm." + std::to_string(seq) + "." + std::to_string(step++), mine);
  };
  gpu::Segment* s = c.new_segment((size_t)bytes, ag);
  if (seg_id) *seg_id = s->id;
  if (has_multicast) *has_multicast = s->mc ? 1 : 0;
  return s->local;
  API_END(nullptr)
}

int bc_symm_contains(const void* p, long long bytes) {
  API_BEGIN
  return comm().allocator().find(p, (size_t)bytes) ? 1 : 0;
  API_END(-1)
}

const char* bc_symm_describe() {
  API_BEGIN
  t_str = comm().allocator().describe();
  return t_str.c_str();
  API_END(nullptr)
}

void* bc_comm_stream(int channel) {
  API_BEGIN
  check_channel(channel);
  return comm().stream(channel);
  API_END(nullptr)
}

int bc_stream_wait_event(void* stream, void* event) {
  API_BEGIN
  if (event) check_cuda(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0), "cudaStreamWaitEvent");
  return 0;
  API_END(-1)
}

// ---- ordered launches (no negotiation; every rank must issue the same sequence per channel) ------

static void stream_prologue(cudaStream_t s, void* wait_event) {
  if (wait_event) check_cuda(cudaStreamWaitEvent(s, (cudaEvent_t)wait_event, 0), "cudaStreamWaitEvent");
}
static void stream_epilogue(cudaStream_t s, void* record_event) {
  if (record_event) check_cuda(cudaEventRecord((cudaEvent_t)record_event, s), "cudaEventRecord");
}

int bc_allreduce_direct(int channel, const void* in, void* out, long long count, int dtype, int average,
                        void* wait_event, void* record_event) {
  API_BEGIN
  require_one_host("an ordered allreduce");
  check_channel(channel);
  gpu::Comm& c = comm();
  require_healthy(c);
  cudaStream_t s = c.stream(channel);
  stream_prologue(s, wait_event);
  const int n = c.world();
  TimedLaunch timed;
  if (rt().device_timing()) timed = rt().timed_begin(s);
  // Nothing was negotiated: whether the tensor is symmetric is this rank's own finding, so the
  // kernel compares the offsets that the ranks pass (check_place).
  gpu::Algo a = c.allreduce(channel, in, out, (size_t)count, (DType)dtype, average ? 1.f / n : 1.f, average ? n : 1, in == out,
                            ReduceOp::SUM, true);
  if (timed.stop) rt().timed_end(timed, s, "allreduce_direct", (int)a, c.last_blocks, count * (long long)dtype_size((DType)dtype), channel);
  stream_epilogue(s, record_event);
  return (int)a;
  API_END(-1)
}

int bc_fused_step(int channel, void* grad, long long count, int dtype, void* param, float* master, float* s1, float* s2,
                  const bc_opt_hyper* h, float scale, void* wait_event, void* record_event, int beside_compute) {
  API_BEGIN
  NvtxRange range("bcoll.fused_step");
  require_one_host("the fused update");
  check_channel(channel);
  gpu::Comm& c = comm();
  require_healthy(c);
  cudaStream_t s = c.stream(channel);
  stream_prologue(s, wait_event);
  static_assert(sizeof(bc_opt_hyper) == sizeof(gpu::OptHyper), "bc_opt_hyper must mirror OptHyper");
  gpu::OptHyper hh;
  memcpy(&hh, h, sizeof(hh));
  TimedLaunch timed;
  if (rt().device_timing()) timed = rt().timed_begin(s);
  gpu::Algo a = c.fused_step(channel, grad, (size_t)count, (DType)dtype, param, master, s1, s2, hh, scale, nullptr, beside_compute != 0);
  if (timed.stop) rt().timed_end(timed, s, "fused_step", (int)a, c.last_blocks, count * (long long)dtype_size((DType)dtype), channel);
  stream_epilogue(s, record_event);
  return (int)a;
  API_END(-1)
}

int bc_set_option(const char* key, long long value) {
  API_BEGIN
  const std::string k = key ? key : "";
  if (k == "device_timing") {
    rt().set_device_timing(value != 0);
  } else if (k == "overlap_blocks") {
    comm().set_overlap_blocks((int)value);
  } else if (k == "staged_pipeline") {
    comm().mutable_config().staged_pipeline = (int)value;
  } else if (k == "pipeline_min_bytes") {
    comm().mutable_config().pipeline_min_bytes = (size_t)std::max<long long>(value, 16);
  } else if (k == "pipeline_chunk_bytes") {
    comm().mutable_config().pipeline_chunk_bytes = (size_t)std::max<long long>(value, 4096);
  } else if (k == "pipeline_slots") {
    comm().mutable_config().pipeline_slots = (int)std::min<long long>(std::max<long long>(value, 2), 1024);
  } else if (k == "pipeline_copiers") {
    comm().mutable_config().pipeline_copiers = (int)std::min<long long>(std::max<long long>(value, 0), 200);
  } else if (k == "pipeline_streaming") {
    comm().mutable_config().pipeline_streaming = value != 0;
  } else if (k == "pipeline_rgroups") {
    comm().mutable_config().pipeline_rgroups = (int)std::min<long long>(std::max<long long>(value, 1), dev::kPipeMaxGroups);
  } else if (k == "pipeline_cgroups") {
    comm().mutable_config().pipeline_cgroups = (int)std::min<long long>(std::max<long long>(value, 1), dev::kPipeMaxGroups);
  } else if (k == "pipeline_reducers") {
    comm().mutable_config().pipeline_reducers = (int)std::min<long long>(std::max<long long>(value, 0), 96);
  } else {
    throw Error("unknown option '" + k + "'");
  }
  return 0;
  API_END(-1)
}

int bc_set_allreduce_profile(void* stamps) {
  API_BEGIN
  comm().set_profile((unsigned long long*)stamps);
  return 0;
  API_END(-1)
}

int bc_allgatherv_direct(int channel, const void* in, long long bytes, void* out_symm, long long capacity_bytes,
                         unsigned long long* sizes_out, void* wait_event, void* record_event) {
  API_BEGIN
  require_one_host("an ordered allgather");
  check_channel(channel);
  gpu::Comm& c = comm();
  require_healthy(c);
  cudaStream_t s = c.stream(channel);
  stream_prologue(s, wait_event);
  c.allgatherv(channel, in, (size_t)bytes, out_symm, nullptr, (size_t)capacity_bytes, sizes_out);
  stream_epilogue(s, record_event);
  return 0;
  API_END(-1)
}

// ---- single-GPU emulation of a rank group --------------------------------------------------------

void* bc_emu_create(int device, int nranks, long long bytes_per_rank) {
  API_BEGIN
  return new gpu::EmuGroup(device, nranks, (size_t)bytes_per_rank);
  API_END(nullptr)
}

int bc_emu_destroy(void* g) { API_BEGIN delete (gpu::EmuGroup*)g; return 0; API_END(-1) }

void* bc_emu_buffer(void* g, int r) { API_BEGIN return ((gpu::EmuGroup*)g)->buffer(r); API_END(nullptr) }

long long bc_emu_damaged_guard_bytes(void* g) {
  API_BEGIN
  return (long long)((gpu::EmuGroup*)g)->damaged_guard_bytes();
  API_END(-1)
}

unsigned bc_emu_status(void* g) { API_BEGIN return ((gpu::EmuGroup*)g)->status(); API_END(0u) }

int bc_emu_clear_status(void* g) { API_BEGIN ((gpu::EmuGroup*)g)->clear_status(); return 0; API_END(-1) }

int bc_emu_allreduce(void* g, long long off, void* const* outs, long long count, int dtype, int algo, float scale, int idiv,
                     int blocks, void* stream, int reduce_op, const void* const* srcs, const unsigned long long* places, void* prof,
                     int phase1_blocks) {
  API_BEGIN
  if (reduce_op < 0 || reduce_op > (int)ReduceOp::MAX) throw Error("unknown reduction");
  check_cuda(((gpu::EmuGroup*)g)->allreduce((size_t)off, outs, (size_t)count, (DType)dtype, (gpu::Algo)algo, scale, idiv, blocks,
                                            (cudaStream_t)stream, (ReduceOp)reduce_op, srcs, places, (unsigned long long*)prof,
                                            phase1_blocks),
             "emulated allreduce launch");
  return 0;
  API_END(-1)
}

int bc_emu_fused_step(void* g, long long off, long long count, int dtype, void* const* params, float* const* masters,
                      float* const* s1, float* const* s2, const bc_opt_hyper* h, float scale, int blocks, void* stream,
                      int phase1_blocks) {
  API_BEGIN
  gpu::OptHyper hh;
  memcpy(&hh, h, sizeof(hh));
  check_cuda(((gpu::EmuGroup*)g)->fused_step((size_t)off, (size_t)count, (DType)dtype, params, masters, s1, s2, hh, scale, blocks,
                                             (cudaStream_t)stream, phase1_blocks), "emulated fused step launch");
  return 0;
  API_END(-1)
}

int bc_emu_staged_pipeline(void* g, long long off, const void* const* srcs, void* const* outs, long long count, int dtype,
                           float scale, int idiv, long long chunk_bytes, int slots, int lag, int reducers, int copiers,
                           int rgroups, int cgroups, int streaming, void* stream) {
  API_BEGIN
  check_cuda(((gpu::EmuGroup*)g)->staged_pipeline((size_t)off, srcs, outs, (size_t)count, (DType)dtype, scale, idiv,
                                                  (size_t)chunk_bytes, slots, lag, reducers, copiers, rgroups, cgroups,
                                                  streaming != 0, (cudaStream_t)stream),
             "emulated staged pipeline launch");
  return 0;
  API_END(-1)
}

int bc_emu_allgatherv(void* g, const void* const* ins, const unsigned long long* bytes, const unsigned long long* out_offs,
                      int blocks, void* stream) {
  API_BEGIN
  check_cuda(((gpu::EmuGroup*)g)->allgatherv(ins, bytes, out_offs, blocks, (cudaStream_t)stream), "emulated allgatherv launch");
  return 0;
  API_END(-1)
}

int bc_emu_barrier_probe(void* g, int absent, double timeout_s, void* stream) {
  API_BEGIN
  check_cuda(((gpu::EmuGroup*)g)->barrier_probe(absent, timeout_s, (cudaStream_t)stream), "barrier probe launch");
  return 0;
  API_END(-1)
}

int bc_max_emulated_blocks(int device, int nranks) { return gpu::max_emulated_blocks(device, nranks, 512); }

// ---- persistent GRU layer -----------------------------------------------------------------------

int bc_gru_supported(int device, int T, int B, int H, int ndir) {
  API_BEGIN
  gpu::GruDims d{T, B, H, ndir};
  return gpu::gru_persistent_supported(d, device) ? 1 : 0;
  API_END(-1)
}

int bc_gru_set_profile(void* stamps) {
  gpu::gru_persistent_set_profile((unsigned long long*)stamps);
  return 0;
}

long long bc_gru_workspace_bytes(int T, int B, int H, int ndir) {
  gpu::GruDims d{T, B, H, ndir};
  return (long long)gpu::gru_persistent_workspace_bytes(d);
}

int bc_gru_forward(int T, int B, int H, int ndir, const float* w_hh, const float* b_hh, const float* gx, float* y, float* rsv,
                   float* workspace, unsigned* sync, unsigned* status, double timeout_s, void* stream) {
  API_BEGIN
  NvtxRange range("bcoll.gru_forward");
  gpu::GruDims d{T, B, H, ndir};
  check_cuda(gpu::gru_persistent_forward(d, w_hh, b_hh, gx, y, rsv, workspace, sync, status, timeout_s, (cudaStream_t)stream),
             "persistent GRU forward launch");
  return 0;
  API_END(-1)
}

int bc_gru_backward(int T, int B, int H, int ndir, const float* w_hh_t, const float* y, const float* rsv, const float* dy,
                    float* dgx, float* dgh, float* workspace, unsigned* sync, unsigned* status, double timeout_s, void* stream) {
  API_BEGIN
  NvtxRange range("bcoll.gru_backward");
  gpu::GruDims d{T, B, H, ndir};
  check_cuda(gpu::gru_persistent_backward(d, w_hh_t, y, rsv, dy, dgx, dgh, workspace, sync, status, timeout_s, (cudaStream_t)stream),
             "persistent GRU backward launch");
  return 0;
  API_END(-1)
}

// ---- batch normalisation fused with the clipped ReLU ---------------------------------------------

int bc_bn_clip_forward(const float* x, float* y, const float* gamma, const float* beta, float* running_mean, float* running_var,
                       float* save_mean, float* save_rstd, double* acc, int N, int C, int HW, float eps, float momentum, float clip_hi,
                       void* stream) {
  API_BEGIN
  check_cuda(gpu::bn_clip_forward(x, y, gamma, beta, running_mean, running_var, save_mean, save_rstd, acc, N, C, HW, eps, momentum,
                                  clip_hi, (cudaStream_t)stream), "batch-norm + clip forward launch");
  return 0;
  API_END(-1)
}

int bc_bn_clip_backward(const float* x, const float* dy, const float* gamma, const float* beta, const float* save_mean,
                        const float* save_rstd, float* dx, float* dgamma, float* dbeta, double* acc, int N, int C, int HW,
                        float clip_hi, void* stream) {
  API_BEGIN
  check_cuda(gpu::bn_clip_backward(x, dy, gamma, beta, save_mean, save_rstd, dx, dgamma, dbeta, acc, N, C, HW, clip_hi,
                                   (cudaStream_t)stream), "batch-norm + clip backward launch");
  return 0;
  API_END(-1)
}

// ---- wire-format helpers exposed for unit tests ------------------------------------------------------

int bc_test_validate(int nranks, const int* ops, const int* dtypes, const int* devices, const int* ndims,
                     const long long* shapes /* nranks x 8 */, char* err_out, int err_cap, long long* dim0_out) {
  API_BEGIN
  std::vector<Request> reqs(nranks);
  for (int r = 0; r < nranks; r++) {
    reqs[r].rank = r;
    reqs[r].op = (OpType)ops[r];
    reqs[r].dtype = (DType)dtypes[r];
    reqs[r].device = (DeviceKind)devices[r];
    reqs[r].name = "t";
    reqs[r].shape.assign(shapes + r * 8, shapes + r * 8 + ndims[r]);
    // round trip through the encoder, as on the wire
    reqs[r] = decode_request(encode(reqs[r]));
  }
  Response resp = decode_response(encode(build_response("t", reqs)));
  if (err_out && err_cap > 0) {
    strncpy(err_out, resp.error.c_str(), (size_t)err_cap - 1);
    err_out[err_cap - 1] = 0;
  }
  if (dim0_out)
    for (size_t i = 0; i < resp.dim0.size(); i++) dim0_out[i] = resp.dim0[i];
  return (int)resp.type;
  API_END(-1)
}

}  // extern "C"
