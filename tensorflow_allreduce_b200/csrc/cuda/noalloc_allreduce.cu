// bc_group_allreduce_static: the group allreduce for callers that cannot allocate. See the header
// for the contract; this file owns the static scratch array and the per-device set-up.
#include "noalloc_allreduce.h"

#include <cuda_runtime.h>
#include <string.h>

#include <mutex>
#include <string>

#include "collectives.h"

namespace {

using namespace bc;
using namespace bc::dev;

constexpr size_t kStage = BC_STATIC_MAX_BYTES_PER_RANK;                   // staging copy of one rank's input
constexpr size_t kFlags = (size_t)kMaxBlocks * kMaxRanks * sizeof(uint32_t);  // barrier flags of one rank
constexpr size_t kEpochs = (size_t)kMaxBlocks * sizeof(uint32_t);          // barrier counters of one rank
constexpr size_t kCtlOff = BC_STATIC_MAX_RANKS * kStage;                   // flags and counters follow the staging areas
constexpr size_t kCtlBytes = BC_STATIC_MAX_RANKS * (kFlags + kEpochs) + 256;  // + a spare, unused word
constexpr size_t kScratchBytes = kCtlOff + kCtlBytes;
static_assert(kScratchBytes == BC_STATIC_SCRATCH_BYTES, "the header states another size of the static scratch");

// The scratch. In host code this name is only a handle for cudaGetSymbolAddress, never a pointer
// that a kernel could use.
static __device__ __align__(256) unsigned char g_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};
// Copies the reason into the caller's buffer (if any) and returns the failure code.
int fail(char* err, int err_cap, const std::string& why) {
  if (err && err_cap > 0) {
    strncpy(err, why.c_str(), (size_t)err_cap - 1);
    err[err_cap - 1] = 0;
  }
  return -1;
}

// Device address of g_scratch on the current device; looked up once per device.
unsigned char* scratch_for_current_device(std::string* why) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *why = std::string("cudaGetDevice: ") + cudaGetErrorString(e); return nullptr; }
  if (dev < 0 || dev >= kMaxDevices) { *why = "device ordinal out of range"; return nullptr; }
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_scratch);
    if (e != cudaSuccess || !p) {
      *why = std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e);
      return nullptr;
    }
    g_scratch_addr[dev] = (unsigned char*)p;
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int bc_group_allreduce_static(int nranks, const void* const* ins, void* const* outs, long long count, int dtype,
                                         float scale, int blocks, unsigned* status_out, void* stream, char* err,
                                         int err_cap) {
  if (err && err_cap > 0) err[0] = 0;
  if (nranks < 1 || nranks > BC_STATIC_MAX_RANKS)
    return fail(err, err_cap, "nranks must be between 1 and " + std::to_string(BC_STATIC_MAX_RANKS));
  if (!ins || !outs) return fail(err, err_cap, "ins and outs must not be null");
  const size_t es = dtype_size((DType)dtype);
  if (es == 0) return fail(err, err_cap, "unknown dtype code " + std::to_string(dtype));
  if (count < 0) return fail(err, err_cap, "count must not be negative");
  // Compared before the multiplication: count * es wraps around for counts near 2^62.
  if ((unsigned long long)count > kStage / es)
    return fail(err, err_cap, "request of " + std::to_string(count) + " elements of " + std::to_string(es) +
                " bytes per rank exceeds the static scratch limit of " + std::to_string(kStage) + " bytes per rank");
  const size_t bytes = (size_t)count * es;
  if (!status_out) return fail(err, err_cap, "status_out must not be null: it is the only place where a timed-out wait is reported");
  auto overlap = [bytes](const void* a, const void* b) {
    const uintptr_t x = (uintptr_t)a, y = (uintptr_t)b;
    return x < y + bytes && y < x + bytes;
  };
  for (int r = 0; r < nranks; r++) {
    if (!ins[r] || !outs[r]) return fail(err, err_cap, "null buffer for rank " + std::to_string(r));
    if ((((uintptr_t)ins[r] | (uintptr_t)outs[r]) & 15) != 0) return fail(err, err_cap, "buffers must be 16-byte aligned");
  }
  if (count == 0) return 0;
  for (int r = 0; r < nranks; r++) {
    for (int q = 0; q < nranks; q++) {
      if (overlap(outs[r], ins[q])) return fail(err, err_cap, "an output aliases an input (their byte ranges overlap)");
      if (q != r && overlap(outs[r], outs[q])) return fail(err, err_cap, "two outputs alias (their byte ranges overlap)");
    }
  }

  std::string why;
  unsigned char* base = scratch_for_current_device(&why);
  if (!base) return fail(err, err_cap, why);
  int dev = 0;
  cudaGetDevice(&dev);
  gpu::LaunchCfg cfg;
  cfg.cooperative = true;
  const int resident = gpu::max_emulated_blocks(dev, nranks, cfg.threads);
  if (blocks <= 0) blocks = resident < 4 ? resident : 4;
  if (blocks > resident || blocks > kMaxBlocks)
    return fail(err, err_cap, "blocks = " + std::to_string(blocks) + " per rank cannot be resident at once for " + std::to_string(nranks) +
                " ranks on this device (limit " + std::to_string(resident < kMaxBlocks ? resident : kMaxBlocks) + ")");

  cudaStream_t s = (cudaStream_t)stream;
  unsigned char* ctl = base + kCtlOff;
  // The array still holds the previous call's flags and counters: start from zero.
  cudaError_t e = cudaMemsetAsync(ctl, 0, kCtlBytes, s);
  if (e != cudaSuccess) return fail(err, err_cap, std::string("clearing the scratch: ") + cudaGetErrorString(e));
  e = cudaMemsetAsync(status_out, 0, sizeof(unsigned), s);
  if (e != cudaSuccess) return fail(err, err_cap, std::string("clearing status_out: ") + cudaGetErrorString(e));
  for (int r = 0; r < nranks; r++) {
    e = cudaMemcpyAsync(base + (size_t)r * kStage, ins[r], bytes, cudaMemcpyDeviceToDevice, s);
    if (e != cudaSuccess) return fail(err, err_cap, std::string("staging the input of rank ") + std::to_string(r) + ": " + cudaGetErrorString(e));
  }

  gpu::ArArgs a;
  memset(&a, 0, sizeof(a));
  a.nranks_here = nranks;
  a.algo = (int)gpu::Algo::TWO_SHOT;
  a.count = (size_t)count;
  a.scale = scale;
  a.idiv = 1;
  for (int r = 0; r < nranks; r++) {
    RankCtx& c = a.r[r].ctx;
    c.rank = r;
    c.world = nranks;
    for (int p = 0; p < nranks; p++) {
      c.flags[p] = (uint32_t*)(ctl + (size_t)p * kFlags);
      c.meta[p] = nullptr;  // only the allgather kernel exchanges metadata
      a.r[r].in[p] = (char*)(base + (size_t)p * kStage);
    }
    c.epochs = (uint32_t*)(ctl + BC_STATIC_MAX_RANKS * kFlags + (size_t)r * kEpochs);
    c.status = (uint32_t*)status_out;
    c.timeout_ns = 20ull * 1000 * 1000 * 1000;
    a.r[r].out = outs[r];
  }
  cfg.blocks = blocks;
  e = gpu::launch_allreduce(a, (DType)dtype, (DType)dtype, cfg, s);
  if (e != cudaSuccess) return fail(err, err_cap, std::string("launching the reduction: ") + cudaGetErrorString(e));
  return 0;
}
