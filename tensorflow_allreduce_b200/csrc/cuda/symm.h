// Symmetric memory: device buffers that every rank of the node maps into its own address space,
// so that kernels can load and store peers' memory directly over NVLink. This is what stands in
// for CUDA-aware MPI in the reference (which hands GPU pointers to MPI_Send / MPI_Recv,
// tensorflow/contrib/mpi_collectives/ring.h:183-225).
//
// A segment is created collectively. Preferred path: CUDA virtual-memory-management allocation
// exported as a POSIX file descriptor and passed to the peers over unix sockets (SCM_RIGHTS);
// with it an NVLS multicast object can be bound to the segment so that multimem.ld_reduce /
// multimem.st work on it. Fallback: cudaMalloc + CUDA IPC handles (no multicast).
#pragma once

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "../common.h"
#include "../control/bootstrap.h"
#include "layout.h"

namespace bc {
namespace gpu {

struct Segment {
  int id = -1;
  size_t size = 0;
  char* local = nullptr;                    // this rank's memory
  char* peer[dev::kMaxRanks] = {nullptr};   // every rank's memory as mapped here (peer[rank] == local)
  char* mc = nullptr;                       // multicast mapping (NVLS) or null
  bool vmm = false;
  // bookkeeping for release
  unsigned long long handles[dev::kMaxRanks] = {0};
  unsigned long long mc_handle = 0;
  size_t mc_size = 0;
};

// Host-side allgather of small blobs; every rank calls it in the same order.
using HostAllgather = std::function<std::vector<std::string>(const std::string&)>;

class SymmAllocator {
 public:
  enum class Mode { AUTO, VMM, IPC };
  SymmAllocator(int rank, int world, int device, uint64_t job_id, Mode mode, bool want_multicast, double timeout_s);
  ~SymmAllocator();

  // Collective. Contents are zero-filled. Throws on failure (on every rank alike).
  Segment* alloc(size_t bytes, const HostAllgather& ag);
  void release_all();

  const std::vector<std::unique_ptr<Segment>>& segments() const { return segs_; }
  // Segment that fully contains [p, p + bytes), or null.
  Segment* find(const void* p, size_t bytes) const;
  bool multicast_available() const { return mc_ok_; }
  bool using_vmm() const { return use_vmm_; }
  std::string describe() const;

 private:
  bool alloc_vmm(Segment* s, size_t bytes, const HostAllgather& ag, std::string* why);
  void alloc_ipc(Segment* s, size_t bytes, const HostAllgather& ag);
  bool bind_multicast(Segment* s, const HostAllgather& ag, std::string* why);

  int rank_, world_, device_;
  uint64_t job_id_;
  bool use_vmm_ = false;
  bool mc_ok_ = false;
  bool want_mc_ = false;
  bool decided_ = false;
  Mode mode_;
  double timeout_s_;
  Socket fd_listener_;
  std::vector<std::unique_ptr<Segment>> segs_;
};

}  // namespace gpu
}  // namespace bc
