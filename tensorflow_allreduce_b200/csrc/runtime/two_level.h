// Allreduce of a job that spans several hosts, in two levels:
//   1. the ranks of a host reduce the tensor among themselves (on GPUs: the NVLink kernels);
//   2. the tensor is cut into local_size slices, and local rank j reduces slice j with the ranks
//      of local rank j on the other hosts over its rail (a ring over the hosts), applying the
//      averaging there;
//   3. the ranks of a host gather the finished slices from one another.
// Every rank moves 2 * (n_nodes - 1) / n_nodes / local_size of the tensor between hosts, against
// 2 * (size - 1) / size of it in the reference's single ring over all ranks
// (tensorflow/contrib/mpi_collectives/ring.h:130-133).
//
// The levels inside a host are behind an interface: the runtime implements it with the GPU
// communicator, `ShmLocalLevel` with the host's shared-memory group (CPU tensors), and
// `HostLocalLevel` with the node group's control sockets (a slow stand-in for tests).
#pragma once

#include <algorithm>
#include <vector>

#include "../common.h"
#include "../control/node_group.h"

namespace bc {

class LocalLevel {
 public:
  virtual ~LocalLevel() {}
  // The tensor (count elements) becomes its reduction over the ranks of this host, unscaled.
  virtual void reduce_in_node(size_t count, DType dtype, ReduceOp red) = 0;
  // Copy elements [begin, begin + len) of the tensor into host memory at `dst`; complete on return.
  virtual void fetch(void* dst, size_t begin, size_t len, DType dtype) = 0;
  // `src` (host memory, len elements) is this rank's finished slice; slice i of the tensor has
  // slice_len[i] elements. On return of `finish` the tensor holds all slices (on a GPU: the work
  // is queued on the communicator's stream).
  virtual void finish(const void* src, size_t begin, size_t len, const std::vector<size_t>& slice_len, DType dtype) = 0;
};

// Element range of slice i when `count` elements are cut into n slices as evenly as possible
// (the first count % n slices get one element more): the same rule as the ring's segments.
inline size_t slice_begin(size_t count, int n, int i) { return (size_t)i * (count / n) + std::min<size_t>((size_t)i, count % n); }
inline size_t slice_len(size_t count, int n, int i) { return count / n + ((size_t)i < count % n ? 1 : 0); }

// `staging` must hold slice_len(count, local_size, 0) elements. Runs on the thread that owns the
// rail's sockets.
// `seconds`, if given, receives the host time spent in the three steps (inside the host, over the
// rail, back inside the host; on GPUs the last two include only what the host waits for).
void two_level_allreduce(NodeGroup& g, LocalLevel& local, void* staging, size_t count, DType dtype, double scale,
                         int64_t int_divisor, ReduceOp red, double deadline, double* seconds = nullptr);

// The same three steps for a CPU tensor, chunk by chunk, with the step over the rail on a helper
// thread: while chunk c travels between the hosts, this thread reduces chunk c + 1 inside the
// host and gathers chunk c - 1. Every rank of the job runs the same schedule, so the collectives
// of the shared-memory group and of the rail come in the same order everywhere.
// `staging` must hold two slices of a chunk: 2 * slice_len(chunk_elems, local_size, 0) elements.
// `seconds`: time this thread spent inside the host before a chunk could leave, waiting for the
// rail, and gathering.
class ShmGroup;
void two_level_allreduce_pipelined(NodeGroup& g, ShmGroup& shm, void* tensor, void* staging, size_t count, size_t chunk_elems,
                                   DType dtype, double scale, int64_t int_divisor, ReduceOp red, double deadline,
                                   double* seconds = nullptr);

// The levels inside a host for CPU tensors: the host's shared-memory group.
class ShmLocalLevel : public LocalLevel {
 public:
  ShmLocalLevel(ShmGroup& shm, void* tensor, double deadline) : shm_(shm), t_((char*)tensor), deadline_(deadline) {}
  void reduce_in_node(size_t count, DType dtype, ReduceOp red) override;
  void fetch(void* dst, size_t begin, size_t len, DType dtype) override;
  void finish(const void* src, size_t begin, size_t len, const std::vector<size_t>& slice_len, DType dtype) override;

 private:
  ShmGroup& shm_;
  char* t_;
  double deadline_;
};

// Host-memory stand-in for the levels inside a host: blobs through the node group's star.
class HostLocalLevel : public LocalLevel {
 public:
  HostLocalLevel(NodeGroup& g, void* tensor, double deadline) : g_(g), t_((char*)tensor), deadline_(deadline) {}
  void reduce_in_node(size_t count, DType dtype, ReduceOp red) override;
  void fetch(void* dst, size_t begin, size_t len, DType dtype) override;
  void finish(const void* src, size_t begin, size_t len, const std::vector<size_t>& slice_len, DType dtype) override;

 private:
  NodeGroup& g_;
  char* t_;
  double deadline_;
};

}  // namespace bc
