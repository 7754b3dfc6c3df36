// CPU collectives among the ranks of ONE host through a shared-memory segment: the role that the
// MPI library's shared-memory transport plays for the reference's ring when all of its ranks run
// on one machine (tensorflow/contrib/mpi_collectives/ring.h:183-225 issues the same MPI calls
// either way). The socket ring (ring.h in this directory) stays the path between hosts.
//
// Layout of the segment: a header with a barrier, one slot per rank and one result area. An
// allreduce works in chunks of one slot: every rank copies its chunk into its slot; after a
// barrier rank r reduces slice r of the chunk over all slots (always in slot order, so the
// result does not depend on timing) into the result area; after a second barrier every rank
// copies the result out. Each rank touches about 3 x the tensor in memory and sends nothing
// through the kernel's socket layer. Every wait has a deadline; a rank that never arrives makes
// the others throw CommLost.
#pragma once

#include <atomic>
#include <functional>
#include <string>
#include <vector>

#include "../common.h"

namespace bc {

class ShmGroup {
 public:
  using Allgather = std::function<std::vector<std::string>(const std::string&)>;

  // Collective over the `local_size` ranks of the host. `name` must be unique to this job and
  // host; `ag` gathers a small blob among exactly these ranks (used during set-up only).
  // `peer_lost`, if given, is asked every few milliseconds of a long wait; a non-empty answer (why
  // a peer is known to be gone) ends the wait on every rank of the group.
  using PeerLost = std::function<std::string()>;
  ShmGroup(int local_rank, int local_size, const std::string& name, size_t slot_bytes, const Allgather& ag,
           const PeerLost& peer_lost = PeerLost());
  ~ShmGroup();
  ShmGroup(const ShmGroup&) = delete;
  ShmGroup& operator=(const ShmGroup&) = delete;

  // `in` and `out` may be the same buffer; they must not overlap otherwise.
  void allreduce(const void* in, void* out, size_t count, DType dtype, double scale, int64_t int_divisor, ReduceOp red, double deadline);
  void allreduce(void* data, size_t count, DType dtype, double scale, int64_t int_divisor, ReduceOp red, double deadline) {
    allreduce(data, data, count, dtype, scale, int_divisor, red, deadline);
  }
  void allgatherv(const void* in, void* out, const std::vector<int64_t>& rows, size_t row_bytes, double deadline);
  size_t slot_bytes() const { return slot_bytes_; }

 private:
  struct Header {
    std::atomic<uint32_t> arrived;
    std::atomic<uint32_t> generation;
    std::atomic<uint32_t> broken;     // set by a rank whose wait ran out, so that the others stop waiting too
  };
  void barrier(double deadline);
  char* slot(int r) const { return base_ + kHeaderBytes + (size_t)r * slot_bytes_; }
  char* result() const { return slot(n_); }

  static constexpr size_t kHeaderBytes = 4096;
  int r_, n_;
  PeerLost peer_lost_;
  size_t slot_bytes_;
  size_t map_bytes_ = 0;
  char* base_ = nullptr;
  Header* hdr_ = nullptr;
};

}  // namespace bc
