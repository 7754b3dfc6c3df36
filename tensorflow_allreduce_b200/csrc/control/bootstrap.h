// Process-group bootstrap over TCP: the part of the reference done by MPI_Init,
// MPI_Comm_rank/size and MPI_Comm_split_type(SHARED)
// (tensorflow/contrib/mpi_collectives/mpi_ops.cc:588-613).
//
// Rank 0 listens on (addr, port). Every other rank connects, announces itself, and receives the
// table of all ranks. The result is a star of control sockets centred on rank 0 plus a ring of
// data sockets (rank r -> r+1) used by the CPU collectives. local_rank is the number of lower
// ranks on the same host.
#pragma once

#include <string>
#include <vector>

#include "socket.h"

namespace bc {

struct Transport {
  int rank = 0;
  int size = 1;
  int local_rank = 0;
  int local_size = 1;
  uint64_t job_id = 0;
  std::vector<std::string> hosts;  // hostname of every rank
  std::vector<std::string> ips;    // address at which every rank's listeners can be reached
  std::vector<int> pids;
  // Control star. On rank 0: ctrl[r] is the socket to rank r (ctrl[0] unused). On other ranks:
  // ctrl[0] is the socket to rank 0.
  std::vector<Socket> ctrl;
  Socket ring_next;  // to (rank + 1) % size
  Socket ring_prev;  // from (rank - 1 + size) % size

  // Host-side collectives on the control star, for use while no background thread owns the
  // sockets (set-up and tear-down). Every rank must call them in the same order.
  std::vector<std::string> allgather(const std::string& mine, double deadline);
  void barrier(double deadline);
  // Name of this job's abstract unix socket for `r` (descriptor passing between local ranks).
  std::string unix_name(int r, const char* purpose) const;
};

// `host` = the host name this rank reports (empty: local_hostname()).
Transport bootstrap(int rank, int size, const std::string& addr, int port, double timeout_s, const std::string& host = std::string());

}  // namespace bc
