// Two-level view of a job whose ranks sit on several hosts: the ranks of one host form a node
// group (a control star centred on the host's lowest rank), and the ranks that have the same
// local rank on every host form a rail (a ring of data sockets over the hosts).
//
// The reference reaches several hosts through MPI: its GPU ring passes device buffers to a
// CUDA-aware MPI (tensorflow/contrib/mpi_collectives/ring.h:183-225) and the local
// communicator comes from MPI_Comm_split_type(SHARED) (mpi_ops.cc:609-613). Here the NVLink
// kernels reduce inside a host and each rail carries 1 / local_size of the tensor between hosts.
#pragma once

#include <string>
#include <vector>

#include "bootstrap.h"

namespace bc {

struct NodeGroup {
  int node_index = 0;            // hosts are numbered by their lowest rank
  int n_nodes = 1;
  int local_rank = 0;
  int local_size = 1;
  std::vector<int> members;      // global ranks of this host, ascending; members[local_rank] = this rank
  // Leader (local rank 0): star[i] is the socket to local rank i. Others: star[0] is the socket
  // to the leader.
  std::vector<Socket> star;
  // Ring over the hosts among the ranks with this local rank. Shaped like the job-wide transport
  // (rank = node_index, size = n_nodes, ring_next / ring_prev) so that the CPU ring algorithms
  // run on it unchanged.
  Transport rail;

  // Allgather of small blobs among the ranks of this host; every member must call it in the
  // same order.
  std::vector<std::string> allgather(const std::string& mine, double deadline);
};

// True when the job's hosts all run the same number of ranks (what the rails need).
bool hosts_are_uniform(const Transport& t, std::string* why);

// Collective over ALL ranks of the job, on the control star, before a background thread owns
// the sockets. Needs more than one host and uniform hosts.
NodeGroup build_node_group(Transport& t, double deadline);

}  // namespace bc
