// Deadline-aware stream sockets (TCP and abstract unix-domain) for the control plane
// and the CPU data plane. This layer stands where the reference uses MPI point-to-point
// calls (tensorflow/contrib/mpi_collectives/mpi_ops.cc:666-771, ring.h:183-225): every
// blocking receive here has a deadline, so a missing peer yields an error, not a hang.
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../common.h"

namespace bc {

class Socket {
 public:
  Socket() = default;
  explicit Socket(int fd) : fd_(fd) {}
  Socket(const Socket&) = delete;
  Socket& operator=(const Socket&) = delete;
  Socket(Socket&& o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
  Socket& operator=(Socket&& o) noexcept;
  ~Socket() { close(); }

  int fd() const { return fd_; }
  bool valid() const { return fd_ >= 0; }
  void close();

  // Blocking with a deadline (seconds, steady clock as returned by now_s()); throw CommLost
  // on EOF, error or expiry.
  void send_all(const void* buf, size_t n, double deadline) const;
  void recv_all(void* buf, size_t n, double deadline) const;

  // Length-prefixed frame: u32 little-endian byte count, then the payload. A zero-length
  // payload and payloads containing zero bytes are both legal.
  void send_frame(const std::string& payload, double deadline) const;
  std::string recv_frame(double deadline) const;

  // Pass an open file descriptor across a unix-domain socket (SCM_RIGHTS) with a 4-byte tag.
  void send_fd(int fd_to_send, int32_t tag, double deadline) const;
  int recv_fd(int32_t* tag, double deadline) const;

  // TCP
  static Socket listen_tcp(const std::string& addr, int port, int backlog, int* bound_port);
  static Socket connect_tcp(const std::string& addr, int port, double deadline);
  // Abstract-namespace unix socket (no file on disk).
  static Socket listen_unix(const std::string& name, int backlog);
  static Socket connect_unix(const std::string& name, double deadline);
  Socket accept(double deadline) const;

 private:
  int fd_ = -1;
};

// Send `sn` bytes on `out` while receiving `rn` bytes from `in`, interleaved through poll(),
// so that two neighbours exchanging large segments cannot block each other (the role of
// MPI_Sendrecv in the reference's ring, ring.h:221,293).
void send_recv(const Socket& out, const void* sbuf, size_t sn,
               const Socket& in, void* rbuf, size_t rn, double deadline);

std::string local_hostname();

}  // namespace bc
