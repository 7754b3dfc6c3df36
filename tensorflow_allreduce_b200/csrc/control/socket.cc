#include "socket.h"

#include <stdlib.h>

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <thread>

namespace bc {

namespace {

int remaining_ms(double deadline) {
  double r = deadline - now_s();
  if (r <= 0) return 0;
  if (r > 3600) r = 3600;
  return (int)(r * 1000.0) + 1;
}

void set_nonblocking(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  if (on) fl |= O_NONBLOCK; else fl &= ~O_NONBLOCK;
  fcntl(fd, F_SETFL, fl);
}

void wait_fd(int fd, short events, double deadline, const char* what) {
  for (;;) {
    struct pollfd p { fd, events, 0 };
    int ms = remaining_ms(deadline);
    int rc = ::poll(&p, 1, ms);
    if (rc > 0) return;
    if (rc == 0) {
      if (now_s() >= deadline) throw CommLost(std::string("timed out in ") + what);
      continue;
    }
    if (errno == EINTR) continue;
    throw CommLost(std::string("poll failed in ") + what + ": " + strerror(errno));
  }
}

}  // namespace

Socket& Socket::operator=(Socket&& o) noexcept {
  if (this != &o) {
    close();
    fd_ = o.fd_;
    o.fd_ = -1;
  }
  return *this;
}

void Socket::close() {
  if (fd_ >= 0) {
    ::close(fd_);
    fd_ = -1;
  }
}

void Socket::send_all(const void* buf, size_t n, double deadline) const {
  const char* p = (const char*)buf;
  while (n > 0) {
    ssize_t k = ::send(fd_, p, n, MSG_NOSIGNAL | MSG_DONTWAIT);
    if (k > 0) { p += k; n -= (size_t)k; continue; }
    if (k < 0 && (errno == EAGAIN || errno == EWOULDBLOCK)) { wait_fd(fd_, POLLOUT, deadline, "send"); continue; }
    if (k < 0 && errno == EINTR) continue;
    throw CommLost(std::string("send failed: ") + (k == 0 ? "closed" : strerror(errno)));
  }
}

void Socket::recv_all(void* buf, size_t n, double deadline) const {
  char* p = (char*)buf;
  while (n > 0) {
    ssize_t k = ::recv(fd_, p, n, MSG_DONTWAIT);
    if (k > 0) { p += k; n -= (size_t)k; continue; }
    if (k == 0) throw CommLost("connection closed by peer");
    if (errno == EAGAIN || errno == EWOULDBLOCK) { wait_fd(fd_, POLLIN, deadline, "recv"); continue; }
    if (errno == EINTR) continue;
    throw CommLost(std::string("recv failed: ") + strerror(errno));
  }
}

void Socket::send_frame(const std::string& payload, double deadline) const {
  uint32_t len = (uint32_t)payload.size();
  std::string buf;
  buf.resize(4 + payload.size());
  memcpy(&buf[0], &len, 4);
  if (len) memcpy(&buf[4], payload.data(), len);
  send_all(buf.data(), buf.size(), deadline);
}

std::string Socket::recv_frame(double deadline) const {
  uint32_t len = 0;
  recv_all(&len, 4, deadline);
  BC_CHECK(len <= (1u << 30), "control frame too large: " << len);
  std::string s(len, '\0');
  if (len) recv_all(&s[0], len, deadline);
  return s;
}

void Socket::send_fd(int fd_to_send, int32_t tag, double deadline) const {
  struct msghdr msg;
  memset(&msg, 0, sizeof(msg));
  struct iovec iov { &tag, sizeof(tag) };
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd_to_send, sizeof(int));
  for (;;) {
    wait_fd(fd_, POLLOUT, deadline, "send_fd");
    ssize_t k = ::sendmsg(fd_, &msg, MSG_NOSIGNAL);
    if (k == (ssize_t)sizeof(tag)) return;
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    throw CommLost(std::string("sendmsg(SCM_RIGHTS) failed: ") + strerror(errno));
  }
}

int Socket::recv_fd(int32_t* tag, double deadline) const {
  for (;;) {
    wait_fd(fd_, POLLIN, deadline, "recv_fd");
    struct msghdr msg;
    memset(&msg, 0, sizeof(msg));
    int32_t t = 0;
    struct iovec iov { &t, sizeof(t) };
    msg.msg_iov = &iov;
    msg.msg_iovlen = 1;
    char ctrl[CMSG_SPACE(sizeof(int))];
    msg.msg_control = ctrl;
    msg.msg_controllen = sizeof(ctrl);
    ssize_t k = ::recvmsg(fd_, &msg, MSG_CMSG_CLOEXEC);
    if (k < 0 && (errno == EINTR || errno == EAGAIN)) continue;
    if (k <= 0) throw CommLost("recvmsg(SCM_RIGHTS) failed or peer closed");
    struct cmsghdr* c = CMSG_FIRSTHDR(&msg);
    if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS)
      throw CommLost("recvmsg: no descriptor attached");
    int fd;
    memcpy(&fd, CMSG_DATA(c), sizeof(int));
    if (tag) *tag = t;
    return fd;
  }
}

Socket Socket::listen_tcp(const std::string& addr, int port, int backlog, int* bound_port) {
  int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  BC_CHECK(fd >= 0, "socket(): " << strerror(errno));
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  struct sockaddr_in sa;
  memset(&sa, 0, sizeof(sa));
  sa.sin_family = AF_INET;
  sa.sin_port = htons((uint16_t)port);
  sa.sin_addr.s_addr = htonl(INADDR_ANY);
  if (!addr.empty() && addr != "0.0.0.0") {
    if (inet_pton(AF_INET, addr.c_str(), &sa.sin_addr) != 1) sa.sin_addr.s_addr = htonl(INADDR_ANY);
  }
  if (::bind(fd, (struct sockaddr*)&sa, sizeof(sa)) != 0) {
    int e = errno;
    ::close(fd);
    throw Error(std::string("bind(") + addr + ":" + std::to_string(port) + "): " + strerror(e));
  }
  if (::listen(fd, backlog) != 0) {
    int e = errno;
    ::close(fd);
    throw Error(std::string("listen(): ") + strerror(e));
  }
  if (bound_port) {
    socklen_t sl = sizeof(sa);
    getsockname(fd, (struct sockaddr*)&sa, &sl);
    *bound_port = ntohs(sa.sin_port);
  }
  return Socket(fd);
}

Socket Socket::connect_tcp(const std::string& addr, int port, double deadline) {
  // Resolve once; retry the connect until the deadline, since the listener may not be up yet.
  struct addrinfo hints;
  memset(&hints, 0, sizeof(hints));
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  struct addrinfo* res = nullptr;
  std::string portstr = std::to_string(port);
  int grc = getaddrinfo(addr.c_str(), portstr.c_str(), &hints, &res);
  BC_CHECK(grc == 0 && res, "cannot resolve " << addr << ": " << gai_strerror(grc));
  std::string last = "no attempt";
  for (;;) {
    int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd >= 0) {
      if (::connect(fd, res->ai_addr, res->ai_addrlen) == 0) {
        // While nobody listens on a local port of the ephemeral range yet, the kernel may give
        // this socket that very port as its source and complete a TCP simultaneous open with
        // itself. Such a socket also keeps the real listener from binding: drop it and retry.
        struct sockaddr_in self, peer;
        socklen_t sl = sizeof(self), pl = sizeof(peer);
        if (getsockname(fd, (struct sockaddr*)&self, &sl) == 0 && getpeername(fd, (struct sockaddr*)&peer, &pl) == 0 &&
            self.sin_port == peer.sin_port && self.sin_addr.s_addr == peer.sin_addr.s_addr) {
          last = "connected to itself";
          ::close(fd);
          if (now_s() >= deadline) break;
          std::this_thread::sleep_for(std::chrono::milliseconds(20));
          continue;
        }
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
        freeaddrinfo(res);
        return Socket(fd);
      }
      last = strerror(errno);
      ::close(fd);
    }
    if (now_s() >= deadline) break;
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
  freeaddrinfo(res);
  throw CommLost("could not connect to " + addr + ":" + portstr + " before the deadline (" + last + ")");
}

static socklen_t fill_abstract(struct sockaddr_un* sa, const std::string& name) {
  memset(sa, 0, sizeof(*sa));
  sa->sun_family = AF_UNIX;
  size_t n = std::min(name.size(), sizeof(sa->sun_path) - 2);
  sa->sun_path[0] = '\0';
  memcpy(sa->sun_path + 1, name.data(), n);
  return (socklen_t)(offsetof(struct sockaddr_un, sun_path) + 1 + n);
}

Socket Socket::listen_unix(const std::string& name, int backlog) {
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  BC_CHECK(fd >= 0, "socket(AF_UNIX): " << strerror(errno));
  struct sockaddr_un sa;
  socklen_t len = fill_abstract(&sa, name);
  if (::bind(fd, (struct sockaddr*)&sa, len) != 0 || ::listen(fd, backlog) != 0) {
    int e = errno;
    ::close(fd);
    throw Error(std::string("unix listen '") + name + "': " + strerror(e));
  }
  return Socket(fd);
}

Socket Socket::connect_unix(const std::string& name, double deadline) {
  struct sockaddr_un sa;
  socklen_t len = fill_abstract(&sa, name);
  std::string last;
  for (;;) {
    int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd >= 0) {
      if (::connect(fd, (struct sockaddr*)&sa, len) == 0) return Socket(fd);
      last = strerror(errno);
      ::close(fd);
    }
    if (now_s() >= deadline) break;
    std::this_thread::sleep_for(std::chrono::milliseconds(10));
  }
  throw CommLost("could not connect to unix socket '" + name + "' (" + last + ")");
}

Socket Socket::accept(double deadline) const {
  for (;;) {
    wait_fd(fd_, POLLIN, deadline, "accept");
    int fd = ::accept4(fd_, nullptr, nullptr, SOCK_CLOEXEC);   // not inherited by programs a rank starts
    if (fd >= 0) {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));  // harmless on unix sockets
      return Socket(fd);
    }
    if (errno == EINTR || errno == EAGAIN) continue;
    throw CommLost(std::string("accept failed: ") + strerror(errno));
  }
}

void send_recv(const Socket& out, const void* sbuf, size_t sn,
               const Socket& in, void* rbuf, size_t rn, double deadline) {
  const char* sp = (const char*)sbuf;
  char* rp = (char*)rbuf;
  while (sn > 0 || rn > 0) {
    struct pollfd p[2];
    int n = 0, si = -1, ri = -1;
    if (sn > 0) { p[n] = { out.fd(), POLLOUT, 0 }; si = n++; }
    if (rn > 0) { p[n] = { in.fd(), POLLIN, 0 }; ri = n++; }
    int rc = ::poll(p, n, remaining_ms(deadline));
    if (rc < 0) {
      if (errno == EINTR) continue;
      throw CommLost(std::string("poll failed in send_recv: ") + strerror(errno));
    }
    if (rc == 0) {
      if (now_s() >= deadline) throw CommLost("timed out exchanging a ring segment with a neighbour");
      continue;
    }
    if (si >= 0 && (p[si].revents & (POLLOUT | POLLERR | POLLHUP))) {
      ssize_t k = ::send(out.fd(), sp, sn, MSG_NOSIGNAL | MSG_DONTWAIT);
      if (k > 0) { sp += k; sn -= (size_t)k; }
      else if (k < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)
        throw CommLost(std::string("ring send failed: ") + strerror(errno));
    }
    if (ri >= 0 && (p[ri].revents & (POLLIN | POLLERR | POLLHUP))) {
      ssize_t k = ::recv(in.fd(), rp, rn, MSG_DONTWAIT);
      if (k > 0) { rp += k; rn -= (size_t)k; }
      else if (k == 0) throw CommLost("ring neighbour closed the connection");
      else if (errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)
        throw CommLost(std::string("ring recv failed: ") + strerror(errno));
    }
  }
}

std::string local_hostname() {
  // BC_HOSTNAME overrides the name this rank reports: it decides which ranks count as one host
  // (local_rank / local_size), and lets a single machine stand in for several hosts in tests.
  if (const char* forced = getenv("BC_HOSTNAME"))
    if (forced[0]) return forced;
  char buf[256];
  if (gethostname(buf, sizeof(buf)) != 0) return "localhost";
  buf[255] = 0;
  return buf;
}

}  // namespace bc
