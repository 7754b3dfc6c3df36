#include "bootstrap.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <random>

namespace bc {

namespace {

struct Buf {
  std::string s;
  void i32(int32_t v) { s.append((const char*)&v, 4); }
  void u64(uint64_t v) { s.append((const char*)&v, 8); }
  void str(const std::string& v) { i32((int32_t)v.size()); s.append(v); }
};
struct Rd {
  const std::string& s;
  size_t p = 0;
  explicit Rd(const std::string& in) : s(in) {}
  int32_t i32() { BC_CHECK(p + 4 <= s.size(), "short bootstrap message"); int32_t v; memcpy(&v, &s[p], 4); p += 4; return v; }
  uint64_t u64() { BC_CHECK(p + 8 <= s.size(), "short bootstrap message"); uint64_t v; memcpy(&v, &s[p], 8); p += 8; return v; }
  std::string str() { int32_t n = i32(); BC_CHECK(n >= 0 && p + (size_t)n <= s.size(), "short bootstrap message"); std::string v = s.substr(p, n); p += n; return v; }
};

// Bumped whenever a control message or the bootstrap exchange changes its layout.
constexpr int32_t kWireVersion = 3;

std::string peer_ip(int fd) {
  struct sockaddr_in sa;
  socklen_t sl = sizeof(sa);
  if (getpeername(fd, (struct sockaddr*)&sa, &sl) != 0) return "127.0.0.1";
  char buf[64];
  if (!inet_ntop(AF_INET, &sa.sin_addr, buf, sizeof(buf))) return "127.0.0.1";
  return buf;
}

}  // namespace

std::string Transport::unix_name(int r, const char* purpose) const {
  char buf[128];
  snprintf(buf, sizeof(buf), "bcoll-%016llx-%s-%d", (unsigned long long)job_id, purpose, r);
  return buf;
}

std::vector<std::string> Transport::allgather(const std::string& mine, double deadline) {
  std::vector<std::string> all(size);
  if (size == 1) {
    all[0] = mine;
    return all;
  }
  if (rank == 0) {
    all[0] = mine;
    for (int r = 1; r < size; r++) all[r] = ctrl[r].recv_frame(deadline);
    Buf b;
    for (int r = 0; r < size; r++) b.str(all[r]);
    for (int r = 1; r < size; r++) ctrl[r].send_frame(b.s, deadline);
  } else {
    ctrl[0].send_frame(mine, deadline);
    std::string packed = ctrl[0].recv_frame(deadline);
    Rd rd(packed);
    for (int r = 0; r < size; r++) all[r] = rd.str();
  }
  return all;
}

void Transport::barrier(double deadline) { allgather(std::string(), deadline); }

Transport bootstrap(int rank, int size, const std::string& addr, int port, double timeout_s, const std::string& host) {
  BC_CHECK(size >= 1 && rank >= 0 && rank < size, "bad rank/size: " << rank << "/" << size);
  Transport t;
  t.rank = rank;
  t.size = size;
  t.hosts.assign(size, "");
  t.pids.assign(size, 0);
  t.ctrl.resize(size);
  const std::string me = host.empty() ? local_hostname() : host;
  if (size == 1) {
    t.hosts[0] = me;
    t.ips.assign(1, addr);
    t.pids[0] = (int)getpid();
    std::random_device rd;
    t.job_id = ((uint64_t)rd() << 32) ^ rd();
    return t;
  }
  const double deadline = now_s() + timeout_s;

  // Rank 0 binds the rendezvous port before anything of this process asks the kernel for a port
  // of its own choice: a port from the ephemeral range could otherwise go to the data listener.
  Socket listener;
  if (rank == 0) {
    int bound = 0;
    listener = Socket::listen_tcp("0.0.0.0", port, size + 8, &bound);
  }
  int data_port = 0;
  Socket data_listener = Socket::listen_tcp("0.0.0.0", 0, 8, &data_port);

  std::vector<std::string> ips(size);
  std::vector<int> data_ports(size, 0);

  if (rank == 0) {
    t.hosts[0] = me;
    t.pids[0] = (int)getpid();
    ips[0] = addr;
    data_ports[0] = data_port;
    std::random_device rdev;
    t.job_id = ((uint64_t)rdev() << 32) ^ rdev();
    int seen = 1;
    while (seen < size) {
      Socket s = listener.accept(deadline);
      std::string hello = s.recv_frame(deadline);
      Rd rd(hello);
      int32_t magic = rd.i32();
      BC_CHECK(magic == 0x42434F4C, "unexpected client on the bootstrap port");
      int32_t version = rd.i32();
      BC_CHECK(version == kWireVersion, "a rank runs another version of this library (message format " << version
               << ", rank 0 has " << kWireVersion << ")");
      int32_t r = rd.i32();
      int32_t sz = rd.i32();
      BC_CHECK(sz == size, "rank " << r << " was started with world size " << sz << ", rank 0 with " << size);
      BC_CHECK(r > 0 && r < size, "bootstrap hello from out-of-range rank " << r);
      BC_CHECK(!t.ctrl[r].valid(), "two processes claim rank " << r);
      t.hosts[r] = rd.str();
      data_ports[r] = rd.i32();
      t.pids[r] = rd.i32();
      ips[r] = peer_ip(s.fd());
      t.ctrl[r] = std::move(s);
      seen++;
    }
    Buf b;
    b.u64(t.job_id);
    for (int r = 0; r < size; r++) {
      b.str(t.hosts[r]);
      b.str(ips[r]);
      b.i32(data_ports[r]);
      b.i32(t.pids[r]);
    }
    for (int r = 1; r < size; r++) t.ctrl[r].send_frame(b.s, deadline);
  } else {
    Socket s = Socket::connect_tcp(addr, port, deadline);
    Buf b;
    b.i32(0x42434F4C);
    b.i32(kWireVersion);
    b.i32(rank);
    b.i32(size);
    b.str(me);
    b.i32(data_port);
    b.i32((int32_t)getpid());
    s.send_frame(b.s, deadline);
    std::string table = s.recv_frame(deadline);
    Rd rd(table);
    t.job_id = rd.u64();
    for (int r = 0; r < size; r++) {
      t.hosts[r] = rd.str();
      ips[r] = rd.str();
      data_ports[r] = rd.i32();
      t.pids[r] = rd.i32();
    }
    ips[0] = addr;  // rank 0 is reachable where we just reached it
    t.ctrl[0] = std::move(s);
  }

  t.local_rank = 0;
  t.local_size = 0;
  for (int r = 0; r < size; r++) {
    if (t.hosts[r] == t.hosts[rank]) {
      if (r < rank) t.local_rank++;
      t.local_size++;
    }
  }

  t.ips = ips;

  // Data ring: connect to the next rank, accept from the previous one.
  const int next = (rank + 1) % size;
  t.ring_next = Socket::connect_tcp(ips[next], data_ports[next], deadline);
  int32_t my = rank;
  t.ring_next.send_all(&my, 4, deadline);
  t.ring_prev = data_listener.accept(deadline);
  int32_t from = -1;
  t.ring_prev.recv_all(&from, 4, deadline);
  BC_CHECK(from == (rank - 1 + size) % size, "ring neighbour mismatch: expected " << (rank - 1 + size) % size << " got " << from);
  t.barrier(deadline);
  return t;
}

}  // namespace bc
