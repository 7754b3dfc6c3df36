#include "node_group.h"

#include <string.h>

#include <algorithm>
#include <map>

namespace bc {

namespace {

// hosts in the order of their lowest rank, each with its ranks ascending
std::vector<std::vector<int>> ranks_by_host(const Transport& t) {
  std::vector<std::vector<int>> nodes;
  std::map<std::string, int> index;
  for (int r = 0; r < t.size; r++) {
    auto it = index.find(t.hosts[r]);
    if (it == index.end()) {
      it = index.emplace(t.hosts[r], (int)nodes.size()).first;
      nodes.emplace_back();
    }
    nodes[it->second].push_back(r);
  }
  return nodes;
}

std::string pack(const std::vector<std::string>& v) {
  std::string s;
  for (const auto& e : v) {
    uint32_t n = (uint32_t)e.size();
    s.append((const char*)&n, 4);
    s.append(e);
  }
  return s;
}

std::vector<std::string> unpack(const std::string& s, size_t count) {
  std::vector<std::string> v;
  size_t p = 0;
  for (size_t i = 0; i < count; i++) {
    BC_CHECK(p + 4 <= s.size(), "short node-group message");
    uint32_t n;
    memcpy(&n, &s[p], 4);
    p += 4;
    BC_CHECK(p + n <= s.size(), "short node-group message");
    v.push_back(s.substr(p, n));
    p += n;
  }
  return v;
}

}  // namespace

bool hosts_are_uniform(const Transport& t, std::string* why) {
  auto nodes = ranks_by_host(t);
  for (size_t k = 1; k < nodes.size(); k++) {
    if (nodes[k].size() != nodes[0].size()) {
      if (why)
        *why = "host '" + t.hosts[nodes[0][0]] + "' runs " + std::to_string(nodes[0].size()) + " rank(s), host '" +
               t.hosts[nodes[k][0]] + "' runs " + std::to_string(nodes[k].size());
      return false;
    }
  }
  return true;
}

std::vector<std::string> NodeGroup::allgather(const std::string& mine, double deadline) {
  std::vector<std::string> all(local_size);
  if (local_size == 1) {
    all[0] = mine;
    return all;
  }
  if (local_rank == 0) {
    all[0] = mine;
    for (int i = 1; i < local_size; i++) all[i] = star[i].recv_frame(deadline);
    const std::string packed = pack(all);
    for (int i = 1; i < local_size; i++) star[i].send_frame(packed, deadline);
  } else {
    star[0].send_frame(mine, deadline);
    all = unpack(star[0].recv_frame(deadline), (size_t)local_size);
  }
  return all;
}

NodeGroup build_node_group(Transport& t, double deadline) {
  std::string why;
  BC_CHECK(hosts_are_uniform(t, &why), "the hosts of this job run different numbers of ranks (" << why << ")");
  const auto nodes = ranks_by_host(t);
  BC_CHECK(nodes.size() > 1, "all ranks are on one host; no node group is needed");

  NodeGroup g;
  g.n_nodes = (int)nodes.size();
  for (size_t k = 0; k < nodes.size(); k++)
    if (std::find(nodes[k].begin(), nodes[k].end(), t.rank) != nodes[k].end()) g.node_index = (int)k;
  g.members = nodes[g.node_index];
  g.local_size = (int)g.members.size();
  g.local_rank = (int)(std::find(g.members.begin(), g.members.end(), t.rank) - g.members.begin());
  g.star.resize(g.local_size);

  // The leader's unix listener and every rank's rail listener exist before anybody is told
  // about them: the allgather below is the barrier.
  Socket node_listener;
  if (g.local_rank == 0 && g.local_size > 1) node_listener = Socket::listen_unix(t.unix_name(t.rank, "node"), g.local_size + 4);
  int rail_port = 0;
  Socket rail_listener = Socket::listen_tcp("0.0.0.0", 0, 4, &rail_port);
  std::vector<std::string> ports = t.allgather(std::to_string(rail_port), deadline);

  // node star
  if (g.local_size > 1) {
    if (g.local_rank == 0) {
      for (int seen = 1; seen < g.local_size; seen++) {
        Socket s = node_listener.accept(deadline);
        int32_t who = -1;
        s.recv_all(&who, 4, deadline);
        BC_CHECK(who > 0 && who < g.local_size && !g.star[who].valid(), "unexpected member " << who << " on the node socket");
        g.star[who] = std::move(s);
      }
    } else {
      g.star[0] = Socket::connect_unix(t.unix_name(g.members[0], "node"), deadline);
      int32_t me = g.local_rank;
      g.star[0].send_all(&me, 4, deadline);
    }
  }

  // rail: the same local rank on the next host
  g.rail.rank = g.node_index;
  g.rail.size = g.n_nodes;
  g.rail.local_rank = 0;
  g.rail.local_size = 1;
  g.rail.job_id = t.job_id;
  const int next = nodes[(g.node_index + 1) % g.n_nodes][g.local_rank];
  const int prev = nodes[(g.node_index + g.n_nodes - 1) % g.n_nodes][g.local_rank];
  g.rail.ring_next = Socket::connect_tcp(t.ips[next], atoi(ports[next].c_str()), deadline);
  int32_t my = t.rank;
  g.rail.ring_next.send_all(&my, 4, deadline);
  g.rail.ring_prev = rail_listener.accept(deadline);
  int32_t from = -1;
  g.rail.ring_prev.recv_all(&from, 4, deadline);
  BC_CHECK(from == prev, "rail neighbour mismatch: expected rank " << prev << ", got " << from);
  t.barrier(deadline);
  return g;
}

}  // namespace bc
