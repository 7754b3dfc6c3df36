// Host-side self-test of the control plane, the CPU ring and the runtime, meant to be built with
// -fsanitize=thread or -fsanitize=address: N ranks run as threads of ONE process, each with its
// own Runtime (own sockets, own background thread), on a CPU-only group. The reference has no
// sanitizer configuration at all and its global state has real data races
// (tensorflow/contrib/mpi_collectives/mpi_ops.cc:593,621,816-821).
//
//   host_selftest <nranks> <port> [<port2>]     exit code 0 = all checks passed
//   (with <port2>: a second pass with 4 ranks that report two host names)
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <thread>
#include <vector>

#include "../runtime/runtime.h"

using namespace bc;

static std::atomic<int> g_failures{0};
#define EXPECT(cond, ...)                                   \
  do {                                                      \
    if (!(cond)) {                                          \
      fprintf(stderr, "FAIL %s:%d: ", __FILE__, __LINE__);  \
      fprintf(stderr, __VA_ARGS__);                         \
      fprintf(stderr, "\n");                                \
      g_failures++;                                         \
    }                                                       \
  } while (0)

static void* alloc_cb(int64_t, int64_t rows, void* user, int* is_symm) {
  auto* v = (std::vector<float>*)user;
  v->assign((size_t)rows * 3, -1.f);
  *is_symm = 0;
  return v->data();
}

static int64_t enqueue_allreduce(Runtime& rt, const std::string& name, const float* in, float* out, std::vector<int64_t> shape,
                                 bool average, DType dt = DType::F32) {
  std::unique_ptr<OpRecord> r(new OpRecord());
  r->name = name;
  r->op = OpType::ALLREDUCE;
  r->dtype = dt;
  r->shape = shape;
  r->in = in;
  r->out = out;
  r->average = average;
  return rt.enqueue(std::move(r));
}

static void rank_main(int rank, int size, int port, std::string hostname) {
  try {
    RuntimeOptions o;
    o.rank = rank;
    o.size = size;
    o.port = port;
    o.hostname = hostname;
    o.device = -1;
    o.timeout_s = 3;
    Runtime rt(o);
    EXPECT(rt.rank() == rank && rt.size() == size, "rank/size");

    // many named allreduces in flight at once, enqueued in a rank-dependent order
    const int K = 16, n = 5000;   // 20 kB: several chunks when the shared-memory slots are small
    std::vector<std::vector<float>> in(K, std::vector<float>(n)), out(K, std::vector<float>(n));
    std::vector<int64_t> h(K);
    for (int k = 0; k < K; k++)
      for (int i = 0; i < n; i++) in[k][i] = (float)(rank + k + i % 7);
    for (int j = 0; j < K; j++) {
      int k = (j * 5 + rank * 3) % K;
      h[k] = enqueue_allreduce(rt, "t" + std::to_string(k), in[k].data(), out[k].data(), {n}, false);
    }
    for (int k = 0; k < K; k++) {
      rt.wait(h[k], 30);
      rt.release(h[k]);
      float want = 0;
      for (int r = 0; r < size; r++) want += (float)(r + k + 3);
      EXPECT(out[k][3] == want, "allreduce t%d: got %f want %f", k, out[k][3], want);
    }

    // variable allgather: rank r contributes r+1 rows of 3
    std::vector<float> mine((size_t)(rank + 1) * 3, (float)rank), gathered;
    {
      std::unique_ptr<OpRecord> r(new OpRecord());
      r->name = "gather";
      r->op = OpType::ALLGATHER;
      r->dtype = DType::F32;
      r->shape = {rank + 1, 3};
      r->in = mine.data();
      r->alloc = alloc_cb;
      r->alloc_user = &gathered;
      int64_t id = rt.enqueue(std::move(r));
      rt.wait(id, 30);
      auto rec = rt.get(id);
      EXPECT((int)rec->dim0.size() == size, "dim0 size");
      rt.release(id);
      size_t pos = 0;
      for (int r2 = 0; r2 < size; r2++)
        for (int i = 0; i < (r2 + 1) * 3; i++) EXPECT(gathered[pos++] == (float)r2, "allgather slab of rank %d", r2);
    }

    // a mismatch must fail on every rank and leave the runtime usable
    {
      std::vector<float> a(10 + rank), b(10 + rank);
      int64_t id = enqueue_allreduce(rt, "bad", a.data(), b.data(), {10 + rank}, false);
      bool threw = false;
      try {
        rt.wait(id, 30);
      } catch (const Error& e) {
        threw = strstr(e.what(), "Mismatched allreduce tensor shapes") != nullptr;
      }
      rt.release(id);
      EXPECT(threw || size == 1, "mismatch not reported");
    }
    // failure path under the sanitizers: rank 1 never sends its request for "lost", so every rank
    // gets a time-out that names the missing rank, and the runtime keeps working afterwards
    if (size > 1) {
      rt.set_fault("drop_request:rank=1:name=lost");
      std::vector<float> a(8, 1.f), b(8, 0.f);
      int64_t id = enqueue_allreduce(rt, "lost", a.data(), b.data(), {8}, false);
      bool timed_out = false;
      try {
        rt.wait(id, 30);
      } catch (const Error& e) {
        timed_out = strstr(e.what(), "Timed out") != nullptr && strstr(e.what(), "1") != nullptr;
      }
      rt.release(id);
      EXPECT(timed_out, "dropped request was not reported as a time-out");
      rt.set_fault("");
      int64_t id2 = enqueue_allreduce(rt, "after_timeout", a.data(), b.data(), {8}, false);
      rt.wait(id2, 30);
      rt.release(id2);
      EXPECT(b[0] == (float)size, "runtime unusable after a time-out: got %f", b[0]);
    }
    auto blobs = rt.blob_gather("blob", std::string(1, (char)('a' + rank)));
    for (int r2 = 0; r2 < size; r2++) EXPECT(blobs[r2] == std::string(1, (char)('a' + r2)), "blob of rank %d", r2);
    (void)rt.stats_json();
    rt.shutdown();
  } catch (const std::exception& e) {
    fprintf(stderr, "rank %d: exception: %s\n", rank, e.what());
    g_failures++;
  }
}

// Control messages that were cut short or damaged on the way must be refused with an error, never
// read out of bounds (AddressSanitizer watches) and never accepted with a different meaning for
// the fields that were not touched.
static void wire_checks() {
  Request q;
  q.rank = 2;
  q.op = OpType::ALLGATHER;
  q.dtype = DType::BF16;
  q.device = DeviceKind::GPU;
  q.name = "layer3/weights:0";
  q.shape = {7, 0, 1 << 20};
  q.blob = std::string("\0\1\2payload", 10);
  q.symm_off = ((int64_t)3 << 48) | 4096;
  q.red = ReduceOp::MAX;
  const std::string fq = encode(q);
  Request q2 = decode_request(fq);
  EXPECT(q2.rank == q.rank && q2.op == q.op && q2.dtype == q.dtype && q2.device == q.device && q2.name == q.name &&
         q2.shape == q.shape && q2.blob == q.blob && q2.symm_off == q.symm_off && q2.red == q.red, "request round trip");
  Response p;
  p.type = ResponseType::ALLGATHER;
  p.name = q.name;
  p.error = "";
  p.dim0 = {1, 0, 5};
  p.blobs = {"a", "", std::string(300, 'x')};
  p.flags = kFlagZeroCopy;
  const std::string fp = encode(p);
  Response p2 = decode_response(fp);
  EXPECT(p2.type == p.type && p2.name == p.name && p2.dim0 == p.dim0 && p2.blobs == p.blobs && p2.flags == p.flags, "response round trip");
  int refused = 0, total = 0;
  for (const std::string* f : {&fq, &fp}) {
    for (size_t cut = 0; cut < f->size(); cut++) {     // every proper prefix
      total++;
      try {
        if (f == &fq) (void)decode_request(f->substr(0, cut));
        else (void)decode_response(f->substr(0, cut));
      } catch (const Error&) {
        refused++;
      }
    }
  }
  EXPECT(refused == total, "%d of %d truncated messages were accepted", total - refused, total);
  uint32_t x = 12345;
  for (int it = 0; it < 20000; it++) {                 // damaged bytes: anything but a crash is fine
    std::string f = (it & 1) ? fq : fp;
    for (int k = 0; k < 1 + it % 3; k++) {
      x = x * 1664525u + 1013904223u;
      f[(x >> 8) % f.size()] = (char)(x >> 24);
    }
    try {
      if (it & 1) (void)decode_request(f);
      else (void)decode_response(f);
    } catch (const Error&) {
    }
  }
}

// A descriptor handed over a unix socket (how the ranks of a host share their GPU allocations)
// arrives usable, tagged, and close-on-exec.
static void descriptor_passing_check() {
  char name[64];
  snprintf(name, sizeof(name), "bcoll-selftest-%d", (int)getpid());
  Socket listener = Socket::listen_unix(name, 2);
  std::thread sender([&] {
    Socket c = Socket::connect_unix(name, now_s() + 5);
    int fds[2];
    if (pipe(fds) != 0) { g_failures++; return; }
    c.send_fd(fds[0], 77, now_s() + 5);       // the read end travels
    ::close(fds[0]);
    const char msg[] = "through the pipe";
    if (write(fds[1], msg, sizeof(msg)) != (ssize_t)sizeof(msg)) g_failures++;
    ::close(fds[1]);
  });
  Socket a = listener.accept(now_s() + 5);
  int32_t tag = 0;
  int fd = a.recv_fd(&tag, now_s() + 5);
  sender.join();
  char buf[32] = {0};
  ssize_t k = read(fd, buf, sizeof(buf));
  EXPECT(tag == 77 && k == 17 && strcmp(buf, "through the pipe") == 0, "descriptor passing: tag %d, %zd bytes", (int)tag, k);
  EXPECT((fcntl(fd, F_GETFD) & FD_CLOEXEC) != 0, "received descriptor is not close-on-exec");
  ::close(fd);
}

int main(int argc, char** argv) {
  wire_checks();
  descriptor_passing_check();
  int n = argc > 1 ? atoi(argv[1]) : 3;
  int port = argc > 2 ? atoi(argv[2]) : 29650;
  int port2 = argc > 3 ? atoi(argv[3]) : 0;
  std::vector<std::thread> ts;
  for (int r = 0; r < n; r++) ts.emplace_back(rank_main, r, n, port, std::string());
  for (auto& t : ts) t.join();
  if (port2 > 0) {
    // The same program with the ranks spread over two host names (2 + 2): node groups, rails, and
    // the allreduce in two levels (shared memory inside a "host" unless BC_SHM=0).
    ts.clear();
    for (int r = 0; r < 4; r++) ts.emplace_back(rank_main, r, 4, port2, std::string(r < 2 ? "hostA" : "hostB"));
    for (auto& t : ts) t.join();
  }
  if (g_failures.load() == 0) printf("host_selftest ok (%d ranks)\n", n);
  return g_failures.load() == 0 ? 0 : 1;
}
