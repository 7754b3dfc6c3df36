#include "two_level.h"

#include <string.h>

#include <condition_variable>
#include <exception>
#include <mutex>
#include <thread>

#include "../cpu/ring.h"
#include "../cpu/shm_group.h"

namespace bc {

void two_level_allreduce(NodeGroup& g, LocalLevel& local, void* staging, size_t count, DType dtype, double scale,
                         int64_t int_divisor, ReduceOp red, double deadline, double* seconds) {
  const double t0 = now_s();
  local.reduce_in_node(count, dtype, red);
  const int L = g.local_size;
  std::vector<size_t> lens(L);
  for (int i = 0; i < L; i++) lens[i] = slice_len(count, L, i);
  const size_t begin = slice_begin(count, L, g.local_rank), len = lens[g.local_rank];
  local.fetch(staging, begin, len, dtype);
  const double t1 = now_s();
  // The ranks of one rail hold the same slice of their hosts' sums, so the lengths agree.
  cpu_ring_allreduce(g.rail, staging, len, dtype, scale, int_divisor, deadline, red);
  const double t2 = now_s();
  local.finish(staging, begin, len, lens, dtype);
  if (seconds) {
    seconds[0] = t1 - t0;
    seconds[1] = t2 - t1;
    seconds[2] = now_s() - t2;
  }
}

void two_level_allreduce_pipelined(NodeGroup& g, ShmGroup& shm, void* tensor, void* staging, size_t count, size_t chunk_elems,
                                   DType dtype, double scale, int64_t int_divisor, ReduceOp red, double deadline, double* seconds) {
  const size_t e = dtype_size(dtype);
  const int L = g.local_size;
  BC_CHECK(chunk_elems > 0, "two-level allreduce: empty chunks");
  const size_t K = (count + chunk_elems - 1) / chunk_elems;
  char* t = (char*)tensor;
  char* buf[2] = {(char*)staging, (char*)staging + slice_len(chunk_elems, L, 0) * e};
  auto chunk_begin = [&](size_t c) { return c * chunk_elems; };
  auto chunk_len = [&](size_t c) { return std::min(chunk_elems, count - c * chunk_elems); };

  // What the two threads tell each other: how many chunks have been handed to the rail, how many
  // have come back, and whether either side has given up.
  struct {
    std::mutex mu;
    std::condition_variable cv;
    size_t fetched = 0, ringed = 0;
    bool abort = false;
    std::exception_ptr err;
  } st;

  std::thread rail([&] {
    for (size_t c = 0; c < K; c++) {
      {
        std::unique_lock<std::mutex> lk(st.mu);
        st.cv.wait(lk, [&] { return st.fetched > c || st.abort; });
        if (st.abort) return;
      }
      try {
        // The ranks of one rail hold the same slice of their hosts' sums, so the lengths agree.
        cpu_ring_allreduce(g.rail, buf[c & 1], slice_len(chunk_len(c), L, g.local_rank), dtype, scale, int_divisor, deadline, red);
      } catch (...) {
        std::lock_guard<std::mutex> lk(st.mu);
        st.err = std::current_exception();
        st.abort = true;
        st.cv.notify_all();
        return;
      }
      std::lock_guard<std::mutex> lk(st.mu);
      st.ringed = c + 1;
      st.cv.notify_all();
    }
  });

  double spent[3] = {0, 0, 0};
  auto gather = [&](size_t c) {   // wait for chunk c to come back over the rail, then spread it inside the host
    double t0 = now_s();
    {
      std::unique_lock<std::mutex> lk(st.mu);
      st.cv.wait(lk, [&] { return st.ringed > c || st.abort; });
      if (st.abort) std::rethrow_exception(st.err ? st.err : std::make_exception_ptr(Error("two-level allreduce was aborted")));
    }
    double t1 = now_s();
    spent[1] += t1 - t0;
    const size_t n = chunk_len(c);
    std::vector<int64_t> rows(L);
    for (int i = 0; i < L; i++) rows[i] = (int64_t)slice_len(n, L, i);     // one "row" per element
    shm.allgatherv(buf[c & 1], t + chunk_begin(c) * e, rows, e, deadline);
    spent[2] += now_s() - t1;
  };
  try {
    for (size_t c = 0; c < K; c++) {
      const double t0 = now_s();
      const size_t n = chunk_len(c);
      shm.allreduce(t + chunk_begin(c) * e, n, dtype, 1.0, 1, red, deadline);
      const size_t len = slice_len(n, L, g.local_rank);
      // buf[c & 1] last held chunk c - 2, which was gathered in the previous round
      if (len) memcpy(buf[c & 1], t + (chunk_begin(c) + slice_begin(n, L, g.local_rank)) * e, len * e);
      spent[0] += now_s() - t0;
      {
        std::lock_guard<std::mutex> lk(st.mu);
        st.fetched = c + 1;
        st.cv.notify_all();
      }
      if (c >= 1) gather(c - 1);
    }
    gather(K - 1);
  } catch (...) {
    {
      std::lock_guard<std::mutex> lk(st.mu);
      st.abort = true;
      st.cv.notify_all();
    }
    rail.join();     // a ring step in flight ends at its deadline at the latest
    throw;
  }
  rail.join();
  if (seconds)
    for (int i = 0; i < 3; i++) seconds[i] = spent[i];
}

namespace {

template <typename T>
void combine(T* dst, const T* src, size_t n, ReduceOp red) {
  for (size_t i = 0; i < n; i++) {
    switch (red) {
      case ReduceOp::SUM: dst[i] += src[i]; break;
      case ReduceOp::PROD: dst[i] *= src[i]; break;
      case ReduceOp::MIN: dst[i] = src[i] < dst[i] ? src[i] : dst[i]; break;
      case ReduceOp::MAX: dst[i] = src[i] > dst[i] ? src[i] : dst[i]; break;
    }
  }
}

}  // namespace

void ShmLocalLevel::reduce_in_node(size_t count, DType dtype, ReduceOp red) {
  shm_.allreduce(t_, count, dtype, 1.0, 1, red, deadline_);
}

void ShmLocalLevel::fetch(void* dst, size_t begin, size_t len, DType dtype) {
  const size_t e = dtype_size(dtype);
  if (len) memcpy(dst, t_ + begin * e, len * e);
}

void ShmLocalLevel::finish(const void* src, size_t begin, size_t len, const std::vector<size_t>& lens, DType dtype) {
  (void)begin;
  (void)len;
  std::vector<int64_t> rows(lens.begin(), lens.end());     // one "row" per element
  shm_.allgatherv(src, t_, rows, dtype_size(dtype), deadline_);
}

void HostLocalLevel::reduce_in_node(size_t count, DType dtype, ReduceOp red) {
  const size_t bytes = count * dtype_size(dtype);
  std::vector<std::string> all = g_.allgather(std::string(t_, bytes), deadline_);
  // every member folds the blobs in the same order, so the results agree bit for bit
  memcpy(t_, all[0].data(), bytes);
  for (int i = 1; i < g_.local_size; i++) {
    BC_CHECK(all[i].size() == bytes, "node members passed tensors of different sizes");
    switch (dtype) {
      case DType::F32: combine((float*)t_, (const float*)all[i].data(), count, red); break;
      case DType::F64: combine((double*)t_, (const double*)all[i].data(), count, red); break;
      case DType::I32: combine((int32_t*)t_, (const int32_t*)all[i].data(), count, red); break;
      case DType::I64: combine((int64_t*)t_, (const int64_t*)all[i].data(), count, red); break;
      case DType::U8: combine((uint8_t*)t_, (const uint8_t*)all[i].data(), count, red); break;
      default: throw Error("HostLocalLevel: unsupported element type");
    }
  }
}

void HostLocalLevel::fetch(void* dst, size_t begin, size_t len, DType dtype) {
  const size_t e = dtype_size(dtype);
  if (len) memcpy(dst, t_ + begin * e, len * e);
}

void HostLocalLevel::finish(const void* src, size_t begin, size_t len, const std::vector<size_t>& lens, DType dtype) {
  const size_t e = dtype_size(dtype);
  (void)begin;
  std::vector<std::string> all = g_.allgather(std::string((const char*)src, len * e), deadline_);
  size_t off = 0;
  for (int i = 0; i < g_.local_size; i++) {
    BC_CHECK(all[i].size() == lens[i] * e, "slice " << i << " arrived with " << all[i].size() << " bytes, expected " << lens[i] * e);
    if (lens[i]) memcpy(t_ + off, all[i].data(), lens[i] * e);
    off += lens[i] * e;
  }
}

}  // namespace bc
