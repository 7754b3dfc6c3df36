#include "shm_group.h"

#include <fcntl.h>
#include <sched.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>

#include "ring.h"

namespace bc {

namespace {

inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
  __builtin_ia32_pause();
#else
  sched_yield();
#endif
}

template <typename T>
inline T fold(T a, T b, ReduceOp red) {
  switch (red) {
    case ReduceOp::SUM: return a + b;
    case ReduceOp::PROD: return a * b;
    case ReduceOp::MIN: return b < a ? b : a;
    default: return b > a ? b : a;
  }
}

// out[i] = reduction over the n slots of element i, for i in [0, len); slots are `stride` bytes apart.
template <typename T, ReduceOp RED>
void reduce_slots_t(T* out, const char* slot0, size_t stride, int n, size_t first, size_t len) {
  const T* s0 = (const T*)slot0 + first;
  for (size_t i = 0; i < len; i++) out[i] = s0[i];
  for (int p = 1; p < n; p++) {
    const T* sp = (const T*)(slot0 + (size_t)p * stride) + first;
    for (size_t i = 0; i < len; i++) out[i] = fold<T>(out[i], sp[i], RED);
  }
}

template <typename T>
void reduce_slots(T* out, const char* slot0, size_t stride, int n, size_t first, size_t len, ReduceOp red) {
  switch (red) {
    case ReduceOp::SUM: reduce_slots_t<T, ReduceOp::SUM>(out, slot0, stride, n, first, len); break;
    case ReduceOp::PROD: reduce_slots_t<T, ReduceOp::PROD>(out, slot0, stride, n, first, len); break;
    case ReduceOp::MIN: reduce_slots_t<T, ReduceOp::MIN>(out, slot0, stride, n, first, len); break;
    case ReduceOp::MAX: reduce_slots_t<T, ReduceOp::MAX>(out, slot0, stride, n, first, len); break;
  }
}

template <typename T>
void scale_float(T* p, size_t n, double scale) {
  if (scale == 1.0) return;
  const T s = (T)scale;
  for (size_t i = 0; i < n; i++) p[i] *= s;
}

template <typename T>
void divide_int(T* p, size_t n, int64_t d) {
  if (d <= 1) return;
  for (size_t i = 0; i < n; i++) p[i] = (T)(p[i] / (T)d);
}

}  // namespace

ShmGroup::ShmGroup(int local_rank, int local_size, const std::string& name, size_t slot_bytes, const Allgather& ag,
                   const PeerLost& peer_lost)
    : r_(local_rank), n_(local_size), peer_lost_(peer_lost), slot_bytes_((slot_bytes + 4095) / 4096 * 4096) {
  BC_CHECK(n_ >= 1 && r_ >= 0 && r_ < n_, "bad local rank " << r_ << "/" << n_);
  BC_CHECK(slot_bytes_ >= 4096, "shared-memory slot too small");
  map_bytes_ = kHeaderBytes + (size_t)(n_ + 1) * slot_bytes_;
  const std::string path = "/" + name;
  // The leader creates and sizes the object, the others open it once they hear that it exists,
  // and the name is removed as soon as everybody has it mapped: nothing is left behind when a
  // rank dies later.
  std::string err;
  int fd = -1;
  if (r_ == 0) {
    shm_unlink(path.c_str());
    fd = shm_open(path.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) err = std::string("shm_open(create): ") + strerror(errno);
    else if (ftruncate(fd, (off_t)map_bytes_) != 0) err = std::string("ftruncate: ") + strerror(errno);
    else if (int rc = posix_fallocate(fd, 0, (off_t)map_bytes_))   // claim the pages now: a full /dev/shm must
      err = std::string("posix_fallocate: ") + strerror(rc);       // show up here, not as SIGBUS on first touch
  }
  std::vector<std::string> st = ag(err);
  if (!st[0].empty()) {
    if (fd >= 0) { ::close(fd); shm_unlink(path.c_str()); }
    throw Error("shared-memory group: " + st[0]);
  }
  if (r_ != 0) {
    fd = shm_open(path.c_str(), O_RDWR, 0600);
    if (fd < 0) err = std::string("shm_open: ") + strerror(errno);
  }
  if (err.empty()) {
    void* p = mmap(nullptr, map_bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    if (p == MAP_FAILED) err = std::string("mmap: ") + strerror(errno);
    else base_ = (char*)p;
  }
  if (fd >= 0) ::close(fd);
  if (base_ && r_ == 0) {
    hdr_ = new (base_) Header();
    hdr_->arrived.store(0);
    hdr_->generation.store(0);
    hdr_->broken.store(0);
  }
  st = ag(err);
  if (r_ == 0) shm_unlink(path.c_str());
  for (int i = 0; i < n_; i++) {
    if (!st[i].empty()) {
      if (base_) munmap(base_, map_bytes_);
      base_ = nullptr;
      throw Error("shared-memory group (local rank " + std::to_string(i) + "): " + st[i]);
    }
  }
  hdr_ = (Header*)base_;
  // Touch this rank's slot now, so that the first collective does not pay for the page faults.
  memset(slot(r_), 0, slot_bytes_);
  if (r_ == 0) memset(result(), 0, slot_bytes_);
}

ShmGroup::~ShmGroup() {
  if (base_) munmap(base_, map_bytes_);
}

void ShmGroup::barrier(double deadline) {
  if (n_ == 1) return;
  const uint32_t gen = hdr_->generation.load(std::memory_order_acquire);
  if (hdr_->arrived.fetch_add(1, std::memory_order_acq_rel) == (uint32_t)n_ - 1) {
    hdr_->arrived.store(0, std::memory_order_relaxed);
    hdr_->generation.store(gen + 1, std::memory_order_release);
    return;
  }
  // Spin briefly (the peers are usually a few microseconds away), then yield, then sleep.
  for (uint64_t spins = 0;; spins++) {
    if (hdr_->generation.load(std::memory_order_acquire) != gen) return;
    if (spins < 4000) {
      cpu_relax();
    } else if (spins < 20000) {
      sched_yield();
    } else {
      struct timespec ts = {0, 50000};
      nanosleep(&ts, nullptr);
      if ((spins & 63) == 0 && peer_lost_) {   // every few milliseconds: is everybody still there?
        const std::string why = peer_lost_();
        if (!why.empty()) {
          hdr_->broken.store(1, std::memory_order_release);
          throw CommLost(why);
        }
      }
    }
    if ((spins & 1023) == 1023) {
      if (hdr_->broken.load(std::memory_order_acquire)) throw CommLost("a rank of this host gave up waiting in a shared-memory collective");
      if (now_s() >= deadline) {
        hdr_->broken.store(1, std::memory_order_release);
        throw CommLost("timed out waiting for the ranks of this host in a shared-memory collective");
      }
    }
  }
}

void ShmGroup::allreduce(const void* in, void* data, size_t count, DType dtype, double scale, int64_t int_divisor, ReduceOp red,
                         double deadline) {
  const size_t e = dtype_size(dtype);
  if (count == 0) return;
  if (n_ == 1) {
    if (in != data) memcpy(data, in, count * e);
    switch (dtype) {
      case DType::F32: scale_float((float*)data, count, scale); break;
      case DType::F64: scale_float((double*)data, count, scale); break;
      case DType::I32: divide_int((int32_t*)data, count, int_divisor); break;
      case DType::I64: divide_int((int64_t*)data, count, int_divisor); break;
      case DType::U8: divide_int((uint8_t*)data, count, int_divisor); break;
      default: break;
    }
    return;
  }
  const size_t chunk = slot_bytes_ / e;
  std::vector<float> wide;   // 16-bit floats are accumulated in fp32
  for (size_t off = 0; off < count; off += chunk) {
    const size_t n = std::min(chunk, count - off);
    char* mine = (char*)data + off * e;
    memcpy(slot(r_), (const char*)in + off * e, n * e);
    barrier(deadline);
    // slice r of this chunk, cut like the ring's segments
    const size_t q = n / n_, rem = n % n_;
    const size_t first = (size_t)r_ * q + std::min<size_t>((size_t)r_, rem);
    const size_t len = q + ((size_t)r_ < rem ? 1 : 0);
    char* res = result() + first * e;
    switch (dtype) {
      case DType::F32:
        reduce_slots((float*)res, slot(0), slot_bytes_, n_, first, len, red);
        scale_float((float*)res, len, scale);
        break;
      case DType::F64:
        reduce_slots((double*)res, slot(0), slot_bytes_, n_, first, len, red);
        scale_float((double*)res, len, scale);
        break;
      case DType::I32:
        reduce_slots((int32_t*)res, slot(0), slot_bytes_, n_, first, len, red);
        divide_int((int32_t*)res, len, int_divisor);
        break;
      case DType::I64:
        reduce_slots((int64_t*)res, slot(0), slot_bytes_, n_, first, len, red);
        divide_int((int64_t*)res, len, int_divisor);
        break;
      case DType::U8:
        reduce_slots((uint8_t*)res, slot(0), slot_bytes_, n_, first, len, red);
        divide_int((uint8_t*)res, len, int_divisor);
        break;
      case DType::BF16:
      case DType::F16: {
        wide.resize(2 * len);
        float* acc = wide.data();
        float* tmp = wide.data() + len;
        widen_to_f32(slot(0) + first * e, acc, len, dtype);
        for (int p = 1; p < n_; p++) {
          widen_to_f32(slot(p) + first * e, tmp, len, dtype);
          for (size_t i = 0; i < len; i++) acc[i] = fold<float>(acc[i], tmp[i], red);
        }
        scale_float(acc, len, scale);
        narrow_from_f32(acc, res, len, dtype);
        break;
      }
      default:
        throw Error("shared-memory allreduce: unsupported element type");
    }
    barrier(deadline);
    memcpy(mine, result(), n * e);
    // No third barrier: the result area is next written after the first barrier of the next chunk
    // or collective, which every rank reaches only after this copy; until then the ranks write
    // their own slots only, and nobody reads slots between the second barrier and that one.
  }
}

void ShmGroup::allgatherv(const void* in, void* out, const std::vector<int64_t>& rows, size_t row_bytes, double deadline) {
  BC_CHECK((int)rows.size() == n_, "allgatherv: need one row count per rank");
  std::vector<size_t> off(n_ + 1, 0);
  for (int i = 0; i < n_; i++) off[i + 1] = off[i] + (size_t)rows[i] * row_bytes;
  if (off[n_] == 0) return;
  char* o = (char*)out;
  if (n_ == 1) {
    if (in != o) memcpy(o, in, off[1]);
    return;
  }
  // Pass p moves bytes [p * slot, (p + 1) * slot) of every slab: owners publish, everybody copies.
  size_t longest = 0;
  for (int i = 0; i < n_; i++) longest = std::max(longest, off[i + 1] - off[i]);
  for (size_t done = 0; done < longest; done += slot_bytes_) {
    const size_t my_len = off[r_ + 1] - off[r_];
    if (done < my_len) memcpy(slot(r_), (const char*)in + done, std::min(slot_bytes_, my_len - done));
    barrier(deadline);
    for (int i = 0; i < n_; i++) {
      const size_t len_i = off[i + 1] - off[i];
      if (done >= len_i) continue;
      const size_t piece = std::min(slot_bytes_, len_i - done);
      if (i == r_) {
        if ((const char*)in + done != o + off[i] + done) memcpy(o + off[i] + done, (const char*)in + done, piece);
      } else {
        memcpy(o + off[i] + done, slot(i), piece);
      }
    }
    barrier(deadline);
  }
}

}  // namespace bc
