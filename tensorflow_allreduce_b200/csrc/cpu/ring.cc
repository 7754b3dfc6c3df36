#include "ring.h"

#include <string.h>

#include <algorithm>
#include <cmath>

namespace bc {

namespace {

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;  // round to nearest, ties to even
  return (uint16_t)(u >> 16);
}

// Element range of ring slice `i` when `count` elements are split as evenly as possible over
// `n` slices (the first count % n slices get one extra element).
struct Slices {
  size_t q, rem;
  Slices(size_t count, int n) : q(count / n), rem(count % n) {}
  size_t begin(int i) const { return (size_t)i * q + std::min<size_t>((size_t)i, rem); }
  size_t len(int i) const { return q + ((size_t)i < rem ? 1 : 0); }
};

template <typename T>
void add_into(T* dst, const T* src, size_t n, ReduceOp red) {
  switch (red) {
    case ReduceOp::SUM: for (size_t i = 0; i < n; i++) dst[i] += src[i]; break;
    case ReduceOp::PROD: for (size_t i = 0; i < n; i++) dst[i] *= src[i]; break;
    case ReduceOp::MIN: for (size_t i = 0; i < n; i++) dst[i] = src[i] < dst[i] ? src[i] : dst[i]; break;
    case ReduceOp::MAX: for (size_t i = 0; i < n; i++) dst[i] = src[i] > dst[i] ? src[i] : dst[i]; break;
  }
}

template <typename T>
void ring_sum(Transport& t, T* buf, size_t count, double deadline, ReduceOp red) {
  const int n = t.size, r = t.rank;
  if (n == 1 || count == 0) return;
  Slices sl(count, n);
  std::vector<T> incoming(sl.q + 1);
  // Reduce-scatter: after step k, slice (r - k - 1) holds the partial sum of k + 2 ranks.
  for (int k = 0; k < n - 1; k++) {
    const int out_i = ((r - k) % n + n) % n;
    const int in_i = ((r - k - 1) % n + n) % n;
    send_recv(t.ring_next, buf + sl.begin(out_i), sl.len(out_i) * sizeof(T),
              t.ring_prev, incoming.data(), sl.len(in_i) * sizeof(T), deadline);
    add_into(buf + sl.begin(in_i), incoming.data(), sl.len(in_i), red);
  }
  // Allgather: the fully reduced slice (r + 1) travels round; received slices land in place.
  for (int k = 0; k < n - 1; k++) {
    const int out_i = ((r - k + 1) % n + n) % n;
    const int in_i = ((r - k) % n + n) % n;
    send_recv(t.ring_next, buf + sl.begin(out_i), sl.len(out_i) * sizeof(T),
              t.ring_prev, buf + sl.begin(in_i), sl.len(in_i) * sizeof(T), deadline);
  }
}

template <typename T>
void scale_float(T* buf, size_t n, double scale) {
  if (scale == 1.0) return;
  const T s = (T)scale;
  for (size_t i = 0; i < n; i++) buf[i] *= s;
}

template <typename T>
void divide_int(T* buf, size_t n, int64_t d) {
  if (d <= 1) return;
  for (size_t i = 0; i < n; i++) buf[i] = (T)(buf[i] / (T)d);
}

}  // namespace

void widen_to_f32(const void* src, float* dst, size_t n, DType dtype) {
  if (dtype == DType::BF16) {
    const uint16_t* s = (const uint16_t*)src;
    for (size_t i = 0; i < n; i++) dst[i] = bf16_to_f32(s[i]);
  } else if (dtype == DType::F16) {
    const _Float16* s = (const _Float16*)src;
    for (size_t i = 0; i < n; i++) dst[i] = (float)s[i];
  } else {
    throw Error("widen_to_f32: not a 16-bit float type");
  }
}

void narrow_from_f32(const float* src, void* dst, size_t n, DType dtype) {
  if (dtype == DType::BF16) {
    uint16_t* d = (uint16_t*)dst;
    for (size_t i = 0; i < n; i++) d[i] = f32_to_bf16(src[i]);
  } else if (dtype == DType::F16) {
    _Float16* d = (_Float16*)dst;
    for (size_t i = 0; i < n; i++) d[i] = (_Float16)src[i];
  } else {
    throw Error("narrow_from_f32: not a 16-bit float type");
  }
}

void cpu_ring_allreduce(Transport& t, void* data, size_t count, DType dtype, double scale,
                        int64_t int_divisor, double deadline, ReduceOp red) {
  switch (dtype) {
    case DType::F32:
      ring_sum(t, (float*)data, count, deadline, red);
      scale_float((float*)data, count, scale);
      break;
    case DType::F64:
      ring_sum(t, (double*)data, count, deadline, red);
      scale_float((double*)data, count, scale);
      break;
    case DType::I32:
      ring_sum(t, (int32_t*)data, count, deadline, red);
      divide_int((int32_t*)data, count, int_divisor);
      break;
    case DType::I64:
      ring_sum(t, (int64_t*)data, count, deadline, red);
      divide_int((int64_t*)data, count, int_divisor);
      break;
    case DType::U8:
      ring_sum(t, (uint8_t*)data, count, deadline, red);
      divide_int((uint8_t*)data, count, int_divisor);
      break;
    case DType::BF16:
    case DType::F16: {
      std::vector<float> wide(count);
      widen_to_f32(data, wide.data(), count, dtype);
      ring_sum(t, wide.data(), count, deadline, red);
      scale_float(wide.data(), count, scale);
      narrow_from_f32(wide.data(), data, count, dtype);
      break;
    }
    default:
      throw Error("cpu_ring_allreduce: unsupported dtype");
  }
}

void cpu_ring_allgatherv(Transport& t, const void* in, void* out, const std::vector<int64_t>& rows,
                         size_t row_bytes, double deadline) {
  const int n = t.size, r = t.rank;
  BC_CHECK((int)rows.size() == n, "allgatherv: need one row count per rank");
  std::vector<size_t> off(n + 1, 0);
  for (int i = 0; i < n; i++) off[i + 1] = off[i] + (size_t)rows[i] * row_bytes;
  char* o = (char*)out;
  if (off[r + 1] > off[r] && in != o + off[r]) memcpy(o + off[r], in, off[r + 1] - off[r]);
  // At step k every rank forwards the slab that originated k ranks behind it.
  for (int k = 0; k < n - 1; k++) {
    const int out_i = ((r - k) % n + n) % n;
    const int in_i = ((r - k - 1) % n + n) % n;
    send_recv(t.ring_next, o + off[out_i], off[out_i + 1] - off[out_i],
              t.ring_prev, o + off[in_i], off[in_i + 1] - off[in_i], deadline);
  }
}

}  // namespace bc
