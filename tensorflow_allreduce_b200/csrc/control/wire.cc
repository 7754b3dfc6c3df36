#include "wire.h"

#include <string.h>

namespace bc {

namespace {

struct Writer {
  std::string s;
  void u8(uint8_t v) { s.push_back((char)v); }
  void u32(uint32_t v) { s.append((const char*)&v, 4); }
  void i32(int32_t v) { s.append((const char*)&v, 4); }
  void i64(int64_t v) { s.append((const char*)&v, 8); }
  void str(const std::string& v) { u32((uint32_t)v.size()); s.append(v); }
};

struct Reader {
  const std::string& s;
  size_t pos = 0;
  explicit Reader(const std::string& in) : s(in) {}
  void need(size_t n) { BC_CHECK(pos + n <= s.size(), "truncated control message"); }
  uint8_t u8() { need(1); return (uint8_t)s[pos++]; }
  uint32_t u32() { need(4); uint32_t v; memcpy(&v, &s[pos], 4); pos += 4; return v; }
  int32_t i32() { need(4); int32_t v; memcpy(&v, &s[pos], 4); pos += 4; return v; }
  int64_t i64() { need(8); int64_t v; memcpy(&v, &s[pos], 8); pos += 8; return v; }
  std::string str() { uint32_t n = u32(); need(n); std::string v = s.substr(pos, n); pos += n; return v; }
};

constexpr uint8_t kReqMagic = 0xA1;
constexpr uint8_t kRespMagic = 0xB2;

}  // namespace

std::string encode(const Request& r) {
  Writer w;
  w.u8(kReqMagic);
  w.i32(r.rank);
  w.u8((uint8_t)r.op);
  w.u8((uint8_t)r.dtype);
  w.u8((uint8_t)r.device);
  w.str(r.name);
  w.u32((uint32_t)r.shape.size());
  for (int64_t d : r.shape) w.i64(d);
  w.str(r.blob);
  w.i64(r.symm_off);
  w.u8((uint8_t)r.red);
  return w.s;
}

Request decode_request(const std::string& s) {
  Reader rd(s);
  BC_CHECK(rd.u8() == kReqMagic, "bad request magic");
  Request r;
  r.rank = rd.i32();
  r.op = (OpType)rd.u8();
  r.dtype = (DType)rd.u8();
  r.device = (DeviceKind)rd.u8();
  r.name = rd.str();
  uint32_t nd = rd.u32();
  BC_CHECK(nd <= 64, "too many dimensions in request");
  r.shape.resize(nd);
  for (uint32_t i = 0; i < nd; i++) r.shape[i] = rd.i64();
  r.blob = rd.str();
  r.symm_off = rd.i64();
  r.red = (ReduceOp)rd.u8();
  BC_CHECK((uint8_t)r.red <= (uint8_t)ReduceOp::MAX, "bad reduction in request");
  BC_CHECK((uint8_t)r.op <= (uint8_t)OpType::SHUTDOWN, "bad operation in request");
  BC_CHECK((uint8_t)r.dtype <= (uint8_t)DType::U8 || r.dtype == DType::INVALID, "bad element type in request");
  BC_CHECK((uint8_t)r.device <= (uint8_t)DeviceKind::GPU, "bad device kind in request");
  BC_CHECK(rd.pos == s.size(), "trailing bytes after a request");
  return r;
}

std::string encode(const Response& r) {
  Writer w;
  w.u8(kRespMagic);
  w.u8((uint8_t)r.type);
  w.str(r.name);
  w.str(r.error);
  w.u32((uint32_t)r.dim0.size());
  for (int64_t d : r.dim0) w.i64(d);
  w.u32((uint32_t)r.blobs.size());
  for (const auto& b : r.blobs) w.str(b);
  w.u32(r.flags);
  return w.s;
}

Response decode_response(const std::string& s) {
  Reader rd(s);
  BC_CHECK(rd.u8() == kRespMagic, "bad response magic");
  Response r;
  r.type = (ResponseType)rd.u8();
  r.name = rd.str();
  r.error = rd.str();
  uint32_t n = rd.u32();
  BC_CHECK(n <= 65536, "bad dim0 count");
  r.dim0.resize(n);
  for (uint32_t i = 0; i < n; i++) r.dim0[i] = rd.i64();
  uint32_t nb = rd.u32();
  BC_CHECK(nb <= 65536, "bad blob count");
  r.blobs.resize(nb);
  for (uint32_t i = 0; i < nb; i++) r.blobs[i] = rd.str();
  r.flags = rd.u32();
  BC_CHECK((uint8_t)r.type <= (uint8_t)ResponseType::ABORT, "bad response type");
  BC_CHECK(rd.pos == s.size(), "trailing bytes after a response");
  return r;
}

std::string shape_string(const std::vector<int64_t>& shape) {
  std::string s = "[";
  for (size_t i = 0; i < shape.size(); i++) {
    if (i) s += ",";
    s += std::to_string(shape[i]);
  }
  return s + "]";
}

Response build_response(const std::string& name, const std::vector<Request>& reqs) {
  Response resp;
  resp.name = name;
  BC_CHECK(!reqs.empty(), "no requests for " << name);
  std::ostringstream err;
  bool bad = false;
  const Request& first = reqs[0];

  for (size_t i = 1; i < reqs.size() && !bad; i++) {
    if (reqs[i].dtype != first.dtype) {
      bad = true;
      err << "Mismatched data types: One rank had type " << dtype_name(first.dtype)
          << ", but another rank had type " << dtype_name(reqs[i].dtype) << ".";
    }
  }
  for (size_t i = 1; i < reqs.size() && !bad; i++) {
    if (reqs[i].op != first.op) {
      bad = true;
      err << "Mismatched MPI operations: One rank did an " << op_name(first.op)
          << ", but another rank did an " << op_name(reqs[i].op) << ".";
    }
  }
  for (size_t i = 1; i < reqs.size() && !bad; i++) {
    if (reqs[i].device != first.device) {
      bad = true;
      err << "Mismatched devices: One rank passed a " << (first.device == DeviceKind::GPU ? "GPU" : "CPU")
          << " tensor, but another rank passed a " << (reqs[i].device == DeviceKind::GPU ? "GPU" : "CPU")
          << " tensor.";
    }
  }

  if (!bad && first.op == OpType::ALLREDUCE) {
    for (size_t i = 1; i < reqs.size() && !bad; i++) {
      if (reqs[i].red != first.red) {
        bad = true;
        err << "Mismatched reductions: One rank asked for " << reduce_name(first.red) << ", but another rank asked for "
            << reduce_name(reqs[i].red) << ".";
      }
    }
    for (size_t i = 1; i < reqs.size() && !bad; i++) {
      if (reqs[i].shape != first.shape) {
        bad = true;
        err << "Mismatched allreduce tensor shapes: One rank reduced a tensor of shape "
            << shape_string(first.shape) << ", but another rank sent a tensor of shape "
            << shape_string(reqs[i].shape) << ".";
      }
    }
  }

  if (!bad && first.op == OpType::ALLGATHER) {
    if (first.shape.empty()) {
      bad = true;
      err << "Rank zero tried to gather a rank-zero tensor.";
    }
    for (size_t i = 1; i < reqs.size() && !bad; i++) {
      if (reqs[i].shape.size() != first.shape.size()) {
        bad = true;
        err << "Mismatched allgather tensor shapes: One rank gathered a tensor of rank "
            << first.shape.size() << ", but another rank sent a tensor of rank " << reqs[i].shape.size() << ".";
        break;
      }
      for (size_t d = 1; d < first.shape.size(); d++) {
        if (reqs[i].shape[d] != first.shape[d]) {
          bad = true;
          err << "Mismatched allgather tensor shapes: One rank gathered a tensor with dimension " << d
              << " equal to " << first.shape[d] << ", but another rank sent a tensor with dimension " << d
              << " equal to " << reqs[i].shape[d] << ".";
          break;
        }
      }
    }
  }

  if (bad) {
    resp.type = ResponseType::ERROR;
    resp.error = err.str();
    return resp;
  }
  switch (first.op) {
    case OpType::ALLREDUCE: {
      resp.type = ResponseType::ALLREDUCE;
      bool zc = first.symm_off >= 0;
      for (const auto& r : reqs) zc = zc && r.symm_off == first.symm_off;
      if (zc) resp.flags |= kFlagZeroCopy;
      break;
    }
    case OpType::ALLGATHER:
      resp.type = ResponseType::ALLGATHER;
      for (const auto& r : reqs) resp.dim0.push_back(r.shape[0]);
      break;
    case OpType::BLOB_GATHER:
      resp.type = ResponseType::BLOB_GATHER;
      for (const auto& r : reqs) resp.blobs.push_back(r.blob);
      break;
    case OpType::SHUTDOWN:
      resp.type = ResponseType::SHUTDOWN;
      break;
  }
  return resp;
}

}  // namespace bc
