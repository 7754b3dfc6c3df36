// Control-plane messages and their binary encoding.
//
// Same roles as MPIRequest / MPIResponse in the reference
// (tensorflow/contrib/mpi_collectives/mpi_message.proto:12-63), as plain structs with a
// length-prefixed little-endian encoding instead of protobuf-in-a-C-string: any byte value
// (a zero-sized dimension included) survives the trip. The response to an allgather carries every
// rank's first-dimension size, which removes the reference's separate sizing pass
// (mpi_ops.py:152-160).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "../common.h"

namespace bc {

enum class DeviceKind : uint8_t { CPU = 0, GPU = 1 };

struct Request {
  int32_t rank = 0;
  OpType op = OpType::ALLREDUCE;
  DType dtype = DType::F32;
  DeviceKind device = DeviceKind::CPU;
  std::string name;
  std::vector<int64_t> shape;
  std::string blob;  // BLOB_GATHER payload (small host data), empty otherwise
  // GPU allreduce in place on symmetric memory: (segment id << 48) | offset of the tensor inside
  // that segment, or -1. The zero-copy path is taken only if all ranks report the same value.
  int64_t symm_off = -1;
  ReduceOp red = ReduceOp::SUM;   // allreduce only
};

enum class ResponseType : uint8_t { ALLREDUCE = 0, ALLGATHER = 1, BLOB_GATHER = 2, ERROR = 3, SHUTDOWN = 4, ABORT = 5 };

struct Response {
  ResponseType type = ResponseType::ERROR;
  std::string name;
  std::string error;
  std::vector<int64_t> dim0;        // ALLGATHER: first-dimension size of every rank, in rank order
  std::vector<std::string> blobs;   // BLOB_GATHER: every rank's payload, in rank order
  uint32_t flags = 0;               // kFlagZeroCopy
};
constexpr uint32_t kFlagZeroCopy = 1u;

std::string encode(const Request& r);
std::string encode(const Response& r);
Request decode_request(const std::string& s);
Response decode_response(const std::string& s);

// Validation performed by the coordinator once every rank has asked for `name`
// (reference: ConstructMPIResponse, mpi_ops.cc:277-432; same rules and error wording):
// same dtype, same operation, same device kind, allreduce -> identical shapes,
// allgather -> same rank (not scalar) and equal dimensions except the first.
// `requests` must hold one entry per rank, in rank order.
Response build_response(const std::string& name, const std::vector<Request>& requests);

std::string shape_string(const std::vector<int64_t>& shape);

}  // namespace bc
