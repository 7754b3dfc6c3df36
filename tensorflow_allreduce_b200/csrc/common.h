// Shared definitions for the native runtime: dtypes, status/error type, logging.
//
// The element types cover what the reference's collective ops accept
// (float32 / int32 / int64, tensorflow/contrib/mpi_collectives/mpi_ops.cc:836-847)
// plus bf16 / fp16 / fp64 / uint8, which the B200 data paths need.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <chrono>
#include <sstream>
#include <stdexcept>
#include <string>

namespace bc {

enum class DType : uint8_t { F32 = 0, I32 = 1, I64 = 2, BF16 = 3, F16 = 4, F64 = 5, U8 = 6, INVALID = 255 };

inline size_t dtype_size(DType t) {
  switch (t) {
    case DType::F32: case DType::I32: return 4;
    case DType::I64: case DType::F64: return 8;
    case DType::BF16: case DType::F16: return 2;
    case DType::U8: return 1;
    default: return 0;
  }
}

inline const char* dtype_name(DType t) {
  switch (t) {
    case DType::F32: return "float32";
    case DType::I32: return "int32";
    case DType::I64: return "int64";
    case DType::BF16: return "bfloat16";
    case DType::F16: return "float16";
    case DType::F64: return "float64";
    case DType::U8: return "uint8";
    default: return "invalid";
  }
}

// Element-wise reduction of an allreduce. The reference's MPI collectives only sum
// (tensorflow/contrib/mpi_collectives/ring.cc:42-50); its single-process NCCL ops also offer
// prod / min / max (tensorflow/contrib/nccl/kernels/nccl_ops.cc:68-79).
enum class ReduceOp : uint8_t { SUM = 0, PROD = 1, MIN = 2, MAX = 3 };

inline const char* reduce_name(ReduceOp r) {
  switch (r) {
    case ReduceOp::SUM: return "sum";
    case ReduceOp::PROD: return "prod";
    case ReduceOp::MIN: return "min";
    case ReduceOp::MAX: return "max";
  }
  return "?";
}

enum class OpType : uint8_t { ALLREDUCE = 0, ALLGATHER = 1, BLOB_GATHER = 2, SHUTDOWN = 3 };

inline const char* op_name(OpType t) {
  switch (t) {
    case OpType::ALLREDUCE: return "ALLREDUCE";
    case OpType::ALLGATHER: return "ALLGATHER";
    case OpType::BLOB_GATHER: return "BLOB_GATHER";
    case OpType::SHUTDOWN: return "SHUTDOWN";
  }
  return "?";
}

// Error carried through the runtime; the C API turns it into a return code + message.
struct Error : public std::runtime_error {
  explicit Error(const std::string& m) : std::runtime_error(m) {}
};

// A peer went away or a deadline ran out: the communicator is unusable afterwards.
struct CommLost : public Error {
  explicit CommLost(const std::string& m) : Error(m) {}
};

#define BC_CHECK(cond, msg)                                                     \
  do {                                                                          \
    if (!(cond)) {                                                              \
      std::ostringstream _os;                                                   \
      _os << msg;                                                               \
      throw ::bc::Error(_os.str());                                             \
    }                                                                           \
  } while (0)

inline double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Log level from BC_LOG_LEVEL: 0 = errors only (default), 1 = info, 2 = debug, 3 = trace.
int log_level();
void log_line(int level, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// NVTX range for profilers (header-only NVTX 3: without an attached tool a push/pop is a load and
// a branch). The reference relies on TensorFlow's tracing (direct_session.cc:538-566); here the
// runtime marks negotiation, launches and the ring itself.
struct NvtxRange {
  explicit NvtxRange(const char* name);
  ~NvtxRange();
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

#define BC_LOG(level, ...)                                   \
  do {                                                       \
    if (::bc::log_level() >= (level)) ::bc::log_line((level), __VA_ARGS__); \
  } while (0)

}  // namespace bc
