// CPU collectives over the data ring: sum-allreduce and variable-length allgather.
//
// These play the role of RingAllreduce / RingAllgather with the CPU primitives of the reference
// (tensorflow/contrib/mpi_collectives/ring.h:136-301, ring.cc:36-50): a reduce-scatter pass
// followed by an allgather pass around the ring, each rank moving 2*K*(N-1)/N bytes for a K-byte
// tensor. They are the numerical oracle for the GPU kernels and the CPU data path of the library.
// bf16 / fp16 tensors are widened to fp32 for the whole exchange and rounded once at the end.
#pragma once

#include <cstddef>
#include <cstdint>
#include <vector>

#include "../common.h"
#include "../control/bootstrap.h"

namespace bc {

// In place: on return `data` holds the element-wise sum over all ranks (times `scale` for
// floating types when scale != 1; integer types divide by `int_divisor` when it is > 1, using
// C++ truncating division).
// `red` selects sum / prod / min / max; scale and divisor apply to sums.
void cpu_ring_allreduce(Transport& t, void* data, size_t count, DType dtype, double scale,
                        int64_t int_divisor, double deadline, ReduceOp red = ReduceOp::SUM);

// `rows[r]` rows of `row_bytes` bytes come from rank r; `out` receives all slabs in rank order.
void cpu_ring_allgatherv(Transport& t, const void* in, void* out, const std::vector<int64_t>& rows,
                         size_t row_bytes, double deadline);

// Helpers shared with tests and the GPU oracle.
void widen_to_f32(const void* src, float* dst, size_t n, DType dtype);
void narrow_from_f32(const float* src, void* dst, size_t n, DType dtype);

}  // namespace bc
