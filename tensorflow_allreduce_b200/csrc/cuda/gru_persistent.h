// Persistent bidirectional GRU layer for sm_100a: the recurrent weights of a layer stay in shared
// memory for all time steps, the per-step recurrent product runs on the 5th-generation tensor
// cores (tcgen05.mma, TF32 operands, fp32 accumulator in tensor memory), operands arrive by TMA,
// groups of blocks split the reduction length of the product among themselves, and the two
// directions run side by side in one cooperative launch.
//
// The reference's speech-model pieces are GRU cells that launch one GEMM plus elementwise
// kernels per time step (tensorflow/contrib/rnn/kernels/gru_ops.h:69-119, gru_ops_gpu.cu.cc) or
// cuDNN's RNN (contrib/cudnn_rnn/kernels/cudnn_rnn_ops.cc:738-1091); on B200 that is about
// 7000 launches of 9 us per training step of the DeepSpeech2-style benchmark model.
//
// Gate equations (PyTorch / cuDNN form, gate order r, z, n):
//   r = sigmoid(gx_r + W_hr h + b_hr)      z = sigmoid(gx_z + W_hz h + b_hz)
//   n = tanh(gx_n + r * (W_hn h + b_hn))   h' = n + z * (h - n)
// where gx = W_i x + b_i for all time steps is computed beforehand by one large library GEMM.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace bc {
namespace gpu {

struct GruDims {
  int T;        // time steps
  int B;        // batch, 1..32
  int H;        // hidden size per direction: multiple of 128, at most 1024
  int ndir;     // 1 or 2 (direction 1 runs the sequence backwards)
};

// Status bits written to status[0] by a block whose bounded wait ran out (the kernel then
// returns early; outputs are incomplete).
constexpr uint32_t kGruTimeoutGrid = 1u;      // waiting for the other blocks of its direction
constexpr uint32_t kGruTimeoutCopy = 2u;      // waiting for a TMA copy
constexpr uint32_t kGruTimeoutMma = 4u;       // waiting for the tensor core to finish

// Forward. All tensors are fp32, contiguous, on the current device, 16-byte aligned.
//   w_hh  [ndir, 3H, H]        recurrent weights
//   b_hh  [ndir, 3H]
//   gx    [T, B, ndir, 3H]     input projections including b_ih
//   y     [T, B, ndir*H]       output (also read back as h_{t-1} by the next step)
//   rsv   [ndir, T, B, 4, H]   r, z, n and (W_hn h + b_hn) of every step, for the backward pass
//   workspace                  gru_persistent_workspace_bytes(d) bytes of scratch, zeroed once when it is
//                              allocated and then reused as it is by every later call on the stream
//   sync  [256] uint32         zero on entry; counters of the step and group barriers
//   status[1] uint32           ORed with kGruTimeout* on failure
// `timeout_s` bounds every wait inside the kernel. Returns cudaErrorInvalidValue for unsupported
// dimensions and cudaErrorCooperativeLaunchTooLarge if the grid cannot be co-resident.
cudaError_t gru_persistent_forward(const GruDims& d, const float* w_hh, const float* b_hh, const float* gx, float* y, float* rsv,
                                   float* workspace, uint32_t* sync, uint32_t* status, double timeout_s, cudaStream_t stream);

// Backward through time.
//   w_hh_t [ndir, H, 3H]       transposed recurrent weights
//   y, rsv                     from the forward pass
//   dy     [T, B, ndir*H]      gradient of the output
//   dgx    [T, B, ndir, 3H]    out: gradient of gx                = (dr, dz, dn)
//   dgh    [T, B, ndir, 3H]    out: gradient of (W_h h + b_h)     = (dr, dz, dn * r)
// The caller forms dW_ih, dx, dW_hh and the bias gradients from dgx / dgh with library GEMMs.
cudaError_t gru_persistent_backward(const GruDims& d, const float* w_hh_t, const float* y, const float* rsv, const float* dy,
                                    float* dgx, float* dgh, float* workspace, uint32_t* sync, uint32_t* status, double timeout_s,
                                    cudaStream_t stream);

// Bytes of scratch memory that a forward or backward call needs for these dimensions.
size_t gru_persistent_workspace_bytes(const GruDims& d);

// Tuning aid: when `stamps` (device memory, 8 x T uint64) is non-null, block (0, 0) of every later
// launch records %globaltimer at fixed points of each step: [0] step start, [1] peers' data
// published, [2] first operand stage landed, [3] last MMA issued, [4] accumulator complete,
// [5] gate math and stores done, [6] step published. Null switches it off.
void gru_persistent_set_profile(unsigned long long* stamps);

// True if this device and these dimensions can run the persistent kernels.
bool gru_persistent_supported(const GruDims& d, int device);

}  // namespace gpu
}  // namespace bc
