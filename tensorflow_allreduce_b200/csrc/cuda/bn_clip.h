// Training-mode batch normalisation of NCHW fp32 activations fused with the clipped ReLU that
// follows it (y = clamp(bn(x), 0, clip_hi)), forward and backward; see bn_clip.cu.
//
// Reference counterparts: FusedBatchNorm (cuDNN plus the helper kernels of
// tensorflow/core/kernels/fused_batch_norm_op.cu.cc:26-60) and the separate clipping kernel
// (core/kernels/relu_op_gpu.cu.cc).
#pragma once

#include <cuda_runtime.h>

namespace bc {
namespace gpu {

// x, y: [N, C, HW] contiguous fp32 (HW = H * W); gamma, beta, save_mean, save_rstd: [C];
// running_mean / running_var: [C] or null (then no running statistics are kept); acc: scratch of
// 2 * C doubles. Batch statistics are biased (divided by N * HW), the running variance takes the
// unbiased estimate, both as torch.nn.BatchNorm2d does; momentum is the weight of the new value.
cudaError_t bn_clip_forward(const float* x, float* y, const float* gamma, const float* beta, float* running_mean, float* running_var,
                            float* save_mean, float* save_rstd, double* acc, int N, int C, int HW, float eps, float momentum,
                            float clip_hi, cudaStream_t stream);

// dx: [N, C, HW]; dgamma, dbeta: [C]. The clip mask is recomputed from x, so the forward output
// is not needed.
cudaError_t bn_clip_backward(const float* x, const float* dy, const float* gamma, const float* beta, const float* save_mean,
                             const float* save_rstd, float* dx, float* dgamma, float* dbeta, double* acc, int N, int C, int HW,
                             float clip_hi, cudaStream_t stream);

}  // namespace gpu
}  // namespace bc
