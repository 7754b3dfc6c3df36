"""Batch normalisation fused with the clipped ReLU behind it, for training on CUDA.

`BatchNormClip2d` is a `torch.nn.BatchNorm2d` (same parameters, buffers and `state_dict` keys)
whose output is `clamp(bn(x), 0, clip)`. In training mode on contiguous fp32 CUDA activations it
runs the library's two-pass kernels (`csrc/cuda/bn_clip.cu`): each pass reads its inputs once, so
forward moves 3 and backward 5 tensor sizes through HBM, and the clip mask of the backward pass is
recomputed from the input instead of being stored. Everywhere else (evaluation, CPU, other
dtypes or layouts) it is `F.batch_norm` followed by `F.hardtanh`.

The reference's pieces are FusedBatchNorm on cuDNN and a separate clipping kernel
(tensorflow/core/kernels/fused_batch_norm_op.cu.cc, relu_op_gpu.cu.cc).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.nn.functional as F

from .. import _lib

launch_count = 0   # fused forward and backward calls made by this process


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class _BNClip(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, eps, momentum, clip):
        n, c = x.shape[0], x.shape[1]
        hw = x.numel() // (n * c)
        y = torch.empty_like(x)
        save_mean = torch.empty(c, dtype=torch.float32, device=x.device)
        save_rstd = torch.empty(c, dtype=torch.float32, device=x.device)
        acc = torch.empty(2 * c, dtype=torch.float64, device=x.device)
        rc = _lib.lib().bc_bn_clip_forward(_ptr(x), _ptr(y), _ptr(weight), _ptr(bias), _ptr(running_mean), _ptr(running_var),
                                           _ptr(save_mean), _ptr(save_rstd), _ptr(acc), n, c, hw, float(eps), float(momentum),
                                           float(clip), C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
        _lib.check(rc, "bc_bn_clip_forward")
        global launch_count
        launch_count += 1
        ctx.save_for_backward(x, weight, bias, save_mean, save_rstd)
        ctx.clip = float(clip)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias, save_mean, save_rstd = ctx.saved_tensors
        n, c = x.shape[0], x.shape[1]
        hw = x.numel() // (n * c)
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.empty_like(weight)
        db = torch.empty_like(bias)
        acc = torch.empty(2 * c, dtype=torch.float64, device=x.device)
        rc = _lib.lib().bc_bn_clip_backward(_ptr(x), _ptr(dy), _ptr(weight), _ptr(bias), _ptr(save_mean), _ptr(save_rstd), _ptr(dx),
                                            _ptr(dw), _ptr(db), _ptr(acc), n, c, hw, ctx.clip,
                                            C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
        _lib.check(rc, "bc_bn_clip_backward")
        global launch_count
        launch_count += 1
        return dx, dw, db, None, None, None, None, None


def bn_clip(x, weight, bias, running_mean, running_var, eps: float, momentum: float, clip: float) -> torch.Tensor:
    """Training-mode `clamp(batch_norm(x), 0, clip)` on the fused kernels; `running_mean` /
    `running_var` (or None) are updated in place with weight `momentum` for the new value."""
    return _BNClip.apply(x, weight, bias, running_mean, running_var, eps, momentum, clip)


class BatchNormClip2d(torch.nn.BatchNorm2d):
    """`BatchNorm2d` followed by `Hardtanh(0, clip)` in one module (and, in training on CUDA, in
    two kernels per pass)."""

    def __init__(self, num_features: int, clip: float = 20.0, **kw):
        super().__init__(num_features, **kw)
        self.clip = float(clip)

    def _fused_ok(self, x: torch.Tensor) -> bool:
        return (self.training and x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and x.is_contiguous() and self.affine
                and self.weight.dtype == torch.float32 and self.momentum is not None
                and (not self.track_running_stats or self.running_mean is not None) and x.numel() > 0
                and x.numel() // (x.shape[0] * x.shape[1]) < 2 ** 31)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self._fused_ok(x):
            return F.hardtanh(super().forward(x), 0.0, self.clip)
        if self.track_running_stats and self.num_batches_tracked is not None:
            self.num_batches_tracked.add_(1)
        rm = self.running_mean if self.track_running_stats else None
        rv = self.running_var if self.track_running_stats else None
        return bn_clip(x, self.weight, self.bias, rm, rv, self.eps, self.momentum, self.clip)

    def extra_repr(self) -> str:
        return super().extra_repr() + f", clip={self.clip}"
