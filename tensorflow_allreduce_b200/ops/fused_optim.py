"""Hyper-parameter packing for the fused reduce+update kernels and plain-PyTorch references of
the same formulas (used by tests as the fp32 oracle).

Formulas: TensorFlow `ApplyMomentum` / `ApplyAdam`
(tensorflow/core/kernels/training_ops_gpu.cu.cc:82-145, python/training/adam.py:50-60) and
`torch.optim.SGD` / `Adam` / `AdamW`."""
from __future__ import annotations

from .. import _lib


def sgd_hyper(lr, momentum=0.0, weight_decay=0.0, dampening=0.0, nesterov=False, first_step=False, zero_grad=False) -> _lib.OptHyper:
    h = _lib.OptHyper()
    h.kind = 1
    h.lr, h.momentum, h.weight_decay, h.dampening = lr, momentum, weight_decay, dampening
    h.nesterov, h.first_step, h.zero_grad = int(nesterov), int(first_step), int(zero_grad)
    return h


def adam_hyper(lr, step, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled=True, tf_epsilon_hat=False, zero_grad=False) -> _lib.OptHyper:
    h = _lib.OptHyper()
    h.kind = 2
    h.lr, h.weight_decay = lr, weight_decay
    h.beta1, h.beta2, h.eps = betas[0], betas[1], eps
    h.bias_c1 = 1.0 - betas[0] ** step
    h.bias_c2 = 1.0 - betas[1] ** step
    h.decoupled_wd, h.tf_epsilon_hat, h.zero_grad = int(decoupled), int(tf_epsilon_hat), int(zero_grad)
    return h


def sgd_reference(p, g, buf, lr, momentum=0.0, weight_decay=0.0, dampening=0.0, nesterov=False, first_step=False):
    """fp32 reference; returns (p, buf)."""
    p, g = p.float(), g.float()
    if weight_decay:
        g = g + weight_decay * p
    if momentum:
        buf = g.clone() if first_step else momentum * buf.float() + (1 - dampening) * g
        g = g + momentum * buf if nesterov else buf
    return p - lr * g, buf


def adam_reference(p, g, m, v, lr, step, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, decoupled=True, tf_epsilon_hat=False):
    """fp32 reference; returns (p, m, v)."""
    p, g, m, v = p.float(), g.float(), m.float(), v.float()
    b1, b2 = betas
    if weight_decay:
        if decoupled:
            p = p * (1 - lr * weight_decay)
        else:
            g = g + weight_decay * p
    m = b1 * m + (1 - b1) * g
    v = b2 * v + (1 - b2) * g * g
    bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
    if tf_epsilon_hat:
        p = p - lr * (bc2 ** 0.5) / bc1 * m / (v.sqrt() + eps)
    else:
        p = p - (lr / bc1) * m / (v.sqrt() / (bc2 ** 0.5) + eps)
    return p, m, v
