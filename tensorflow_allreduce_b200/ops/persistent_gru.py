"""Persistent GRU layers on the tcgen05 / TMA kernels of `csrc/cuda/gru_persistent.cu`.

A GRU layer is split the usual way into the input projections of all time steps (one library
GEMM) and the recurrence. The recurrence of both directions of a layer runs in ONE cooperative
kernel launch whose blocks keep their slice of the recurrent weights in shared memory for the
whole sequence; see the kernel file for the design. The reference's counterparts launch at least
one GEMM and one elementwise kernel per time step (tensorflow/contrib/rnn/kernels/gru_ops.h:69-119,
contrib/cudnn_rnn/kernels/cudnn_rnn_ops.cc:738-1091).

`gru_forward(rnn, x)` evaluates a `torch.nn.GRU` with its own parameters (same gate order and
equations as `torch.nn.GRU`, zero initial state, time-major input) and is differentiable, so a
model keeps its `nn.GRU` module, parameters and `state_dict` and only swaps the call.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Optional

import torch

from .. import _lib

_TIMEOUT_S = float(os.environ.get("BC_GRU_TIMEOUT_S", "10"))   # bound of every wait inside the kernels
_status: Dict[int, torch.Tensor] = {}
launch_count = 0   # persistent kernels launched by this process (forward and backward)


def _status_word(device: torch.device) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[idx] = t
    return t


_work: Dict[int, torch.Tensor] = {}


def _workspace(device: torch.device, T: int, B: int, H: int, nd: int) -> torch.Tensor:
    """Scratch through which the blocks of a group exchange their partial sums (coalesced 16-byte
    tiles; a release and a per-step counter in `sync` tell the readers when a tile is complete, so
    the contents need no initial value). It is reused by every launch; kernels on one stream use
    it one after the other, so one buffer per device is enough."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    need = int(_lib.lib().bc_gru_workspace_bytes(T, B, H, nd))
    t = _work.get(idx)
    if t is None or t.numel() * 4 < need:
        t = torch.zeros(max(need // 4, 4), dtype=torch.float32, device=device)
        _work[idx] = t
    return t


def check_status(device=None) -> None:
    """Raise if a persistent GRU kernel on `device` gave up on a bounded wait since the last
    check (this synchronises with the device)."""
    for idx, t in list(_status.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code = int(t.item())
        if code:
            t.zero_()
            raise RuntimeError(f"a persistent GRU kernel timed out on cuda:{idx} (status 0x{code:x}); its outputs are incomplete")


def supported(T: int, B: int, H: int, ndir: int, device=None) -> bool:
    """Can the persistent kernels run these dimensions on this device? (B <= 32, H a multiple of
    128 up to 1024, a compute-capability-10 GPU with enough SMs for H/16 blocks per direction.)"""
    if not torch.cuda.is_available():
        return False
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    return _lib.lib().bc_gru_supported(idx, int(T), int(B), int(H), int(ndir)) == 1


def _ptr(t: Optional[torch.Tensor]):
    return C.c_void_p(t.data_ptr()) if t is not None else None


class _GRULayer(torch.autograd.Function):
    """One (bi)directional GRU layer. w_ih [nd, 3H, I], w_hh [nd, 3H, H], b_ih / b_hh [nd, 3H]."""

    @staticmethod
    def forward(ctx, x, w_ih, w_hh, b_ih, b_hh):
        T, B, I = x.shape
        nd, H3, H = w_hh.shape
        lib = _lib.lib()
        x2 = x.reshape(T * B, I)
        # input projections of both directions in one GEMM: [T*B, nd*3H]
        gx = torch.addmm(b_ih.reshape(-1), x2, w_ih.reshape(nd * H3, I).t())
        y = torch.empty(T, B, nd * H, dtype=torch.float32, device=x.device)
        rsv = torch.empty(nd, T, B, 4, H, dtype=torch.float32, device=x.device)
        sync = torch.zeros(256, dtype=torch.int32, device=x.device)
        work = _workspace(x.device, T, B, H, nd)
        status = _status_word(x.device)
        w_hh_c = w_hh.contiguous()
        rc = lib.bc_gru_forward(T, B, H, nd, _ptr(w_hh_c), _ptr(b_hh.contiguous()), _ptr(gx), _ptr(y), _ptr(rsv), _ptr(work), _ptr(sync),
                                _ptr(status), _TIMEOUT_S, C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
        _lib.check(rc, "bc_gru_forward")
        global launch_count
        launch_count += 1
        ctx.save_for_backward(x, w_ih, w_hh_c, y, rsv)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w_ih, w_hh, y, rsv = ctx.saved_tensors
        T, B, I = x.shape
        nd, H3, H = w_hh.shape
        lib = _lib.lib()
        dy = dy.contiguous()
        dgx = torch.empty(T, B, nd, H3, dtype=torch.float32, device=x.device)
        dgh = torch.empty(T, B, nd, H3, dtype=torch.float32, device=x.device)
        sync = torch.zeros(256, dtype=torch.int32, device=x.device)
        work = _workspace(x.device, T, B, H, nd)
        w_hh_t = w_hh.transpose(1, 2).contiguous()            # [nd, H, 3H]
        rc = lib.bc_gru_backward(T, B, H, nd, _ptr(w_hh_t), _ptr(y), _ptr(rsv), _ptr(dy), _ptr(dgx), _ptr(dgh), _ptr(work), _ptr(sync),
                                 _ptr(_status_word(x.device)), _TIMEOUT_S, C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
        _lib.check(rc, "bc_gru_backward")
        global launch_count
        launch_count += 1
        x2 = x.reshape(T * B, I)
        dgx2 = dgx.view(T * B, nd * H3)
        dx = dw_ih = db_ih = dw_hh = db_hh = None
        if ctx.needs_input_grad[0]:
            dx = (dgx2 @ w_ih.reshape(nd * H3, I)).view(T, B, I)
        if ctx.needs_input_grad[1]:
            dw_ih = (dgx2.t() @ x2).view(nd, H3, I)
        if ctx.needs_input_grad[3]:
            db_ih = dgx2.sum(0).view(nd, H3)
        if ctx.needs_input_grad[2]:
            dw_hh = torch.empty_like(w_hh)
            if T > 1:
                # direction 0: h_{t-1} = y[t-1]; direction 1 runs backwards in time: h_prev = y[t+1]
                torch.mm(dgh[1:, :, 0, :].reshape(-1, H3).t(), y[:-1, :, :H].reshape(-1, H), out=dw_hh[0])
                if nd == 2:
                    torch.mm(dgh[:-1, :, 1, :].reshape(-1, H3).t(), y[1:, :, H:].reshape(-1, H), out=dw_hh[1])
            else:
                dw_hh.zero_()
        if ctx.needs_input_grad[4]:
            db_hh = dgh.view(T * B, nd * H3).sum(0).view(nd, H3)
        return dx, dw_ih, dw_hh, db_ih, db_hh


def gru_layer(x: torch.Tensor, w_ih: torch.Tensor, w_hh: torch.Tensor, b_ih: torch.Tensor, b_hh: torch.Tensor) -> torch.Tensor:
    """One GRU layer over a time-major fp32 sequence x [T, B, I] with zero initial state.
    Parameters are stacked over the directions (1 or 2). Returns [T, B, ndir * H]."""
    return _GRULayer.apply(x.contiguous(), w_ih, w_hh, b_ih, b_hh)


def gru_forward(rnn: torch.nn.GRU, x: torch.Tensor) -> torch.Tensor:
    """`rnn(x)[0]` for a time-major `torch.nn.GRU` with biases and zero initial state, computed by
    the persistent kernels. Raises if the module or the shapes are not supported (use `supported`)."""
    if rnn.batch_first or not rnn.bias or rnn.dropout != 0.0 or getattr(rnn, "proj_size", 0):
        raise ValueError("gru_forward needs a time-major nn.GRU with biases, no dropout and no projection")
    nd = 2 if rnn.bidirectional else 1
    out = x
    for layer in range(rnn.num_layers):
        sfx = [f"_l{layer}"] + ([f"_l{layer}_reverse"] if nd == 2 else [])
        w_ih = torch.stack([getattr(rnn, "weight_ih" + s) for s in sfx])
        w_hh = torch.stack([getattr(rnn, "weight_hh" + s) for s in sfx])
        b_ih = torch.stack([getattr(rnn, "bias_ih" + s) for s in sfx])
        b_hh = torch.stack([getattr(rnn, "bias_hh" + s) for s in sfx])
        out = gru_layer(out, w_ih, w_hh, b_ih, b_hh)
    return out
