"""Ordered collectives without negotiation.

`allreduce_direct_` launches the reduction kernel at once on one of the library's private
streams. There is no name and no coordinator round trip: every rank must issue the same sequence
of direct calls (per channel), exactly as with NCCL. This is the path `DistributedOptimizer`
uses for its gradient buckets after the bucket layout has been agreed once.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from ..core import _DTYPES, CollectiveError

_events = {}


def _pair(channel):
    if channel not in _events:
        _events[channel] = (torch.cuda.Event(), torch.cuda.Event())
        # give both events a native handle
        for e in _events[channel]:
            e.record(torch.cuda.current_stream())
    return _events[channel]


def allreduce_direct_(tensor: torch.Tensor, average: bool = False, channel: int = 2) -> torch.Tensor:
    """In-place sum (or average) of a contiguous, 16-byte aligned CUDA tensor. Tensors in
    symmetric memory are reduced where they are; others go through the staging area."""
    if not (tensor.is_cuda and tensor.is_contiguous() and tensor.data_ptr() % 16 == 0):
        raise CollectiveError("allreduce_direct_ needs a contiguous, 16-byte aligned CUDA tensor")
    lib = _lib.lib()
    ready, done = _pair(channel)
    cur = torch.cuda.current_stream()
    ready.record(cur)
    rc = lib.bc_allreduce_direct(channel, C.c_void_p(tensor.data_ptr()), C.c_void_p(tensor.data_ptr()), tensor.numel(),
                                 _DTYPES[tensor.dtype], int(average), C.c_void_p(ready.cuda_event), C.c_void_p(done.cuda_event))
    if rc < 0:
        raise CollectiveError(_lib.last_error())
    cur.wait_event(done)
    return tensor


def allgatherv_direct(tensor: torch.Tensor, out: torch.Tensor, sizes_out: torch.Tensor = None, channel: int = 2) -> torch.Tensor:
    """Concatenate every rank's `tensor` (rows may differ per rank) into `out`, a tensor of equal
    capacity on all ranks that lives in the symmetric heap (`ops.symmetric.empty`). Nothing about
    the sizes passes through the host: each rank publishes its byte count on the device and the
    kernel computes the displacements there. `sizes_out` (int64 CUDA tensor, one entry per rank)
    receives the byte counts; rows beyond their sum are left untouched."""
    if not (tensor.is_cuda and tensor.is_contiguous() and out.is_contiguous()):
        raise CollectiveError("allgatherv_direct needs contiguous CUDA tensors")
    lib = _lib.lib()
    ready, done = _pair(channel)
    cur = torch.cuda.current_stream()
    ready.record(cur)
    rc = lib.bc_allgatherv_direct(channel, C.c_void_p(tensor.data_ptr() if tensor.numel() else 0), tensor.numel() * tensor.element_size(),
                                  C.c_void_p(out.data_ptr()), out.numel() * out.element_size(),
                                  C.c_void_p(sizes_out.data_ptr()) if sizes_out is not None else None,
                                  C.c_void_p(ready.cuda_event), C.c_void_p(done.cuda_event))
    if rc < 0:
        raise CollectiveError(_lib.last_error())
    cur.wait_event(done)
    return out
