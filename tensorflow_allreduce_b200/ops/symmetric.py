"""Tensors in symmetric memory: device memory that every rank of the node has mapped, so that the
collective kernels can read and write it on the peers directly.

Two sources:
  * the general heap inside the first symmetric segment (`BC_HEAP_MB`), sub-allocated here with a
    first-fit free list. Allocations are local decisions (offsets may differ between ranks); the
    allgather kernel learns every peer's offset on the device. `try_empty` / `empty` use it.
  * dedicated segments created collectively with `new_segment` (gradient buckets): these are at
    the same place on every rank, which is what the in-place reductions need.

A block returns to the heap when the last tensor that views it is freed; reuse is deferred until
work queued on the freeing stream has finished.
"""
from __future__ import annotations

import collections
import ctypes as C
import threading
from typing import Optional, Sequence, Tuple

import torch

from .. import _lib

_ALIGN = 256
_TYPESTR = {
    torch.float32: "<f4", torch.int32: "<i4", torch.int64: "<i8", torch.float16: "<f2",
    torch.float64: "<f8", torch.uint8: "|u1", torch.int8: "|i1", torch.int16: "<i2",
}


class _Block:
    """Owner of a device memory range; exposes it through `__cuda_array_interface__`."""

    def __init__(self, ptr: int, nbytes: int, shape, typestr: str, on_free=None):
        self.ptr = ptr
        self.nbytes = nbytes
        self._on_free = on_free
        self.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 2, "strides": None,
        }

    def __del__(self):
        cb, self._on_free = self._on_free, None
        if cb is not None:
            try:
                cb()
            except Exception:
                pass


def tensor_from_ptr(ptr: int, shape: Sequence[int], dtype: torch.dtype, device: torch.device, on_free=None) -> torch.Tensor:
    """A tensor that aliases `ptr` (no copy). bf16 goes through a 16-bit integer view."""
    n = 1
    for s in shape:
        n *= int(s)
    if n == 0:
        return torch.empty(tuple(shape), dtype=dtype, device=device)
    if dtype == torch.bfloat16:
        blk = _Block(ptr, n * 2, (n,), "<i2", on_free)
        return torch.as_tensor(blk, device=device).view(torch.bfloat16).view(tuple(shape))
    if dtype not in _TYPESTR:
        raise TypeError(f"unsupported dtype for symmetric tensors: {dtype}")
    esize = torch.empty((), dtype=dtype).element_size()
    blk = _Block(ptr, n * esize, (n,), _TYPESTR[dtype], on_free)
    return torch.as_tensor(blk, device=device).view(tuple(shape))


class _Heap:
    """First-fit allocator over [base, base + size). Freed blocks become reusable once the event
    recorded at free time has completed."""

    def __init__(self, base: int, size: int, device: torch.device):
        self.base, self.size, self.device = base, size, device
        self.free = [(0, size)]          # (offset, length), sorted, coalesced
        # Freed blocks wait here. A block's finalizer can run at any point of any thread (even in
        # the middle of alloc() below, when the garbage collector kicks in), so it must not take
        # the lock: deque.append is atomic.
        self.limbo = collections.deque()  # (event, offset, length)
        self.lock = threading.RLock()

    def _release(self, off: int, length: int):
        self.free.append((off, length))
        self.free.sort()
        merged = []
        for o, l in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + l)
            else:
                merged.append((o, l))
        self.free = merged

    def _reap(self):
        for _ in range(len(self.limbo)):
            try:
                ev, off, length = self.limbo.popleft()
            except IndexError:
                break
            if ev is None or ev.query():
                self._release(off, length)
            else:
                self.limbo.append((ev, off, length))

    def alloc(self, nbytes: int) -> Optional[int]:
        need = (max(nbytes, 1) + _ALIGN - 1) // _ALIGN * _ALIGN
        with self.lock:
            for attempt in range(2):
                self._reap()
                for i, (o, l) in enumerate(self.free):
                    if l >= need:
                        if l == need:
                            self.free.pop(i)
                        else:
                            self.free[i] = (o + need, l - need)
                        return o
                # Out of space while freed blocks still wait for their events: wait, then retry.
                pending = [ev for ev, _, _ in list(self.limbo) if ev is not None]
                if attempt or not pending:
                    break
                for ev in pending:
                    ev.synchronize()
        return None

    def release_later(self, off: int, nbytes: int):
        need = (max(nbytes, 1) + _ALIGN - 1) // _ALIGN * _ALIGN
        ev = None
        try:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))
        except Exception:
            ev = None
        self.limbo.append((ev, off, need))


_heap: Optional[_Heap] = None
_segments = []  # (ptr, nbytes, seg_id, has_multicast)


def _reset():
    global _heap
    _heap = None
    _segments.clear()


def _get_heap(device: torch.device) -> Optional[_Heap]:
    global _heap
    if _heap is None:
        lib = _lib.lib()
        if not lib.bc_initialized() or not lib.bc_on_gpu():
            return None
        nbytes = C.c_longlong(0)
        base = lib.bc_symm_heap(C.byref(nbytes))
        if not base or nbytes.value <= 0:
            return None
        _heap = _Heap(int(base), int(nbytes.value), device)
    return _heap


def try_empty(shape: Sequence[int], dtype: torch.dtype, device) -> Optional[torch.Tensor]:
    """Uninitialised tensor in the symmetric heap, or None if it does not fit."""
    device = torch.device(device)
    heap = _get_heap(device)
    if heap is None:
        return None
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * torch.empty((), dtype=dtype).element_size()
    if nbytes == 0:
        return None
    off = heap.alloc(nbytes)
    if off is None:
        return None
    return tensor_from_ptr(heap.base + off, shape, dtype, device, on_free=lambda: heap.release_later(off, nbytes))


def empty(shape: Sequence[int], dtype: torch.dtype = torch.float32, device=None) -> torch.Tensor:
    """Uninitialised tensor in the symmetric heap; raises if the heap (`BC_HEAP_MB`) is too small."""
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    t = try_empty(shape, dtype, device)
    if t is None:
        raise RuntimeError("symmetric heap exhausted or not initialised on a GPU; raise BC_HEAP_MB or use new_segment()")
    return t


def new_segment(nbytes: int, device=None) -> Tuple[torch.Tensor, bool]:
    """Collective: every rank allocates `nbytes` of symmetric memory at the same place. Returns a
    zero-filled uint8 tensor over it and whether an NVLS multicast mapping was bound. The memory
    stays allocated until `shutdown()`."""
    lib = _lib.lib()
    device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    seg = C.c_int(0)
    mc = C.c_int(0)
    ptr = lib.bc_symm_new_segment(int(nbytes), C.byref(seg), C.byref(mc))
    if not ptr:
        raise RuntimeError(_lib.last_error())
    _segments.append((int(ptr), int(nbytes), seg.value, bool(mc.value)))
    return tensor_from_ptr(int(ptr), (int(nbytes),), torch.uint8, device), bool(mc.value)


def is_symmetric(t: torch.Tensor) -> bool:
    """True if the tensor's memory lies inside a symmetric segment of this process."""
    lib = _lib.lib()
    if not t.is_cuda or not lib.bc_initialized() or not lib.bc_on_gpu():
        return False
    return lib.bc_symm_contains(C.c_void_p(t.data_ptr()), t.numel() * t.element_size()) == 1


def describe() -> str:
    """Back end in use: "vmm", "vmm+multicast" or "ipc"."""
    s = _lib.lib().bc_symm_describe()
    return s.decode() if s else ""
