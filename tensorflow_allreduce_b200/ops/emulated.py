"""A group of ranks emulated on ONE GPU.

All ranks' buffers and signal pads live on the same device and each collective is a single
cooperative launch of the production kernels (grid.y = rank). This exercises the complete
multi-rank protocol (flag barriers, peer loads and stores, slice ownership, fused epilogues) on a
machine with one GPU, where separate launches that wait on one another must never be used. The
reference's closest analogue is its NCCL test that maps several "devices" onto one GPU
(tensorflow/contrib/nccl/python/ops/nccl_ops_test.py:46).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from .. import _lib
from ..core import _DTYPES
from .symmetric import tensor_from_ptr

ALGOS = {"one_shot": 1, "two_shot": 2}


def _check(rc, what):
    if rc is None or rc < 0:
        raise RuntimeError(f"{what}: {_lib.last_error()}")
    return rc


class EmulatedGroup:
    def __init__(self, nranks: int, bytes_per_rank: int, device: Optional[int] = None):
        self.lib = _lib.lib()
        self.device = torch.cuda.current_device() if device is None else device
        self.nranks = nranks
        self.bytes_per_rank = int(bytes_per_rank)
        self._g = self.lib.bc_emu_create(self.device, nranks, self.bytes_per_rank)
        if not self._g:
            raise RuntimeError(_lib.last_error())

    def close(self):
        if self._g:
            torch.cuda.synchronize(self.device)
            self.lib.bc_emu_destroy(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def buffer(self, r: int, dtype: torch.dtype, numel: int, offset_bytes: int = 0) -> torch.Tensor:
        """View of rank r's symmetric buffer."""
        ptr = self.lib.bc_emu_buffer(self._g, r)
        return tensor_from_ptr(int(ptr) + offset_bytes, (numel,), dtype, torch.device("cuda", self.device))

    @property
    def status(self) -> int:
        return int(self.lib.bc_emu_status(self._g))

    def damaged_guard_bytes(self) -> int:
        """Every rank's buffer and signal pad lies between guard regions; this counts guard bytes
        that a kernel overwrote (0 = no out-of-bounds store). Synchronises the device."""
        return int(_check(self.lib.bc_emu_damaged_guard_bytes(self._g), "guard check"))

    def max_blocks(self) -> int:
        return int(self.lib.bc_max_emulated_blocks(self.device, self.nranks))

    def allreduce(self, count: int, dtype: torch.dtype, algo: str = "two_shot", outs: Optional[Sequence[torch.Tensor]] = None,
                  scale: float = 1.0, idiv: int = 1, blocks: int = 4, offset_bytes: int = 0, op: str = "sum",
                  srcs: Optional[Sequence[torch.Tensor]] = None, places: Optional[Sequence[int]] = None,
                  profile: Optional[torch.Tensor] = None, phase1_blocks: int = 0):
        """Reduce the first `count` elements (at `offset_bytes`) of all ranks' buffers. `outs`
        defaults to in place (two-shot only). `op`: sum, prod, min or max. `srcs`: private inputs
        that the kernel itself copies into the ranks' buffers first (the staged path of a real
        group). `places`: the offsets that the ranks claim for an in-place reduction; ranks that
        disagree set the layout bit of the status word. `profile`: int64 CUDA tensor of 5 time
        stamps written by block 0 of rank 0. `phase1_blocks` > 0 (two-shot): a mixed grid, only
        that many blocks of every rank run the cross-rank phase, all of them the local phases."""
        n = self.nranks
        arr = (C.c_void_p * n)()
        for r in range(n):
            if outs is None:
                arr[r] = int(self.lib.bc_emu_buffer(self._g, r)) + offset_bytes
            else:
                arr[r] = outs[r].data_ptr()
        sp = None
        if srcs is not None:
            sp = (C.c_void_p * n)(*[t.data_ptr() for t in srcs])
        pl = None
        if places is not None:
            pl = (C.c_ulonglong * n)(*[int(v) for v in places])
        s = torch.cuda.current_stream(self.device).cuda_stream
        _check(self.lib.bc_emu_allreduce(self._g, offset_bytes, arr, count, _DTYPES[dtype], ALGOS[algo], float(scale), int(idiv),
                                         blocks, C.c_void_p(s), {"sum": 0, "prod": 1, "min": 2, "max": 3}[op], sp, pl,
                                         C.c_void_p(profile.data_ptr()) if profile is not None else None, int(phase1_blocks)),
               "emulated allreduce")

    def clear_status(self):
        self.lib.bc_emu_clear_status(self._g)

    def fused_step(self, count: int, dtype: torch.dtype, params: Sequence[torch.Tensor], hyper: "_lib.OptHyper",
                   masters: Optional[Sequence[torch.Tensor]] = None, state1: Optional[Sequence[torch.Tensor]] = None,
                   state2: Optional[Sequence[torch.Tensor]] = None, scale: float = 1.0, blocks: int = 4, offset_bytes: int = 0,
                   phase1_blocks: int = 0):
        n = self.nranks

        def ptrs(ts):
            if ts is None:
                return None
            a = (C.c_void_p * n)()
            for r in range(n):
                a[r] = ts[r].data_ptr()
            return a

        s = torch.cuda.current_stream(self.device).cuda_stream
        _check(self.lib.bc_emu_fused_step(self._g, offset_bytes, count, _DTYPES[dtype], ptrs(params), ptrs(masters), ptrs(state1),
                                          ptrs(state2), C.byref(hyper), float(scale), blocks, C.c_void_p(s), int(phase1_blocks)),
               "emulated fused step")

    def staged_pipeline(self, srcs: Sequence[torch.Tensor], outs: Sequence[torch.Tensor], scale: float = 1.0, idiv: int = 1,
                        chunk_bytes: int = 64 << 10, slots: int = 4, lag: int = 2, reducers: int = 2, copiers: int = 3,
                        rgroups: int = 1, cgroups: int = 1, streaming: bool = False, offset_bytes: int = 0):
        """Allreduce of the private tensors `srcs[r]` into `outs[r]` (may be the same tensors) with
        the staged pipeline kernel: `copiers` blocks of every rank copy chunks into a ring of
        `slots` chunks inside the rank's buffer and finished chunks out again, `reducers` blocks
        reduce chunk after chunk with peer loads and stores; the reducers form `rgroups` groups
        and the copiers `cgroups` groups that take every groups-th chunk each (`lag`, and `slots`
        when the ring wraps, must be multiples of `cgroups`). `streaming`: reducer blocks whose
        warps split into 15 that move data without ever draining and one that waits and
        publishes. The tensors' size must be a multiple of 16 bytes."""
        n = self.nranks
        sp = (C.c_void_p * n)()
        op = (C.c_void_p * n)()
        for r in range(n):
            sp[r] = srcs[r].data_ptr()
            op[r] = outs[r].data_ptr()
        s = torch.cuda.current_stream(self.device).cuda_stream
        _check(self.lib.bc_emu_staged_pipeline(self._g, offset_bytes, sp, op, srcs[0].numel(), _DTYPES[srcs[0].dtype], float(scale),
                                               int(idiv), int(chunk_bytes), int(slots), int(lag), int(reducers), int(copiers),
                                               int(rgroups), int(cgroups), int(streaming), C.c_void_p(s)), "emulated staged pipeline")

    def allgatherv(self, ins: Sequence[torch.Tensor], out_offsets: Sequence[int], blocks: int = 2):
        """Each rank r pushes `ins[r]` into every rank's buffer at `out_offsets[that rank]` plus
        the displacement of r's slab (computed on the device)."""
        n = self.nranks
        ip = (C.c_void_p * n)()
        nb = (C.c_ulonglong * n)()
        oo = (C.c_ulonglong * n)()
        for r in range(n):
            ip[r] = ins[r].data_ptr() if ins[r].numel() else 0
            nb[r] = ins[r].numel() * ins[r].element_size()
            oo[r] = int(out_offsets[r])
        s = torch.cuda.current_stream(self.device).cuda_stream
        _check(self.lib.bc_emu_allgatherv(self._g, ip, nb, oo, blocks, C.c_void_p(s)), "emulated allgatherv")

    def barrier_probe(self, absent: int = -1, timeout_s: float = 0.5):
        """Barrier-only launch; rank `absent` does not take part, so the others run into the
        bounded wait, record a status word and return."""
        s = torch.cuda.current_stream(self.device).cuda_stream
        _check(self.lib.bc_emu_barrier_probe(self._g, absent, float(timeout_s), C.c_void_p(s)), "barrier probe")
