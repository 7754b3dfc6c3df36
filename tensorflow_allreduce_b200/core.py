"""Process group and the two collectives: the Python face of the native runtime.

API parity with `tensorflow/contrib/mpi_collectives` (`__init__.py:114-164`, `mpi_ops.py:62-160`):
`init / size / rank / local_rank`, `allreduce(tensor, average=True)` for dense and sparse tensors,
`allgather(tensor)` with a per-rank first dimension. Collectives are keyed by name; a name given
by only some ranks, or with mismatching dtype / shape / operation, fails on every rank with the
reference's error wording instead of hanging. Collective results carry no autograd history
(the reference marks the ops NotDifferentiable, `mpi_ops.py:135,163`).
"""
from __future__ import annotations

import ctypes as C
import itertools
import json
import os
import threading
from typing import List, Optional, Sequence

import torch

from . import _lib
from .config import Config

__all__ = [
    "CollectiveError", "init", "shutdown", "is_initialized", "size", "rank", "local_rank", "local_size",
    "allreduce", "allreduce_", "allreduce_async", "all_sum", "all_prod", "all_min", "all_max", "allgather",
    "allgather_async", "broadcast", "barrier",
    "host_allgather", "stats", "clear_stats", "on_gpu", "config", "set_fault", "check_device_status", "set_device_timing", "bus_gbs",
]


class CollectiveError(RuntimeError):
    """A collective failed: mismatched requests, a lost peer, a timeout, or use before `init()`.

    Counterpart of the reference's `FailedPreconditionError` (mpi_ops.cc:506-507, 827-833)."""


_DTYPES = {
    torch.float32: 0, torch.int32: 1, torch.int64: 2, torch.bfloat16: 3, torch.float16: 4,
    torch.float64: 5, torch.uint8: 6,
}

_state = {"config": None, "device": None}
_counter_lock = threading.Lock()
_counters = {"allreduce": itertools.count(), "allgather": itertools.count(), "blob": itertools.count(),
             "broadcast": itertools.count(), "barrier": itertools.count()}
_tokens = itertools.count(1)
_pending_allocs = {}


def _call(rc, what=""):
    try:
        return _lib.check(rc, what)
    except _lib.NativeError as e:
        raise CollectiveError(str(e)) from None


def _auto_name(kind: str) -> str:
    with _counter_lock:
        return f"{kind}.{next(_counters[kind])}"


def _env_rank_size():
    """Rank / size / local rank from the launcher's environment. torchrun's names first, then the
    Open MPI and PMI names that the reference's tests read (mpi_ops_test.py:30-62)."""
    env = os.environ
    for r, s, lr in (("RANK", "WORLD_SIZE", "LOCAL_RANK"),
                     ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_RANK"),
                     ("PMI_RANK", "PMI_SIZE", "MPI_LOCALRANKID")):
        if r in env and s in env:
            return int(env[r]), int(env[s]), (int(env[lr]) if lr in env else -1)
    return 0, 1, -1


def _resolve_port(rank_: int, size_: int, addr: str) -> int:
    """Port of the control plane's rendezvous.

    Under torchrun the port in MASTER_PORT belongs to the launcher's key-value store, so rank 0
    picks a free port and publishes it through that store. Otherwise `BC_PORT` or MASTER_PORT is
    used directly (nothing else is listening there)."""
    if "BC_PORT" in os.environ:
        return int(os.environ["BC_PORT"])
    port = int(os.environ.get("MASTER_PORT", "29500"))
    if size_ > 1 and os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "") == "True":
        import datetime

        from torch.distributed import TCPStore

        store = TCPStore(addr, port, None, False, timeout=datetime.timedelta(seconds=120), wait_for_workers=False)
        key = "bcoll/ctrl_port/" + os.environ.get("TORCHELASTIC_RUN_ID", "0") + "/" + os.environ.get("TORCHELASTIC_RESTART_COUNT", "0")
        if rank_ == 0:
            from .utils.spawn import free_port

            free = free_port()
            store.set(key, str(free))
            return free
        return int(store.get(key).decode())
    return port


def init(device=None, config: Optional[Config] = None, rank: Optional[int] = None, size: Optional[int] = None,
         addr: Optional[str] = None, port: Optional[int] = None) -> None:
    """Start the runtime of this process and join the group.

    `device` is a CUDA device (index, `torch.device`, or "cuda") to bind to, `"cpu"` for a
    host-only group, or None: then `cuda:LOCAL_RANK` is used when CUDA is available, else the CPU.
    Like the reference, the group is bound to that one device (mpi_ops.cc:900-907); CPU tensors
    are accepted by a GPU group as well.
    """
    lib = _lib.lib()
    if lib.bc_initialized():
        raise CollectiveError("init() was already called in this process")
    cfg = config or Config.from_env()
    cfg.validate()
    env_rank, env_size, env_local = _env_rank_size()
    rank_ = env_rank if rank is None else rank
    size_ = env_size if size is None else size
    addr_ = addr or os.environ.get("MASTER_ADDR", "127.0.0.1")
    port_ = port if port is not None else _resolve_port(rank_, size_, addr_)

    dev_index = -1
    if device is None:
        if torch.cuda.is_available():
            dev_index = env_local if env_local >= 0 else rank_ % max(torch.cuda.device_count(), 1)
    elif isinstance(device, int):
        dev_index = device
    else:
        d = torch.device(device)
        if d.type == "cuda":
            dev_index = d.index if d.index is not None else (env_local if env_local >= 0 else torch.cuda.current_device())
        elif d.type != "cpu":
            raise ValueError(f"unsupported device {device!r}")
    if dev_index >= 0:
        torch.cuda.set_device(dev_index)
        torch.cuda.init()

    _call(lib.bc_init(rank_, size_, env_local, addr_.encode(), port_, dev_index, cfg.timeout_s, cfg.device_timeout_s,
                      cfg.staging_mb << 20, cfg.heap_mb << 20, cfg.algo_code, cfg.one_shot_max_kb << 10,
                      cfg.nvls_min_kb << 10, int(cfg.nvls), cfg.max_blocks, cfg.symm_code, cfg.fault.encode()), "bc_init")
    _state["config"] = cfg
    _state["device"] = dev_index
    if dev_index >= 0 and cfg.overlap_blocks > 0:
        _call(lib.bc_set_option(b"overlap_blocks", cfg.overlap_blocks), "bc_set_option")
    if dev_index >= 0:
        for key, value in (("staged_pipeline", cfg.staged_pipeline), ("pipeline_min_bytes", cfg.pipeline_min_mb << 20), ("pipeline_chunk_bytes", cfg.pipeline_chunk_kb << 10),
                           ("pipeline_slots", cfg.pipeline_slots), ("pipeline_copiers", cfg.pipeline_copiers),
                           ("pipeline_reducers", cfg.pipeline_reducers), ("pipeline_rgroups", cfg.pipeline_rgroups),
                           ("pipeline_streaming", int(cfg.pipeline_streaming)),
                           ("pipeline_cgroups", cfg.pipeline_cgroups)):
            _call(lib.bc_set_option(key.encode(), int(value)), "bc_set_option")
    for k in _counters:
        _counters[k] = itertools.count()


def shutdown() -> None:
    """Leave the group: a last handshake with the other ranks, then stop the background thread."""
    lib = _lib.lib()
    if lib.bc_initialized():
        from .ops import symmetric

        _dump_stats_jsonl()
        symmetric._reset()
        _call(lib.bc_shutdown(), "bc_shutdown")
    _state["config"] = None
    _state["device"] = None


def _dump_stats_jsonl() -> None:
    """`BC_STATS_JSONL=path`: on shutdown every rank appends one JSON line per completed collective
    (rank, name, operation, algorithm, bytes, CTAs, negotiation and launch/run microseconds) to
    `path` (a `{rank}` in the path is replaced by the rank)."""
    path = os.environ.get("BC_STATS_JSONL", "")
    if not path:
        return
    try:
        r = rank()
        recs = stats()
        with open(path.replace("{rank}", str(r)), "a") as f:
            for e in recs:
                rec = {"rank": r, "name": e["name"], "op": e["op"], "algo": e["algo"], "bytes": e["bytes"],
                       "blocks": e["blocks"], "device": "cuda" if e["device"] else "cpu",
                       "negotiation_us": round(e["negotiation_us"], 1),
                       "run_us": round((e["t_done"] - e["t_negotiated"]) * 1e6, 1)}
                if "device_us" in e:
                    rec.update(device_us=round(e["device_us"], 2), bus_gbs=round(e.get("bus_gbs", 0.0), 2),
                               link_frac=round(e.get("link_frac", 0.0), 4))
                f.write(json.dumps(rec) + "\n")
    except Exception:      # observability must never break a shutdown
        pass


def is_initialized() -> bool:
    return bool(_lib.lib().bc_initialized())


def size() -> int:
    """Number of ranks (reference: `mpi_ops.py:62-71`)."""
    return _call(_lib.lib().bc_size())


def rank() -> int:
    """Rank of this process (reference: `mpi_ops.py:77-86`)."""
    return _call(_lib.lib().bc_rank())


def local_rank() -> int:
    """Rank among the processes of this host; pick the GPU with it (reference: `mpi_ops.py:104-115`)."""
    return _call(_lib.lib().bc_local_rank())


def local_size() -> int:
    return _call(_lib.lib().bc_local_size())


def on_gpu() -> bool:
    return bool(_call(_lib.lib().bc_on_gpu()))


def is_broken() -> bool:
    """True once the group has lost a peer or a deadline ran out: every later collective fails at
    once. The way on is `shutdown()` and a new `init()` among the ranks that are left."""
    return bool(_call(_lib.lib().bc_broken()))


def n_nodes() -> int:
    """Hosts of a group that runs in two levels, else 1. A group whose ranks sit on several hosts
    (the same number on each) reduces inside each host first, GPU tensors with the NVLink kernels
    and CPU tensors in shared memory, and between hosts over sockets (the reference crosses hosts
    through MPI, `ring.h:183-225`); the gradient buckets in symmetric memory and the fused update
    need all ranks on one host and are switched off then."""
    return _call(_lib.lib().bc_n_nodes())


def node_index() -> int:
    return _call(_lib.lib().bc_node_index())


def config() -> Config:
    if _state["config"] is None:
        raise CollectiveError("MPI has not been initialized; use Session or init() first.")
    return _state["config"]


def set_fault(spec: str) -> None:
    """Arm a host-side fault (tests): `drop_request`, `delay_ms=N`, `exit_before`,
    `exit_in_collective`, `close_ctrl`, each optionally followed by `:rank=R` and `:name=NAME`;
    an empty string disarms."""
    _call(_lib.lib().bc_set_fault(spec.encode()))


def check_device_status() -> None:
    """Raise if a device-side wait on a peer has timed out since `init()`."""
    st = _lib.lib().bc_device_status()
    if st & 0x20000000:
        raise CollectiveError(f"an in-place reduction found its tensor at different offsets of symmetric memory on different "
                              f"ranks (status 0x{st:08x}); its result is wrong and the group is unusable")
    if st:
        raise CollectiveError(f"a device-side wait on a peer timed out (status 0x{st:08x}); the group is unusable")


# ---- handles -----------------------------------------------------------------------------------


class Handle:
    """An in-flight collective. `wait()` returns the result tensor.

    For CUDA tensors `wait()` blocks the host only until the kernel has been enqueued on the
    library's private stream, then makes the caller's current stream wait for it on the device."""

    def __init__(self, hid: int, keep, on_gpu_: bool, result=None, finalize=None):
        self._hid = hid
        self._keep = keep
        self._gpu = on_gpu_
        self._result = result
        self._finalize = finalize
        self._done = False
        self.algo = 0

    def done(self) -> bool:
        return self._done or bool(_call(_lib.lib().bc_poll(self._hid)))

    def wait(self, timeout_s: Optional[float] = None):
        if self._done:
            return self._result
        lib = _lib.lib()
        t = timeout_s if timeout_s is not None else config().timeout_s + 10.0
        try:
            _call(lib.bc_wait(self._hid, float(t)))
            if self._gpu:
                ev = lib.bc_done_event(self._hid)
                _call(lib.bc_stream_wait_event(C.c_void_p(torch.cuda.current_stream().cuda_stream), C.c_void_p(ev)))
            self.algo = lib.bc_result_algo(self._hid)
            if self._finalize is not None:
                self._result = self._finalize(self)
        finally:
            lib.bc_release(self._hid)
            self._done = True
            self._keep = None
        return self._result


def _prep(tensor: torch.Tensor):
    if tensor.dtype not in _DTYPES:
        raise CollectiveError(f"unsupported dtype {tensor.dtype}; supported: {sorted(str(k) for k in _DTYPES)}")
    t = tensor.detach()
    if not t.is_contiguous():
        t = t.contiguous()
    if t.is_cuda and t.data_ptr() % 16 != 0:
        t = t.clone()
    return t


def _shape_array(shape: Sequence[int]):
    arr = (C.c_longlong * max(len(shape), 1))(*shape)
    return arr


def _ready_event(t: torch.Tensor):
    if not t.is_cuda:
        return None
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(t.device))
    return ev


_REDUCTIONS = {"sum": 0, "prod": 1, "min": 2, "max": 3}


def _resolve_reduction(op: str, average: Optional[bool]):
    if op not in _REDUCTIONS:
        raise ValueError(f"op must be one of {sorted(_REDUCTIONS)}, got {op!r}")
    if average is None:
        average = op == "sum"
    if average and op != "sum":
        raise ValueError("average=True goes with op='sum' only")
    return _REDUCTIONS[op], bool(average)


def allreduce_async(tensor: torch.Tensor, average: Optional[bool] = None, name: Optional[str] = None,
                    out: Optional[torch.Tensor] = None, op: str = "sum") -> Handle:
    """Start a reduction over all ranks; returns a `Handle`. `op` is "sum" (averaged unless
    `average=False`), "prod", "min" or "max"."""
    lib = _lib.lib()
    red, average = _resolve_reduction(op, average)
    name = name or _auto_name("allreduce")
    t = _prep(tensor)
    in_place = out is not None and out.data_ptr() == t.data_ptr() and out.is_contiguous()
    if out is None or (not in_place and (not out.is_contiguous() or out.shape != t.shape or out.dtype != t.dtype
                                         or (out.is_cuda and out.data_ptr() % 16 != 0))):
        result = torch.empty_like(t)
        copy_back = out
    else:
        result = out.detach()
        copy_back = None
    ev = _ready_event(t)
    zero_copy = int(in_place and t.is_cuda)
    hid = _call(lib.bc_allreduce_async(name.encode(), C.c_void_p(t.data_ptr()), C.c_void_p(result.data_ptr()), _DTYPES[t.dtype],
                                       t.dim(), _shape_array(t.shape), int(t.is_cuda), int(average), zero_copy,
                                       C.c_void_p(ev.cuda_event) if ev is not None else None, red), "allreduce")

    def fin(_h):
        if copy_back is not None:
            copy_back.copy_(result)
            return copy_back
        return result

    return Handle(hid, (t, result, ev, out), t.is_cuda, finalize=fin)


def allreduce(tensor: torch.Tensor, average: Optional[bool] = None, name: Optional[str] = None, op: str = "sum") -> torch.Tensor:
    """Sum `tensor` over all ranks, or average it (`average=True`, the default for sums).

    `op` selects the element-wise reduction: "sum" (the reference's only one,
    `mpi_collectives/ring.cc:42-50`), or "prod" / "min" / "max" as in the reference's NCCL ops
    (`contrib/nccl/python/ops/nccl_ops.py:34-137`); those are never averaged.

    Dense tensors of identical shape and dtype on every rank give a new tensor of that shape.
    Integer tensors are averaged with truncating integer division. A sparse COO tensor is reduced
    the way the reference reduces `IndexedSlices` (`__init__.py:148-158`): values and indices are
    allgathered, values divided by `size()` when averaging; repeated indices are left uncoalesced
    and sum up when the tensor is used.
    """
    if tensor.is_sparse:
        if op != "sum":
            raise ValueError("sparse tensors can only be summed or averaged")
        average = True if average is None else average
        base = name or _auto_name("allreduce")
        t = tensor.detach()
        idx = t._indices().t().contiguous()          # [nnz, ndim]
        vals = t._values().contiguous()              # [nnz, ...]
        g_vals = allgather(vals, name=base + ".values")
        g_idx = allgather(idx, name=base + ".indices")
        if average:
            g_vals = g_vals / size() if g_vals.is_floating_point() else torch.div(g_vals, size(), rounding_mode="trunc")
        return torch.sparse_coo_tensor(g_idx.t(), g_vals, t.shape)
    return allreduce_async(tensor, average=average, name=name, op=op).wait()


def grouped_allreduce(tensors, average: Optional[bool] = None, name: Optional[str] = None, op: str = "sum") -> List[torch.Tensor]:
    """`allreduce` of several dense tensors at the price of one collective per dtype and device:
    the tensors are packed into one flat buffer, reduced, and cut apart again. Every rank must
    pass tensors of the same shapes in the same order. (The reference reduces tensor by tensor,
    `mpi_collectives/__init__.py:199-220`; each of those pays a negotiation round.)"""
    tensors = list(tensors)
    name = name or _auto_name("allreduce")
    out: List[Optional[torch.Tensor]] = [None] * len(tensors)
    groups = {}
    for i, t in enumerate(tensors):
        if t.is_sparse:
            raise CollectiveError("grouped_allreduce takes dense tensors")
        groups.setdefault((t.dtype, t.device), []).append(i)
    for k, (key, idx) in enumerate(sorted(groups.items(), key=lambda kv: kv[1][0])):
        flat = torch.cat([tensors[i].detach().reshape(-1) for i in idx])
        allreduce_(flat, average=average, name=f"{name}.{k}", op=op)
        off = 0
        for i in idx:
            n = tensors[i].numel()
            out[i] = flat[off:off + n].view(tensors[i].shape)
            off += n
    return out


def all_sum(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    """Element-wise sum over all ranks (`nccl_ops.all_sum`, contrib/nccl/python/ops/nccl_ops.py:34-51)."""
    return allreduce(tensor, average=False, name=name, op="sum")


def all_prod(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    """Element-wise product over all ranks (`nccl_ops.all_prod`, nccl_ops.py:54-71)."""
    return allreduce(tensor, name=name, op="prod")


def all_min(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    """Element-wise minimum over all ranks (`nccl_ops.all_min`, nccl_ops.py:74-91)."""
    return allreduce(tensor, name=name, op="min")


def all_max(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    """Element-wise maximum over all ranks (`nccl_ops.all_max`, nccl_ops.py:94-111)."""
    return allreduce(tensor, name=name, op="max")


def allreduce_(tensor: torch.Tensor, average: Optional[bool] = None, name: Optional[str] = None, op: str = "sum") -> torch.Tensor:
    """In-place `allreduce`. A CUDA tensor that lives in symmetric memory (see `ops.symmetric`) at
    the same place on every rank is reduced where it is, with no staging copy."""
    if not tensor.is_contiguous():
        raise CollectiveError("allreduce_ needs a contiguous tensor")
    allreduce_async(tensor, average=average, name=name, out=tensor, op=op).wait()
    return tensor


@_lib.ALLOC_FN
def _alloc_callback(handle, total_rows, user, is_symm):
    # Runs on the native background thread once every rank's first dimension is known.
    try:
        ctx = _pending_allocs.get(int(user or 0))
        if ctx is None:
            return None
        t = ctx["input"]
        shape = (int(total_rows),) + tuple(t.shape[1:])
        out = None
        if t.is_cuda:
            from .ops import symmetric

            out = symmetric.try_empty(shape, t.dtype, t.device)
            if out is not None:
                is_symm[0] = 1
        if out is None:
            is_symm[0] = 0
            out = torch.empty(shape, dtype=t.dtype, device=t.device)
        ctx["out"] = out
        return out.data_ptr() if out.numel() else None
    except Exception as e:  # never let an exception cross into native code
        ctx = _pending_allocs.get(int(user or 0))
        if ctx is not None:
            ctx["error"] = e
        return None


def allgather_async(tensor: torch.Tensor, name: Optional[str] = None) -> Handle:
    """Start a concatenation along dimension 0 over all ranks; returns a `Handle`."""
    lib = _lib.lib()
    name = name or _auto_name("allgather")
    t = _prep(tensor)
    token = next(_tokens)
    ctx = {"input": t, "out": None, "error": None}
    _pending_allocs[token] = ctx
    ev = _ready_event(t)
    try:
        hid = _call(lib.bc_allgather_async(name.encode(), C.c_void_p(t.data_ptr()), _DTYPES[t.dtype], t.dim(), _shape_array(t.shape),
                                           int(t.is_cuda), _alloc_callback, C.c_void_p(token),
                                           C.c_void_p(ev.cuda_event) if ev is not None else None), "allgather")
    except Exception:
        _pending_allocs.pop(token, None)
        raise

    def fin(h):
        _pending_allocs.pop(token, None)
        if ctx["error"] is not None:
            raise CollectiveError(f"allgather output allocation failed: {ctx['error']}")
        n = size()
        dims = (C.c_longlong * n)()
        _call(lib.bc_result_dim0(h._hid, dims, n))
        h.sizes = [int(x) for x in dims]
        out = ctx["out"]
        if out is None:
            out = torch.empty((0,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
        return out

    h = Handle(hid, (t, ev, ctx), t.is_cuda, finalize=fin)
    orig_wait = h.wait

    def wait(timeout_s=None):
        try:
            return orig_wait(timeout_s)
        finally:
            _pending_allocs.pop(token, None)

    h.wait = wait
    return h


def allgather(tensor: torch.Tensor, name: Optional[str] = None) -> torch.Tensor:
    """Concatenate `tensor` from all ranks along dimension 0, in rank order.

    Ranks may differ in the first dimension (zero rows included); all other dimensions and the
    dtype must match, and the tensor must have at least one dimension
    (reference: `mpi_ops.py:138-160`, `ring.h:230-301`). One negotiation round carries every
    rank's row count, so there is no separate sizing pass. On CUDA the result lives in the
    library's symmetric heap when it fits (peers store their rows straight into it)."""
    return allgather_async(tensor, name=name).wait()


def broadcast(tensor: torch.Tensor, root: int = 0, name: Optional[str] = None) -> torch.Tensor:
    """Value of `tensor` on rank `root`, delivered to every rank (same shape and dtype everywhere).

    The reference has no broadcast; this is an allgather in which only `root` contributes rows."""
    name = name or _auto_name("broadcast")
    flat = tensor.detach().reshape(-1)
    part = flat if rank() == root else flat[:0]
    out = allgather(part, name=name)
    return out.reshape(tensor.shape)


def host_allgather(obj, name: Optional[str] = None) -> List:
    """Allgather of one small picklable Python object per rank through the control plane."""
    import pickle

    lib = _lib.lib()
    name = name or _auto_name("blob")
    data = pickle.dumps(obj)
    n = size()
    cap = max(1 << 20, len(data) * n * 4 + 4096)
    for _ in range(2):
        buf = C.create_string_buffer(cap)
        lens = (C.c_int * n)()
        rc = lib.bc_blob_gather(name.encode(), data, len(data), buf, cap, lens)
        if rc == 0:
            break
        if "too small" in _lib.last_error():
            raise CollectiveError("host_allgather payloads are limited to about 1 MiB per rank")
        _call(rc)
    out, pos = [], 0
    for r in range(n):
        out.append(pickle.loads(buf.raw[pos:pos + lens[r]]))
        pos += lens[r]
    return out


def barrier(name: Optional[str] = None) -> None:
    """Host-side barrier over the control plane."""
    host_allgather(None, name=name or _auto_name("barrier"))


def bus_gbs(op: str, nbytes: int, world: int, seconds: float) -> float:
    """Bus bandwidth in GB/s of one collective, the figure that is comparable between group sizes
    and with the link rate: allreduce `bytes / time * 2 (P - 1) / P`, allgather (`nbytes` = the
    gathered total) `bytes / time * (P - 1) / P`. One rank moves nothing: 0."""
    if seconds <= 0 or world <= 1:
        return 0.0
    factor = 2.0 * (world - 1) / world if op == "allreduce" else (world - 1) / world
    return nbytes / seconds * factor / 1e9


def set_device_timing(on: bool) -> None:
    """Switch the device timing of GPU collectives on or off: while on, every ordered launch
    (gradient buckets, `allreduce_direct_`) and every negotiated GPU allreduce is bracketed by two
    timing CUDA events on its private stream, and its record in `stats()` carries `device_us`,
    `bus_gbs` and `link_frac`. Costs two event records per launch and nothing else; the host never
    waits (a record shows up in `stats()` once its kernels have finished)."""
    _call(_lib.lib().bc_set_option(b"device_timing", int(bool(on))), "bc_set_option")


def stats() -> List[dict]:
    """One record per completed collective since the last `clear_stats()`: name, operation,
    algorithm, bytes, CTA count and host timestamps (enqueue, negotiated, done/launched). Records
    taken while device timing was on (`set_device_timing`, `Config.device_timing_every`) also
    have `device_us` (time of the kernels between two CUDA events), `bus_gbs` and `link_frac`
    (bus bandwidth as a fraction of `Config.link_gbs`), and `channel` for ordered launches."""
    raw = _lib.lib().bc_stats_json()
    if not raw:
        raise CollectiveError(_lib.last_error())
    ops = {0: "allreduce", 1: "allgather", 2: "host_gather", 3: "shutdown"}
    algos = {0: "cpu_ring", 1: "one_shot", 2: "two_shot", 3: "nvls", 4: "cpu_shm"}
    out = json.loads(raw.decode())
    world = size()
    cfg = _state.get("config")
    link = cfg.link_gbs if cfg is not None else 764.0
    for e in out:
        e["op"] = ops.get(e["op"], str(e["op"]))
        e["algo"] = algos.get(e["algo"], str(e["algo"])) if (e["device"] == 1 or e["algo"] == 4) else "cpu_ring"
        e["negotiation_us"] = (e["t_negotiated"] - e["t_enqueue"]) * 1e6
        if e.get("device_us", -1) > 0:
            e["bus_gbs"] = bus_gbs(e["op"], e["bytes"], world, e["device_us"] * 1e-6)
            e["link_frac"] = e["bus_gbs"] / link if link > 0 else 0.0
    return out


def clear_stats() -> None:
    _call(_lib.lib().bc_clear_stats())
