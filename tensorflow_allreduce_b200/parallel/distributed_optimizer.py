"""`DistributedOptimizer`: wraps a `torch.optim.Optimizer` and averages every gradient over all
ranks before the update is applied.

Reference: `tensorflow/contrib/mpi_collectives/__init__.py:167-234` (a `tf.train.Optimizer` whose
`compute_gradients` allreduces each gradient and which forwards everything else to the wrapped
optimizer; one collective per tensor, no bucketing, averaging and the update as separate kernels).

What is different here, on a CUDA group:
  * gradients of all parameters live in flat buckets inside symmetric memory (`p.grad` is a view
    of its bucket), so a bucket is reduced where it is, with no gather copy and no staging;
  * parameters that share one storage (the weights of an `nn.GRU` after `flatten_parameters()`)
    keep their relative layout, but the flat range is cut at parameter boundaries into buckets
    of about `bucket_mb`, so the gradients of one layer travel while the next layer's backward
    still runs (`plan_buckets`);
  * a bucket is launched from an autograd hook as soon as its last gradient has been accumulated,
    on the library's private stream, behind an event recorded on the compute stream: the
    reduction overlaps the rest of the backward pass. Buckets are launched strictly in bucket
    order, which is identical on all ranks, so this path needs no negotiation per step;
  * for `torch.optim.SGD`, `Adam` and `AdamW` the averaging, the optimizer update, the 16-bit ->
    fp32 master-weight handling and the zeroing of the gradient are fused into the reduction
    kernel (`bc_fused_step`); other optimizers get averaged gradients in `p.grad` and then run
    their own `step()`.

Two consequences of the fused update that differ from `torch.optim`:
  * the update of a bucket is applied by the kernel that reduces it, i.e. DURING `backward()`.
    `step()` only waits for it. Not calling `step()` (say after an overflow check) does not undo
    or prevent the update; a second `backward()` before `step()` outside `no_sync()` is an error;
  * every parameter is updated in every step. A parameter that received no gradient in a step
    counts as having a zero gradient (weight decay and momentum still move it), where
    `torch.optim` skips parameters whose `grad` is None. `fused=False` has the same behaviour
    because `p.grad` is a view of the bucket and never None.
On a CPU group every gradient is allreduced by name through the negotiated path, then the wrapped
optimizer steps.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from typing import List, Optional

import torch

from .. import _lib, core
from ..ops import symmetric

_FUSED_CHANNEL = 1
_ALIGN_BYTES = 256


class _Unit:
    """Parameters that must keep their relative placement (they share one storage, as the weights
    of a cuDNN RNN do after `flatten_parameters()`), or a single parameter."""

    def __init__(self, params, offsets, numel):
        self.params = params      # list of Parameter
        self.offsets = offsets    # element offset of each parameter inside the unit
        self.numel = numel        # elements spanned by the unit


class _Arena:
    """All parameters of one parameter group and dtype in ONE flat element layout, shared by the
    gradients (symmetric memory), the parameters, the master weights and the optimizer state.
    Buckets are ranges of an arena."""

    def __init__(self, group_index, dtype):
        self.group_index = group_index
        self.dtype = dtype
        self.numel = 0
        self.units = []           # (unit, element offset inside the arena)
        self.grad = self.param = self.master = self.state1 = self.state2 = None


class _Bucket:
    """One launch: the elements [lo, hi) of an arena."""

    def __init__(self, index, arena, lo, hi, slots):
        self.index = index
        self.arena = arena
        self.group_index = arena.group_index
        self.dtype = arena.dtype
        self.lo, self.hi = lo, hi
        self.numel = hi - lo
        self.slots = slots        # (parameter, element offset inside the bucket)
        self.params = [p for p, _ in slots]
        self.pending = len(slots)
        self.launched = False
        self.dirty = False        # gradients were accumulated into it after it had been reduced
        self.grad = None          # flat views, set after allocation
        self.param = None
        self.master = None
        self.state1 = None
        self.state2 = None
        self.ready_event = None
        self.done_event = None


def _split_unit(members, numel: int, esize: int, target: int, off: int, pack: int):
    """Launch ranges of one unit that is larger than the target (see `plan_buckets`).

    1. Ready groups: the members in the order in which backward is expected to produce their
       gradients (reverse registration order) are collected into groups of about `target` bytes
       (a group is closed once it holds 3/4 of the target, and before it would exceed 5/4).
    2. Runs: neighbours in the storage that belong to the same group form a run; a boundary that
       is not on a 16-byte boundary cannot be cut and joins its two sides.
    3. A run of less than 1/16 of the target joins a neighbouring run that is ready no earlier
       than itself, so the big run loses nothing and one tiny launch disappears. (A storage that
       keeps all matrices first and all bias vectors last ends up with one small range for the
       bias vectors, launched last, instead of delaying a matrix range of every layer.)
    Returns `[(lo, hi, [(key, offset inside the range), ...]), ...]` in launch order.
    """
    order = sorted(members, key=lambda m: m[1])
    gid, g, acc = {}, 0, 0
    for key, _, n, _ in sorted(members, key=lambda m: -m[3]):
        if acc > 0 and (acc + n) * esize > target + target // 4:
            g, acc = g + 1, 0
        gid[key] = g
        acc += n
        if acc * esize >= target - target // 4:
            g, acc = g + 1, 0
    runs = []                                   # [first member index, last member index, group]
    for i, (key, o, _, _) in enumerate(order):
        if runs and (runs[-1][2] == gid[key] or (off + o) % pack != 0):
            runs[-1][1] = i
            runs[-1][2] = max(runs[-1][2], gid[key])
        else:
            runs.append([i, i, gid[key]])

    def start(r):
        return order[r[0]][1] if r[0] > 0 else 0

    def size(k):
        hi = start(runs[k + 1]) if k + 1 < len(runs) else numel
        return (hi - start(runs[k])) * esize

    small = max(1, target // 16)
    merged = True
    while merged and len(runs) > 1:
        merged = False
        for k in range(len(runs)):
            if size(k) >= small:
                continue
            cands = [j for j in (k - 1, k + 1) if 0 <= j < len(runs) and runs[j][2] >= runs[k][2]]
            if not cands:
                continue
            j = min(cands, key=lambda c: runs[c][2])
            lo_k, hi_k = min(k, j), max(k, j)
            runs[lo_k] = [runs[lo_k][0], runs[hi_k][1], runs[j][2]]
            del runs[hi_k]
            merged = True
            break
    out = []
    for k, r in enumerate(runs):
        lo = start(r)
        hi = start(runs[k + 1]) if k + 1 < len(runs) else numel
        out.append((r[2], -lo, (off + lo, off + hi, [(order[i][0], order[i][1] - lo) for i in range(r[0], r[1] + 1)])))
    out.sort(key=lambda t: (t[0], t[1]))
    return [t[2] for t in out]


def plan_buckets(units, esize: int, bucket_bytes: int, align_bytes: int = 256):
    """Place `units` one after the other in a flat arena, each on an `align_bytes` boundary, and
    cut the arena into launch ranges of about `bucket_bytes`.

    A unit is `(numel, members)`: the elements it spans and its members `(key, offset, numel,
    registration index)` with their element offsets inside it. The units come in the order in
    which backward is expected to finish them (reverse registration order).

    Small units are packed into a range until it is full (a unit larger than the limit gets a
    range of its own). A unit of several members that exceeds the limit is cut at member
    boundaries (`_split_unit`): there `bucket_bytes` is a target that a range may miss by a
    quarter either way, so that matrices of 24 + 12 MiB end up together under a 32 MiB target;
    storage between two members goes with the member before it.

    Returns `(total_elements, placements, ranges)`: `placements[i]` is the arena offset of unit i
    and `ranges` is a list of `(lo, hi, [(key, offset inside the range), ...])` in launch order.
    Pure arithmetic, no tensors: every rank computes the same plan from the same shapes.
    """
    align = max(1, align_bytes // esize)
    pack = max(1, 16 // esize)
    placements, ranges = [], []
    pos = 0
    cur = None                    # open range of small units: [lo, hi, slots]

    def close():
        nonlocal cur
        if cur is not None and cur[2]:
            ranges.append((cur[0], cur[1], cur[2]))
        cur = None

    for numel, members in units:
        off = (pos + align - 1) // align * align
        placements.append(off)
        pos = off + numel
        if len(members) > 1 and numel * esize > bucket_bytes:
            close()
            ranges.extend(_split_unit(members, numel, esize, bucket_bytes, off, pack))
            continue
        if cur is not None and (off + numel - cur[0]) * esize > bucket_bytes:
            close()
        if cur is None:
            cur = [off, off, []]
        cur[2].extend((m[0], off + m[1] - cur[0]) for m in members)
        cur[1] = off + numel
    close()
    return pos, placements, ranges


class _FlatBucket:
    """Dense gradients of one dtype and device that travel as one flat buffer."""

    def __init__(self, index, params):
        self.index = index
        self.params = params
        self.offsets, n = [], 0
        for p in params:
            self.offsets.append(n)
            n += p.numel()
        self.buf = torch.zeros(n, dtype=params[0].dtype, device=params[0].device)
        self.filled = set()
        self.handle = None
        self.dirty = False


def _chunks_by_bytes(tensors, limit: int):
    """Consecutive runs of `tensors` whose sizes add up to at most `limit` bytes (a tensor larger
    than that forms a run of its own)."""
    run, size = [], 0
    for t in tensors:
        b = t.numel() * t.element_size()
        if run and size + b > limit:
            yield run
            run, size = [], 0
        run.append(t)
        size += b
    if run:
        yield run


def _fused_kind(opt) -> int:
    """1 = SGD, 2 = Adam/AdamW when the wrapped optimizer's options are covered by the fused
    kernels, else 0."""
    t = type(opt)
    for g in opt.param_groups:
        if g.get("maximize", False) or g.get("capturable", False) or g.get("differentiable", False):
            return 0
    if t is torch.optim.SGD:
        return 1
    if t in (torch.optim.Adam, torch.optim.AdamW):
        if any(g.get("amsgrad", False) for g in opt.param_groups):
            return 0
        if any(isinstance(g["lr"], torch.Tensor) for g in opt.param_groups):
            return 0
        return 2
    return 0


class DistributedOptimizer(torch.optim.Optimizer):
    """Gradient-averaging wrapper; use it exactly like the optimizer it wraps.

    Args:
      optimizer: the optimizer that computes the update.
      name: prefix of the collective names; defaults to "Distributed" + the optimizer's type name.
      use_locking: accepted for signature compatibility with the reference; unused.
      fused: None = fuse when supported; False = always run the wrapped optimizer's own step.
      bucket_mb: bucket size in MiB (default from `Config.bucket_mb`).
      master_weights: keep fp32 master copies for bf16/fp16 parameters (default True).
      fused_zero_grad: let the fused kernel overwrite consumed gradients with zeros, so that
        `zero_grad()` costs nothing (default True; set False to inspect gradients after `step()`).
      tf_adam: use TensorFlow's "epsilon hat" Adam formula instead of PyTorch's.
      timing_every: time the bucket launches of every Nth step on the device (CUDA events on the
        private stream; `stats()` then holds one record per bucket with `device_us`, `bus_gbs` and
        `link_frac`). Default from `Config.device_timing_every`; 0 = never.

    Construction is collective on a CUDA group (symmetric memory is allocated): every rank must
    build its optimizers in the same order over identically shaped models.
    """

    _instances = 0

    def __init__(self, optimizer: torch.optim.Optimizer, name: Optional[str] = None, use_locking: bool = False, *,
                 fused: Optional[bool] = None, bucket_mb: Optional[float] = None, master_weights: bool = True,
                 fused_zero_grad: bool = True, tf_adam: bool = False, timing_every: Optional[int] = None):
        if not core.is_initialized():
            raise core.CollectiveError("MPI has not been initialized; use Session or init() first.")
        self._optimizer = optimizer
        self.name = name or "Distributed{}".format(type(optimizer).__name__)
        self._use_locking = use_locking
        super().__init__(optimizer.param_groups, optimizer.defaults)
        self.state = optimizer.state
        self._world = core.size()
        self._sync = True
        self._synced = False     # synchronize() has already averaged this iteration's gradients
        self._tf_adam = tf_adam
        self._fused_zero_grad = fused_zero_grad
        self._master_weights = master_weights
        self._hooks = []
        self._step_count = [0 for _ in self.param_groups]
        self._momentum_live = [False for _ in self.param_groups]   # SGD: the momentum buffers hold values to continue from
        params = [p for g in self.param_groups for p in g["params"] if p.requires_grad]
        self._all_params = params
        # Gradient buckets in symmetric memory and ordered launches need all ranks on one host; a
        # group over several hosts averages flat copies of the gradients through the negotiated
        # (two-level) allreduce and runs the wrapped optimizer's own step.
        self._gpu = core.on_gpu() and core.n_nodes() == 1 and len(params) > 0 and all(p.is_cuda for p in params)
        kind = _fused_kind(optimizer) if (fused is None or fused) else 0
        if fused and not kind:
            raise ValueError(f"{type(optimizer).__name__} with these options has no fused update")
        self._kind = kind if self._gpu else 0
        self._buckets: List[_Bucket] = []
        self._next_bucket = 0
        self._launched_any = False
        self._backward_end_queued = False
        self._iteration = 0
        self._timing_every = int(timing_every if timing_every is not None else core.config().device_timing_every) if core.on_gpu() else 0
        self._timing_on = False
        self.launch_count = 0   # collective kernels launched by this optimizer so far
        self._flat: List[_FlatBucket] = []     # groups in two levels: flat copies reduced while backward runs
        if self._gpu:
            cfg = core.config()
            self._bucket_bytes = int((bucket_mb if bucket_mb is not None else cfg.bucket_mb) * (1 << 20))
            self._build_buckets()
            self._verify_layout()
            for p in params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad_ready))
        elif core.n_nodes() > 1 and params:
            limit = int((bucket_mb if bucket_mb is not None else core.config().bucket_mb) * (1 << 20))
            self._build_flat_buckets(params, limit)
            for p in params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_flat_grad_ready))

    # ---- layout ------------------------------------------------------------------------------

    def _make_units(self, group_params):
        by_storage = {}
        for p in group_params:
            key = (p.untyped_storage().data_ptr(), p.dtype)
            by_storage.setdefault(key, []).append(p)
        units, seen = [], set()
        for p in group_params:
            key = (p.untyped_storage().data_ptr(), p.dtype)
            if key in seen:
                continue
            seen.add(key)
            ps = by_storage[key]
            if len(ps) == 1 or not all(q.is_contiguous() for q in ps):
                for q in ps:
                    units.append(_Unit([q], [0], q.numel()))
                continue
            lo = min(q.storage_offset() for q in ps)
            hi = max(q.storage_offset() + q.numel() for q in ps)
            units.append(_Unit(ps, [q.storage_offset() - lo for q in ps], hi - lo))
        return units

    def _build_buckets(self):
        dev = self._all_params[0].device
        arenas: List[_Arena] = []
        buckets: List[_Bucket] = []
        for gi, g in enumerate(self.param_groups):
            ps = [p for p in g["params"] if p.requires_grad]
            for dtype in sorted({p.dtype for p in ps}, key=str):
                units = self._make_units([p for p in ps if p.dtype == dtype])
                units.reverse()                                   # gradients become ready roughly in reverse parameter order
                esize = torch.empty((), dtype=dtype).element_size()
                arena = _Arena(gi, dtype)
                reg = {q: i for i, q in enumerate(ps)}
                spec = [(u.numel, [(q, o, q.numel(), reg[q]) for q, o in zip(u.params, u.offsets)]) for u in units]
                arena.numel, placements, ranges = plan_buckets(spec, esize, self._bucket_bytes, _ALIGN_BYTES)
                arena.units = list(zip(units, placements))
                arenas.append(arena)
                for lo, hi, slots in ranges:
                    buckets.append(_Bucket(len(buckets), arena, lo, hi, slots))
        # One symmetric segment for all gradients; parameters and state in ordinary memory.
        offs, total = [], 0
        for ar in arenas:
            esize = torch.empty((), dtype=ar.dtype).element_size()
            total = (total + _ALIGN_BYTES - 1) // _ALIGN_BYTES * _ALIGN_BYTES
            offs.append(total)
            total += ar.numel * esize
        seg, self._has_multicast = symmetric.new_segment(max(total, _ALIGN_BYTES), dev)
        self._grad_segment = seg
        with torch.no_grad():
            for ar, o in zip(arenas, offs):
                esize = torch.empty((), dtype=ar.dtype).element_size()
                ar.grad = seg[o:o + ar.numel * esize].view(ar.dtype)
                ar.param = torch.zeros(ar.numel, dtype=ar.dtype, device=dev)
                for u, uo in ar.units:
                    if len(u.params) > 1:
                        # copy the whole shared storage range so that gaps keep their contents
                        p0 = u.params[0]
                        lo = p0.storage_offset() - u.offsets[0]
                        src = torch.empty(0, dtype=ar.dtype, device=dev).set_(p0.untyped_storage(), lo, (u.numel,))
                        ar.param[uo:uo + u.numel].copy_(src)
                    for p, po in zip(u.params, u.offsets):
                        view = ar.param[uo + po:uo + po + p.numel()].view(p.shape)
                        if len(u.params) == 1:
                            view.copy_(p.data)
                        p.data = view
                        p.grad = ar.grad[uo + po:uo + po + p.numel()].view(p.shape)
                if self._kind and ar.dtype in (torch.bfloat16, torch.float16) and self._master_weights:
                    ar.master = ar.param.float()
            for b in buckets:
                b.grad = b.arena.grad[b.lo:b.hi]
                b.param = b.arena.param[b.lo:b.hi]
                b.master = b.arena.master[b.lo:b.hi] if b.arena.master is not None else None
                b.ready_event = torch.cuda.Event()
                b.done_event = torch.cuda.Event()
        self._arenas = arenas
        self._buckets = buckets
        self._bucket_of, self._slot_off, self._slot_ptr = {}, {}, {}
        for b in buckets:
            for p, off in b.slots:
                self._bucket_of[p] = b
                self._slot_off[p] = off
                self._slot_ptr[p] = b.grad.data_ptr() + off * b.grad.element_size()
        if self._kind:
            self._alias_state()

    def _alias_state(self):
        """Flat optimizer state per arena, exposed per parameter in `optimizer.state` under the
        keys torch uses, so `state_dict()` / `load_state_dict()` keep working."""
        for ar in self._arenas:
            g = self.param_groups[ar.group_index]
            dev = ar.grad.device
            need1 = self._kind == 2 or g.get("momentum", 0) != 0
            if need1 and ar.state1 is None:
                ar.state1 = torch.zeros(ar.numel, dtype=torch.float32, device=dev)
            if self._kind == 2 and ar.state2 is None:
                ar.state2 = torch.zeros(ar.numel, dtype=torch.float32, device=dev)
        for b in self._buckets:
            ar = b.arena
            g = self.param_groups[b.group_index]
            need1 = ar.state1 is not None
            b.state1 = ar.state1[b.lo:b.hi] if ar.state1 is not None else None
            b.state2 = ar.state2[b.lo:b.hi] if ar.state2 is not None else None
            for p, off in b.slots:
                st = self.state[p]
                sl = slice(off, off + p.numel())
                if self._kind == 1 and need1:
                    old = st.get("momentum_buffer")
                    if old is not None:
                        if old.data_ptr() != b.state1[sl].data_ptr():
                            b.state1[sl].copy_(old.reshape(-1).float())
                        st["momentum_buffer"] = b.state1[sl].view(p.shape)
                        # a momentum buffer that already exists must be continued, not re-seeded
                        self._momentum_live[b.group_index] = True
                elif self._kind == 2:
                    for key, flat in (("exp_avg", b.state1), ("exp_avg_sq", b.state2)):
                        old = st.get(key)
                        if old is not None and old.data_ptr() != flat[sl].data_ptr():
                            flat[sl].copy_(old.reshape(-1).float())
                        st[key] = flat[sl].view(p.shape)
                    if "step" not in st:
                        st["step"] = torch.tensor(0.0, dtype=torch.float32)
        for gi, g in enumerate(self.param_groups):
            steps = [float(self.state[p]["step"]) for p in g["params"] if p in self.state and "step" in self.state[p]]
            if steps:
                self._step_count[gi] = int(max(steps))

    def _verify_layout(self):
        sig = [(b.group_index, str(b.dtype), b.lo, b.hi, len(b.params)) for b in self._buckets] + [self._kind]
        DistributedOptimizer._instances += 1
        allsig = core.host_allgather(sig, name=f"{self.name}.layout.{DistributedOptimizer._instances}")
        if any(s != allsig[0] for s in allsig):
            raise core.CollectiveError("DistributedOptimizer: ranks built different bucket layouts (models or options differ)")

    # ---- backward-time path ------------------------------------------------------------------

    @contextlib.contextmanager
    def no_sync(self):
        """Accumulate gradients locally inside this context; nothing is reduced until a backward
        pass outside it."""
        old, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = old

    def _on_grad_ready(self, p):
        if not self._sync:
            return
        b = self._bucket_of.get(p)
        if b is None:
            return
        if p.grad is not None and p.grad.data_ptr() != self._slot_ptr[p]:
            # autograd replaced the view (e.g. after zero_grad(set_to_none=True)): fold it back
            self._restore_grad_view(b, p)
        if not self._kind and not self._backward_end_queued:
            # Unfused: another backward pass may follow before step() and accumulate into buckets
            # that are still being reduced on the private stream. At the end of this pass the
            # compute stream is made to wait for the reductions launched so far.
            self._backward_end_queued = True
            torch.autograd.Variable._execution_engine.queue_callback(self._on_backward_end)
        if b.launched:
            # A second backward pass before step(): this bucket has already been reduced.
            if self._kind:
                raise RuntimeError(
                    "backward() ran again before step(): the fused update of these gradients was already applied while "
                    "the previous backward pass ran. Wrap every backward pass but the last one of an iteration in "
                    "DistributedOptimizer.no_sync(), or build the optimizer with fused=False.")
            # Unfused: the bucket now holds (average so far) + (new local gradients). Averaging it
            # once more at step() gives average(old) + average(new), because the old part is the
            # same on every rank.
            b.dirty = True
            return
        b.pending -= 1
        if b.pending == 0:
            self._launch_in_order()

    def _on_backward_end(self):
        self._backward_end_queued = False
        cur = torch.cuda.current_stream()
        for b in self._buckets:
            if b.launched:
                cur.wait_event(b.done_event)

    def _restore_grad_view(self, b, p):
        off = self._slot_off[p]
        view = b.grad[off:off + p.numel()].view(p.shape)
        with torch.no_grad():
            view.copy_(p.grad)
        p.grad = view

    def _launch_in_order(self):
        # Launched from an autograd hook, so backward is still running beside this launch, except
        # for the last bucket: once it is complete there is nothing left of backward to overlap.
        while self._next_bucket < len(self._buckets) and self._buckets[self._next_bucket].pending <= 0:
            self._launch(self._buckets[self._next_bucket], beside_compute=self._next_bucket + 1 < len(self._buckets))
            self._next_bucket += 1

    def _hyper(self, b) -> _lib.OptHyper:
        g = self.param_groups[b.group_index]
        h = _lib.OptHyper()
        h.kind = self._kind
        h.lr = float(g["lr"])
        h.weight_decay = float(g.get("weight_decay", 0.0))
        h.zero_grad = int(self._fused_zero_grad)
        t = self._step_count[b.group_index] + 1
        if self._kind == 1:
            h.momentum = float(g.get("momentum", 0.0))
            h.dampening = float(g.get("dampening", 0.0))
            h.nesterov = int(bool(g.get("nesterov", False)))
            # torch seeds a momentum buffer that does not exist yet with the gradient itself; with
            # dampening that differs from the recurrence, so the kernel must know. A buffer that
            # was restored from a state dict (or came with the wrapped optimizer) is continued.
            h.first_step = int(not self._momentum_live[b.group_index] and h.dampening != 0.0)
        else:
            b1, b2 = g["betas"]
            h.beta1, h.beta2, h.eps = float(b1), float(b2), float(g["eps"])
            h.bias_c1 = 1.0 - b1 ** t
            h.bias_c2 = 1.0 - b2 ** t
            is_adamw = isinstance(self._optimizer, torch.optim.AdamW) or bool(g.get("decoupled_weight_decay", False))
            h.decoupled_wd = int(is_adamw)
            h.tf_epsilon_hat = int(self._tf_adam)
        return h

    def _launch(self, b: _Bucket, beside_compute: bool = False):
        lib = _lib.lib()
        if self._timing_every and not self._timing_on and (self._iteration % self._timing_every) == 0:
            # the first launch of a sampled step switches the device timing on; step() switches it off
            core.set_device_timing(True)
            self._timing_on = True
        b.ready_event.record(torch.cuda.current_stream())
        wait_ev = C.c_void_p(b.ready_event.cuda_event)
        # make sure the done event has a native handle before it is handed to the library
        if not getattr(b, "_done_primed", False):
            b.done_event.record(torch.cuda.current_stream())
            b._done_primed = True
        rec_ev = C.c_void_p(b.done_event.cuda_event)
        dt = core._DTYPES[b.dtype]
        if self._kind:
            h = self._hyper(b)
            rc = lib.bc_fused_step(_FUSED_CHANNEL, C.c_void_p(b.grad.data_ptr()), b.numel, dt, C.c_void_p(b.param.data_ptr()),
                                   C.c_void_p(b.master.data_ptr()) if b.master is not None else None,
                                   C.c_void_p(b.state1.data_ptr()) if b.state1 is not None else None,
                                   C.c_void_p(b.state2.data_ptr()) if b.state2 is not None else None,
                                   C.byref(h), 1.0 / self._world, wait_ev, rec_ev, int(beside_compute))
        else:
            rc = lib.bc_allreduce_direct(_FUSED_CHANNEL, C.c_void_p(b.grad.data_ptr()), C.c_void_p(b.grad.data_ptr()), b.numel, dt,
                                         1, wait_ev, rec_ev)
        core._call(rc, "bucket launch")
        b.launched = True
        self._launched_any = True
        self.launch_count += 1

    # ---- optimizer interface -----------------------------------------------------------------

    @torch.no_grad()
    def _finish_reduction(self):
        """Launch the buckets that have not gone yet and make the current stream wait for all."""
        # Buckets whose parameters received no gradient in this pass are reduced now (zeros).
        for b in self._buckets[self._next_bucket:]:
            self._launch(b)
        self._next_bucket = len(self._buckets)
        cur = torch.cuda.current_stream()
        for b in self._buckets:
            if b.dirty:                      # unfused only: gradients arrived after the reduction
                cur.wait_event(b.done_event)
                self._launch(b)
                b.dirty = False
        for b in self._buckets:
            if b.launched:
                cur.wait_event(b.done_event)

    @torch.no_grad()
    def synchronize(self):
        """Finish the gradient averaging of this iteration WITHOUT applying the update: afterwards
        every `p.grad` holds the average over all ranks, so gradients can be inspected or clipped
        before `step()`. Needs the unfused path (`fused=False`): a fused update consumes the
        gradients inside the reduction kernel."""
        if self._kind:
            raise RuntimeError("synchronize() needs DistributedOptimizer(..., fused=False): with a fused update the "
                               "gradients are consumed inside the reduction kernel")
        if self._synced:
            return
        if self._gpu:
            self._finish_reduction()
        else:
            self._reduce_cpu()
        self._synced = True

    @torch.no_grad()
    def step(self, closure=None):
        """Finish the gradient averaging of this iteration and apply the update."""
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if not self._gpu:
            if not self._synced:
                self._reduce_cpu()
            self._synced = False
            self._optimizer.step()
            return loss
        if not self._synced:
            self._finish_reduction()
        self._synced = False
        if self._kind:
            for gi, g in enumerate(self.param_groups):
                self._step_count[gi] += 1
                self._momentum_live[gi] = True
                if self._kind == 2:
                    for p in g["params"]:
                        st = self.state.get(p)
                        if st is not None and "step" in st:
                            st["step"] = torch.tensor(float(self._step_count[gi]), dtype=torch.float32)
        else:
            self._optimizer.step()
        for b in self._buckets:
            b.pending = len(b.params)
            b.launched = False
            b.dirty = False
        self._next_bucket = 0
        self._iteration += 1
        if self._timing_on:
            core.set_device_timing(False)
            self._timing_on = False
        return loss

    # ---- groups in two levels: flat buckets launched from hooks ------------------------------------

    def _build_flat_buckets(self, params, limit: int):
        """Parameters in reverse order (the order in which backward produces gradients), grouped by
        dtype and device and cut into buckets of at most `limit` bytes."""
        groups = {}
        for p in reversed(params):
            groups.setdefault((p.dtype, p.device), []).append(p)
        self._flat_of = {}
        for ps in groups.values():
            for chunk in _chunks_by_bytes(ps, limit):
                b = _FlatBucket(len(self._flat), chunk)
                self._flat.append(b)
                for q, off in zip(chunk, b.offsets):
                    self._flat_of[q] = (b, off)

    def _on_flat_grad_ready(self, p):
        if not self._sync or p.grad is None or p.grad.is_sparse:
            return
        b, off = self._flat_of[p]
        if b.handle is not None:
            b.dirty = True                            # a second backward before step(): reduced again at step()
            return
        with torch.no_grad():
            b.buf[off:off + p.numel()].copy_(p.grad.reshape(-1))
        b.filled.add(p)
        if len(b.filled) == len(b.params):
            self._launch_flat(b)

    def _launch_flat(self, b):
        b.handle = core.allreduce_async(b.buf, average=True, name=f"{self.name}.flat.{b.index}", out=b.buf)

    @torch.no_grad()
    def _finish_flat(self):
        """Launch what the hooks have not launched (missing gradients count as zeros, so that every
        rank issues the same collectives), wait, and hand the averages back to the parameters."""
        for b in self._flat:
            if b.handle is not None and b.dirty:
                b.handle.wait()                       # that average is out of date: the gradients have grown since
                b.handle = None
            if b.handle is None:
                for q, off in zip(b.params, b.offsets):
                    sl = b.buf[off:off + q.numel()]
                    if q.grad is None or q.grad.is_sparse:
                        sl.zero_()
                    else:
                        sl.copy_(q.grad.reshape(-1))          # also picks up gradients accumulated under no_sync()
                self._launch_flat(b)
        idx = 0
        for g in self.param_groups:                            # sparse gradients: gathered one by one
            for q in g["params"]:
                if q.grad is not None and q.grad.is_sparse:
                    q.grad = core.allreduce(q.grad, average=True, name=f"{self.name}.grad.{idx}")
                idx += 1
        for b in self._flat:
            b.handle.wait()
            for q, off in zip(b.params, b.offsets):
                if q.grad is not None and not q.grad.is_sparse:
                    q.grad.copy_(b.buf[off:off + q.numel()].view_as(q.grad))
            b.handle = None
            b.dirty = False
            b.filled.clear()

    # ---- the reference's spelling of a training step --------------------------------------------

    def compute_gradients(self, loss: torch.Tensor):
        """Back-propagate `loss` and average the gradients over all ranks; returns
        `[(gradient, parameter), ...]` like the reference's `compute_gradients`
        (`mpi_collectives/__init__.py:195-205`). The gradients can be changed in place before
        `apply_gradients()`. Needs the unfused path (`fused=False`) on a CUDA group."""
        self.zero_grad()
        loss.backward()
        self.synchronize()
        return [(p.grad, p) for g in self.param_groups for p in g["params"] if p.grad is not None]

    def apply_gradients(self, grads_and_vars=None):
        """Apply the update with the gradients held by the parameters (`grads_and_vars`, if given,
        must be the pairs returned by `compute_gradients`: they alias `p.grad`)."""
        if grads_and_vars is not None:
            for g, p in grads_and_vars:
                if p.grad is not g:
                    raise ValueError("apply_gradients() takes the pairs returned by compute_gradients()")
        return self.step()

    def minimize(self, loss: torch.Tensor):
        """One training step from a loss: clear the gradients, back-propagate (the averaging
        overlaps the backward pass on a CUDA group) and update. `tf.train.Optimizer.minimize` of the
        wrapped optimizer in the reference (`mpi_collectives/__init__.py:167-236`)."""
        self.zero_grad()
        loss.backward()
        self.step()
        return loss.detach()

    def _reduce_cpu(self):
        """Average every gradient with the negotiated allreduce: one collective per tensor (as the
        reference does, `mpi_collectives/__init__.py:199-220`), or the flat buckets of a group in
        two levels."""
        if self._flat:
            return self._finish_flat()
        handles = []
        idx = 0
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is not None:
                    if p.grad.is_sparse:
                        p.grad = core.allreduce(p.grad, average=True, name=f"{self.name}.grad.{idx}")
                    else:
                        handles.append(core.allreduce_async(p.grad, average=True, name=f"{self.name}.grad.{idx}", out=p.grad))
                idx += 1
        for h in handles:
            h.wait()

    def zero_grad(self, set_to_none: bool = True):
        """Reset gradients. On a CUDA group the flat buckets stay in place (they are zeroed, never
        freed); with the fused update and `fused_zero_grad` the kernel has already done it."""
        if not self._gpu:
            return self._optimizer.zero_grad(set_to_none=set_to_none)
        if self._kind and self._fused_zero_grad:
            return
        self._grad_segment.zero_()

    def state_dict(self):
        if self._gpu and self._kind:
            # materialise momentum buffers that torch would have created lazily
            for b in self._buckets:
                g = self.param_groups[b.group_index]
                if self._kind == 1 and g.get("momentum", 0) != 0 and self._momentum_live[b.group_index]:
                    for p, off in b.slots:
                        self.state[p]["momentum_buffer"] = b.state1[off:off + p.numel()].view(p.shape)
        return self._optimizer.state_dict()

    def load_state_dict(self, state_dict):
        self._optimizer.load_state_dict(state_dict)
        self.state = self._optimizer.state
        self.param_groups = self._optimizer.param_groups
        if self._gpu and self._kind:
            self._alias_state()
            if self._master_weights:
                for b in self._buckets:
                    if b.master is not None:
                        b.master.copy_(b.param.float())

    def sync_master_weights(self):
        """Re-read the fp32 master copies from the 16-bit parameters (after loading weights)."""
        for b in self._buckets:
            if b.master is not None:
                b.master.copy_(b.param.float())

    def add_param_group(self, param_group):
        if getattr(self, "_buckets", None):
            raise NotImplementedError("parameters cannot be added after the gradient buckets were built")
        return super().add_param_group(param_group)

    @property
    def fused(self) -> bool:
        return bool(self._kind)

    @property
    def buckets(self):
        """(dtype, elements) of every gradient bucket, in launch order."""
        return [(b.dtype, b.numel) for b in self._buckets]

    @property
    def bucket_parameters(self):
        """The parameters of every gradient bucket, in launch order."""
        return [list(b.params) for b in self._buckets]

    def __repr__(self):
        return f"{self.name}(fused={self.fused}, buckets={len(self._buckets)}, wrapped={self._optimizer!r})"
