"""`DistributedOptimizer`: wraps a `torch.optim.Optimizer` and averages every gradient over all
ranks before the update is applied.

Reference: `tensorflow/contrib/mpi_collectives/__init__.py:167-234` (a `tf.train.Optimizer` whose
`compute_gradients` allreduces each gradient and which forwards everything else to the wrapped
optimizer; one collective per tensor, no bucketing, averaging and the update as separate kernels).

What is different here, on a CUDA group:
  * gradients of all parameters live in flat buckets inside symmetric memory (`p.grad` is a view
    of its bucket), so a bucket is reduced where it is, with no gather copy and no staging;
  * a bucket is launched from an autograd hook as soon as its last gradient has been accumulated,
    on the library's private stream, behind an event recorded on the compute stream: the
    reduction overlaps the rest of the backward pass. Buckets are launched strictly in bucket
    order, which is identical on all ranks, so this path needs no negotiation per step;
  * for `torch.optim.SGD`, `Adam` and `AdamW` the averaging, the optimizer update, the 16-bit ->
    fp32 master-weight handling and the zeroing of the gradient are fused into the reduction
    kernel (`bc_fused_step`); other optimizers get averaged gradients in `p.grad` and then run
    their own `step()`.
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


class _Bucket:
    def __init__(self, index, group_index, dtype):
        self.index = index
        self.group_index = group_index
        self.dtype = dtype
        self.units: List[_Unit] = []
        self.unit_offsets: List[int] = []
        self.numel = 0
        self.params: List[torch.nn.Parameter] = []
        self.pending = 0
        self.launched = False
        self.grad = None      # flat views, set after allocation
        self.param = None
        self.master = None
        self.state1 = None
        self.state2 = None
        self.ready_event = None
        self.done_event = None


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

    Construction is collective on a CUDA group (symmetric memory is allocated): every rank must
    build its optimizers in the same order over identically shaped models.
    """

    _instances = 0

    def __init__(self, optimizer: torch.optim.Optimizer, name: Optional[str] = None, use_locking: bool = False, *,
                 fused: Optional[bool] = None, bucket_mb: Optional[float] = None, master_weights: bool = True,
                 fused_zero_grad: bool = True, tf_adam: bool = False):
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
        buckets: List[_Bucket] = []
        for gi, g in enumerate(self.param_groups):
            ps = [p for p in g["params"] if p.requires_grad]
            for dtype in sorted({p.dtype for p in ps}, key=str):
                units = self._make_units([p for p in ps if p.dtype == dtype])
                esize = torch.empty((), dtype=dtype).element_size()
                align = _ALIGN_BYTES // esize
                cur = None
                # Gradients become ready roughly in reverse parameter order.
                for u in reversed(units):
                    if cur is None or (cur.numel > 0 and (cur.numel + u.numel) * esize > self._bucket_bytes):
                        cur = _Bucket(len(buckets), gi, dtype)
                        buckets.append(cur)
                    off = (cur.numel + align - 1) // align * align
                    cur.units.append(u)
                    cur.unit_offsets.append(off)
                    cur.numel = off + u.numel
                    cur.params.extend(u.params)
        # One symmetric segment for all gradient buckets; parameters and state in ordinary memory.
        offs, total = [], 0
        for b in buckets:
            esize = torch.empty((), dtype=b.dtype).element_size()
            total = (total + _ALIGN_BYTES - 1) // _ALIGN_BYTES * _ALIGN_BYTES
            offs.append(total)
            total += b.numel * esize
        seg, self._has_multicast = symmetric.new_segment(max(total, _ALIGN_BYTES), dev)
        self._grad_segment = seg
        with torch.no_grad():
            for b, o in zip(buckets, offs):
                esize = torch.empty((), dtype=b.dtype).element_size()
                b.grad = seg[o:o + b.numel * esize].view(b.dtype)
                b.param = torch.zeros(b.numel, dtype=b.dtype, device=dev)
                for u, uo in zip(b.units, b.unit_offsets):
                    if len(u.params) > 1:
                        # copy the whole shared storage range so that gaps keep their contents
                        p0 = u.params[0]
                        lo = p0.storage_offset() - u.offsets[0]
                        src = torch.empty(0, dtype=b.dtype, device=dev).set_(p0.untyped_storage(), lo, (u.numel,))
                        b.param[uo:uo + u.numel].copy_(src)
                    for p, po in zip(u.params, u.offsets):
                        view = b.param[uo + po:uo + po + p.numel()].view(p.shape)
                        if len(u.params) == 1:
                            view.copy_(p.data)
                        p.data = view
                        p.grad = b.grad[uo + po:uo + po + p.numel()].view(p.shape)
                b.pending = len(b.params)
                b.ready_event = torch.cuda.Event()
                b.done_event = torch.cuda.Event()
                if self._kind and b.dtype in (torch.bfloat16, torch.float16) and self._master_weights:
                    b.master = b.param.float()
        self._buckets = buckets
        self._bucket_of, self._slot_off, self._slot_ptr = {}, {}, {}
        for b in buckets:
            for u, uo in zip(b.units, b.unit_offsets):
                for p, po in zip(u.params, u.offsets):
                    self._bucket_of[p] = b
                    self._slot_off[p] = uo + po
                    self._slot_ptr[p] = b.grad.data_ptr() + (uo + po) * b.grad.element_size()
        if self._kind:
            self._alias_state()

    def _alias_state(self):
        """Flat optimizer state per bucket, exposed per parameter in `optimizer.state` under the
        keys torch uses, so `state_dict()` / `load_state_dict()` keep working."""
        for b in self._buckets:
            g = self.param_groups[b.group_index]
            dev = b.grad.device
            need1 = self._kind == 2 or g.get("momentum", 0) != 0
            if need1 and b.state1 is None:
                b.state1 = torch.zeros(b.numel, dtype=torch.float32, device=dev)
            if self._kind == 2 and b.state2 is None:
                b.state2 = torch.zeros(b.numel, dtype=torch.float32, device=dev)
            for u, uo in zip(b.units, b.unit_offsets):
                for p, po in zip(u.params, u.offsets):
                    st = self.state[p]
                    sl = slice(uo + po, uo + po + p.numel())
                    if self._kind == 1 and need1:
                        old = st.get("momentum_buffer")
                        if old is not None:
                            b.state1[sl].copy_(old.reshape(-1).float())
                            st["momentum_buffer"] = b.state1[sl].view(p.shape)
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
        sig = [(b.group_index, str(b.dtype), b.numel, len(b.params)) for b in self._buckets] + [self._kind]
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
        b.pending -= 1
        if b.pending == 0:
            self._launch_in_order()

    def _restore_grad_view(self, b, p):
        off = self._slot_off[p]
        view = b.grad[off:off + p.numel()].view(p.shape)
        with torch.no_grad():
            view.copy_(p.grad)
        p.grad = view

    def _launch_in_order(self):
        while self._next_bucket < len(self._buckets) and self._buckets[self._next_bucket].pending <= 0:
            self._launch(self._buckets[self._next_bucket])
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
            h.first_step = int(t == 1 and h.dampening != 0.0)
        else:
            b1, b2 = g["betas"]
            h.beta1, h.beta2, h.eps = float(b1), float(b2), float(g["eps"])
            h.bias_c1 = 1.0 - b1 ** t
            h.bias_c2 = 1.0 - b2 ** t
            is_adamw = isinstance(self._optimizer, torch.optim.AdamW) or bool(g.get("decoupled_weight_decay", False))
            h.decoupled_wd = int(is_adamw)
            h.tf_epsilon_hat = int(self._tf_adam)
        return h

    def _launch(self, b: _Bucket):
        lib = _lib.lib()
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
                                   C.byref(h), 1.0 / self._world, wait_ev, rec_ev)
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
        self._next_bucket = 0
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
                if self._kind == 1 and g.get("momentum", 0) != 0 and self._step_count[b.group_index] > 0:
                    for u, uo in zip(b.units, b.unit_offsets):
                        for p, po in zip(u.params, u.offsets):
                            self.state[p]["momentum_buffer"] = b.state1[uo + po:uo + po + p.numel()].view(p.shape)
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

    def __repr__(self):
        return f"{self.name}(fused={self.fused}, buckets={len(self._buckets)}, wrapped={self._optimizer!r})"
