"""ctypes binding of the native library `lib/libbcoll.so` (interface: `csrc/bcoll.h`).

Plays the role of `_load_library` + the generated op wrappers of the reference
(tensorflow/contrib/mpi_collectives/mpi_ops.py:30-59). The library is built in-tree on first use
if it is missing or older than its sources; a failed build or load raises, it never falls back
to a Python implementation.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_lock = threading.Lock()
_lib = None

ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_longlong, C.c_longlong, C.c_void_p, C.POINTER(C.c_int))


class OptHyper(C.Structure):
    """Mirror of `bc_opt_hyper` (csrc/bcoll.h)."""

    _fields_ = [
        ("kind", C.c_int),
        ("lr", C.c_float),
        ("weight_decay", C.c_float),
        ("momentum", C.c_float),
        ("dampening", C.c_float),
        ("nesterov", C.c_int),
        ("first_step", C.c_int),
        ("beta1", C.c_float),
        ("beta2", C.c_float),
        ("eps", C.c_float),
        ("bias_c1", C.c_float),
        ("bias_c2", C.c_float),
        ("decoupled_wd", C.c_int),
        ("tf_epsilon_hat", C.c_int),
        ("zero_grad", C.c_int),
    ]


class NativeError(RuntimeError):
    """An error reported by the native library."""


def _declare(lib):
    vp, ll, i, d, f, cp = C.c_void_p, C.c_longlong, C.c_int, C.c_double, C.c_float, C.c_char_p
    P = C.POINTER
    sig = {
        "bc_last_error": (cp, []),
        "bc_init": (i, [i, i, i, cp, i, i, d, d, ll, ll, i, ll, ll, i, i, i, cp]),
        "bc_initialized": (i, []),
        "bc_shutdown": (i, []),
        "bc_rank": (i, []),
        "bc_size": (i, []),
        "bc_local_rank": (i, []),
        "bc_local_size": (i, []),
        "bc_on_gpu": (i, []),
        "bc_broken": (i, []),
        "bc_n_nodes": (i, []),
        "bc_node_index": (i, []),
        "bc_two_level_allreduce_host": (i, [vp, ll, i, i, i]),
        "bc_select_algo": (i, [i, ll, i, i, i, i, ll, ll, i]),
        "bc_choose_blocks": (i, [ll, i, i, i, i, i, i]),
        "bc_plan_pipeline": (i, [ll, ll, ll, i, i, ll, P(ll)]),
        "bc_plan_gather_rounds": (ll, [i, P(C.c_ulonglong), ll, P(C.c_ulonglong)]),
        "bc_allreduce_async": (ll, [cp, vp, vp, i, i, P(ll), i, i, i, vp, i]),
        "bc_allgather_async": (ll, [cp, vp, i, i, P(ll), i, ALLOC_FN, vp, vp]),
        "bc_wait": (i, [ll, d]),
        "bc_poll": (i, [ll]),
        "bc_done_event": (vp, [ll]),
        "bc_result_algo": (i, [ll]),
        "bc_result_dim0": (i, [ll, P(ll), i]),
        "bc_release": (i, [ll]),
        "bc_blob_gather": (i, [cp, vp, i, vp, ll, P(i)]),
        "bc_set_fault": (i, [cp]),
        "bc_stats_json": (cp, []),
        "bc_clear_stats": (i, []),
        "bc_device_status": (C.c_uint, []),
        "bc_set_device_timeout": (i, [d]),
        "bc_symm_heap": (vp, [P(ll)]),
        "bc_symm_new_segment": (vp, [ll, P(i), P(i)]),
        "bc_symm_contains": (i, [vp, ll]),
        "bc_symm_describe": (cp, []),
        "bc_comm_stream": (vp, [i]),
        "bc_stream_wait_event": (i, [vp, vp]),
        "bc_allreduce_direct": (i, [i, vp, vp, ll, i, i, vp, vp]),
        "bc_fused_step": (i, [i, vp, ll, i, vp, vp, vp, vp, P(OptHyper), f, vp, vp, i]),
        "bc_set_option": (i, [cp, ll]),
        "bc_set_allreduce_profile": (i, [vp]),
        "bc_allgatherv_direct": (i, [i, vp, ll, vp, ll, vp, vp, vp]),
        "bc_emu_create": (vp, [i, i, ll]),
        "bc_emu_destroy": (i, [vp]),
        "bc_emu_buffer": (vp, [vp, i]),
        "bc_emu_status": (C.c_uint, [vp]),
        "bc_emu_clear_status": (i, [vp]),
        "bc_emu_damaged_guard_bytes": (ll, [vp]),
        "bc_emu_allreduce": (i, [vp, ll, P(vp), ll, i, i, f, i, i, vp, i, P(vp), P(C.c_ulonglong), vp, i]),
        "bc_emu_fused_step": (i, [vp, ll, ll, i, P(vp), P(vp), P(vp), P(vp), P(OptHyper), f, i, vp, i]),
        "bc_emu_staged_pipeline": (i, [vp, ll, P(vp), P(vp), ll, i, f, i, ll, i, i, i, i, i, i, i, vp]),
        "bc_emu_allgatherv": (i, [vp, P(vp), P(C.c_ulonglong), P(C.c_ulonglong), i, vp]),
        "bc_emu_barrier_probe": (i, [vp, i, d, vp]),
        "bc_max_emulated_blocks": (i, [i, i]),
        "bc_gru_supported": (i, [i, i, i, i, i]),
        "bc_gru_set_profile": (i, [vp]),
        "bc_gru_workspace_bytes": (ll, [i, i, i, i]),
        "bc_gru_forward": (i, [i, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp, d, vp]),
        "bc_gru_backward": (i, [i, i, i, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, d, vp]),
        "bc_bn_clip_forward": (i, [vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, f, f, f, vp]),
        "bc_bn_clip_backward": (i, [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, f, vp]),
        "bc_test_validate": (i, [i, P(i), P(i), P(i), P(i), P(ll), cp, i, P(ll)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def lib():
    """The loaded native library (built first if needed)."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        from . import build as _build

        # BC_DEBUG_KERNELS=1 loads the bounds-checked build of the same sources.
        debug = os.environ.get("BC_DEBUG_KERNELS", "0") == "1"
        target = _build.LIB_DEBUG if debug else _build.LIB
        if os.environ.get("BC_NO_BUILD", "0") != "1" and _build.needs_build(debug):
            # Several ranks may start at once: serialise the build through a lock file.
            import fcntl

            _build.LIBDIR.mkdir(parents=True, exist_ok=True)
            with open(_build.LIBDIR / ".build.lock", "w") as lk:
                fcntl.flock(lk, fcntl.LOCK_EX)
                try:
                    if _build.needs_build(debug):
                        _build.build(debug=debug)
                finally:
                    fcntl.flock(lk, fcntl.LOCK_UN)
        if not target.exists():
            raise NativeError(f"native library missing: {target}")
        loaded = C.CDLL(str(target), mode=C.RTLD_GLOBAL)
        _declare(loaded)
        _lib = loaded
    return _lib


def last_error() -> str:
    msg = lib().bc_last_error()
    return msg.decode("utf-8", "replace") if msg else ""


def check(rc, what: str = ""):
    """Raise `NativeError` if a native call reported failure (-1 / NULL)."""
    if rc is None or (isinstance(rc, int) and rc < 0):
        raise NativeError(last_error() or f"native call failed: {what}")
    return rc
