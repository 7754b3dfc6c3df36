"""Run-time configuration: one dataclass, overridable through `BC_*` environment variables.

The reference's collective package has no run-time knobs at all; its only configuration is the
build-time MPI switch (`configure:823-897`). Everything here is new: algorithm cut-overs, bucket
size, grid caps, deadlines, symmetric-memory sizes, NVLS on/off and the log level
(`BC_LOG_LEVEL`, read by the native side). Read elsewhere: `BC_STATS_JSONL` (per-collective records
appended at shutdown, `core.py`), `BC_NVTX` (`csrc/nvtx.cc`), `BC_DEBUG_KERNELS` (bounds-checked
build, `_lib.py`), `BC_GRU_TIMEOUT_S` (`ops/persistent_gru.py`), and by the native runtime at
`init()`: `BC_SHM` (0 = CPU tensors of ranks on one host use the socket ring instead of shared
memory), `BC_SHM_SLOT_KB` (chunk per rank in the shared segment, default 512), `BC_NODE_GROUPS`
(1 = build the node groups and rails of a job over several hosts for a CPU group too),
`BC_HOSTNAME` (the host name this rank reports), `BC_TWO_LEVEL_CHUNK_KB` (CPU tensors of a job over
several hosts: chunk of the pipelined two-level allreduce, default 2048, used from four chunks on; 0 = in
one piece), `BC_SPIN_US` (how long the background thread and
a waiting caller keep polling after an event before they sleep; default 100, or 0 = sleep at once
when the host has fewer than two cores per local rank).
"""
from __future__ import annotations

import dataclasses
import os

_ALGOS = {"auto": 0, "one_shot": 1, "two_shot": 2, "nvls": 3}
_SYMM = {"auto": 0, "vmm": 1, "ipc": 2}


def _env(name, cast, default):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return cast(v)


def _flag(v: str) -> bool:
    return str(v).strip().lower() not in ("0", "false", "no", "off", "")


@dataclasses.dataclass
class Config:
    """Settings read at `init()`; every rank must use the same values."""

    timeout_s: float = 300.0           # host-side deadline: bootstrap, negotiation, ring steps
    device_timeout_s: float = 30.0     # bound of every device-side wait on a peer
    staging_mb: int = 1024             # symmetric staging area for tensors outside symmetric memory (a quarter per channel)
    heap_mb: int = 256                 # symmetric heap for allgather outputs and `symm_empty`
    algo: str = "auto"                 # force one of: one_shot, two_shot, nvls
    one_shot_max_kb: int = 256         # messages up to this size use the one-shot kernel
    nvls_min_kb: int = 512             # messages from this size use NVLS when multicast is bound
    nvls: bool = True                  # bind a multicast object to symmetric segments when possible
    max_blocks: int = 0                # cap on CTAs per collective kernel (0 = heuristic)
    symm: str = "auto"                 # symmetric memory back end: vmm (fd passing) or ipc
    bucket_mb: float = 32.0            # DistributedOptimizer gradient bucket size
    overlap_blocks: int = 0            # CTAs of a bucket launch that runs beside backward (0 = one per SM left free
                                       # by a 128-SM persistent kernel, at least 8)
    staged_pipeline: int = 1           # large tensors outside symmetric memory in one launch whose blocks copy chunks
                                       # in and out while others reduce: 0 = off, 1 = where the switch reduces
                                       # (NVLS), 2 = with peer loads and stores as well
    pipeline_min_mb: int = 96          # ... from this size on
    pipeline_chunk_kb: int = 8192      # largest chunk of that kernel
    pipeline_slots: int = 16           # chunks that its ring inside the staging slice holds
    pipeline_copiers: int = 0          # its blocks that copy (0 = what half of the SMs leaves beside the reducers)
    pipeline_reducers: int = 0         # its blocks that reduce (0 = 16 where the switch reduces, else 32; draining: 32 / 48)
    pipeline_streaming: bool = True    # its reducer blocks never drain between chunks (one warp waits and publishes)
    pipeline_rgroups: int = 8          # draining reducers: groups of blocks; group g takes the chunks c with c % groups == g
    pipeline_cgroups: int = 4          # groups of copier blocks
    device_timing_every: int = 0       # DistributedOptimizer: time every bucket launch of every Nth step on the device
                                       # (CUDA events; records in stats() carry device_us and bus GB/s); 0 = never
    link_gbs: float = 764.0            # NVLink rate per direction per GPU that stats() reports fractions of
                                       # (measured peer copy on B200 / NVSwitch; nominal 900)
    fault: str = ""                    # host-side fault injection, e.g. "drop_request:rank=1:name=x"

    @classmethod
    def from_env(cls, **overrides) -> "Config":
        c = cls(
            timeout_s=_env("BC_TIMEOUT_S", float, cls.timeout_s),
            device_timeout_s=_env("BC_DEVICE_TIMEOUT_S", float, cls.device_timeout_s),
            staging_mb=_env("BC_STAGING_MB", int, cls.staging_mb),
            heap_mb=_env("BC_HEAP_MB", int, cls.heap_mb),
            algo=_env("BC_ALGO", str, cls.algo),
            one_shot_max_kb=_env("BC_ONE_SHOT_MAX_KB", int, cls.one_shot_max_kb),
            nvls_min_kb=_env("BC_NVLS_MIN_KB", int, cls.nvls_min_kb),
            nvls=_env("BC_NVLS", _flag, cls.nvls),
            max_blocks=_env("BC_MAX_BLOCKS", int, cls.max_blocks),
            symm=_env("BC_SYMM", str, cls.symm),
            bucket_mb=_env("BC_BUCKET_MB", float, cls.bucket_mb),
            overlap_blocks=_env("BC_OVERLAP_BLOCKS", int, cls.overlap_blocks),
            staged_pipeline=_env("BC_STAGED_PIPELINE", int, cls.staged_pipeline),
            pipeline_min_mb=_env("BC_PIPELINE_MIN_MB", int, cls.pipeline_min_mb),
            pipeline_chunk_kb=_env("BC_PIPELINE_CHUNK_KB", int, cls.pipeline_chunk_kb),
            pipeline_slots=_env("BC_PIPELINE_SLOTS", int, cls.pipeline_slots),
            pipeline_copiers=_env("BC_PIPELINE_COPIERS", int, cls.pipeline_copiers),
            pipeline_reducers=_env("BC_PIPELINE_REDUCERS", int, cls.pipeline_reducers),
            pipeline_streaming=_env("BC_PIPELINE_STREAMING", _flag, cls.pipeline_streaming),
            pipeline_rgroups=_env("BC_PIPELINE_RGROUPS", int, cls.pipeline_rgroups),
            pipeline_cgroups=_env("BC_PIPELINE_CGROUPS", int, cls.pipeline_cgroups),
            device_timing_every=_env("BC_DEVICE_TIMING_EVERY", int, cls.device_timing_every),
            link_gbs=_env("BC_LINK_GBS", float, cls.link_gbs),
            fault=_env("BC_FAULT", str, cls.fault),
        )
        for k, v in overrides.items():
            if v is not None:
                setattr(c, k, v)
        c.validate()
        return c

    def validate(self) -> None:
        if self.algo not in _ALGOS:
            raise ValueError(f"BC_ALGO must be one of {sorted(_ALGOS)}, got {self.algo!r}")
        if self.symm not in _SYMM:
            raise ValueError(f"BC_SYMM must be one of {sorted(_SYMM)}, got {self.symm!r}")
        if self.timeout_s <= 0 or self.device_timeout_s <= 0:
            raise ValueError("timeouts must be positive")

    @property
    def algo_code(self) -> int:
        return _ALGOS[self.algo]

    @property
    def symm_code(self) -> int:
        return _SYMM[self.symm]
