"""B200-native data-parallel collectives for PyTorch.

Public API, matching `tensorflow/contrib/mpi_collectives` (`__init__.py:114-131`):

    init / shutdown / size / rank / local_rank
    allreduce(tensor, average=True)      dense or sparse; sum or average over all ranks
    allgather(tensor)                    concatenation along dim 0, per-rank first dimension
    Session                              context manager that joins the group on entry
    DistributedOptimizer(optimizer)      averages gradients across ranks before the update

plus the reductions of the reference's NCCL ops (`contrib/nccl/python/ops/nccl_ops.py`): `all_sum`,
`all_prod`, `all_min`, `all_max` (`allreduce(..., op=...)`), `broadcast`;
plus what the reference lacks: `broadcast_parameters`, in-place and asynchronous
variants, symmetric-memory tensors, statistics and a launcher (`python -m
tensorflow_allreduce_b200.launch`).
"""
from .config import Config
from .core import (CollectiveError, all_max, all_min, all_prod, all_sum, allgather, allgather_async, allreduce, allreduce_, allreduce_async, barrier,
                   broadcast, check_device_status, clear_stats, config, grouped_allreduce, host_allgather, init, is_broken, is_initialized,
                   local_rank, local_size, n_nodes, node_index, on_gpu, rank, set_device_timing, set_fault, shutdown, size, stats)
from .session import Session
from .parallel.distributed_optimizer import DistributedOptimizer
from .parallel.broadcast import broadcast_optimizer_state, broadcast_parameters

__all__ = [
    "Config", "CollectiveError", "Session", "DistributedOptimizer", "init", "shutdown", "is_initialized", "is_broken", "size",
    "rank", "local_rank", "local_size", "allreduce", "allreduce_", "allreduce_async", "all_sum", "all_prod", "all_min",
    "all_max", "grouped_allreduce", "allgather", "allgather_async",
    "broadcast", "broadcast_parameters", "broadcast_optimizer_state", "barrier", "host_allgather", "stats",
    "clear_stats", "on_gpu", "n_nodes", "node_index", "config", "set_fault", "set_device_timing", "check_device_status",
]
__version__ = "0.1.0"
