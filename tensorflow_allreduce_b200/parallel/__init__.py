"""Data parallelism: the gradient-averaging optimizer wrapper and weight/state broadcast helpers."""
from .broadcast import broadcast_optimizer_state, broadcast_parameters  # noqa: F401
from .distributed_optimizer import DistributedOptimizer  # noqa: F401
