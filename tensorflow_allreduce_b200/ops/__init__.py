"""Kernel-level operations: symmetric memory, fused reduce+update launches, single-GPU emulation."""
from . import emulated, fused_optim, symmetric  # noqa: F401
