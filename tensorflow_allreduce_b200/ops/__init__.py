"""Kernel-level operations: symmetric memory, ordered launches, fused reduce+update, single-GPU emulation."""
from . import direct, emulated, fused_optim, symmetric  # noqa: F401
