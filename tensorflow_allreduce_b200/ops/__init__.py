"""Kernel-level operations: symmetric memory, fused reduce+update launches, single-GPU emulation."""
from . import symmetric  # noqa: F401
