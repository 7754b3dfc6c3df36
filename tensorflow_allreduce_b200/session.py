"""`Session`: joins the process group when it is created and leaves it when it is closed.

The reference's `mpi.Session` is a `tf.Session` whose only addition is to run the init op on
construction (`tensorflow/contrib/mpi_collectives/__init__.py:237-273`). PyTorch has no session
object, so this is a plain context manager with a `run` convenience.
"""
from __future__ import annotations

from typing import Optional

from . import core
from .config import Config


class Session:
    """`with Session(): ...` = `init()` on entry, `shutdown()` on exit.

    `target` and `graph` exist for signature compatibility with the reference and are ignored.
    """

    def __init__(self, target: str = "", graph=None, config: Optional[Config] = None, device=None):
        self._owns = not core.is_initialized()
        if self._owns:
            core.init(device=device, config=config)
        self._closed = False

    def run(self, fn, *args, **kwargs):
        """Call `fn(*args, **kwargs)` inside the session and return its value. A tensor (or a
        list/tuple/dict of tensors) is returned as is: eager tensors need no fetch step."""
        if self._closed:
            raise core.CollectiveError("Session is closed")
        if callable(fn):
            return fn(*args, **kwargs)
        return fn

    def close(self) -> None:
        if not self._closed and self._owns:
            core.shutdown()
        self._closed = True

    def __enter__(self) -> "Session":
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        self.close()
