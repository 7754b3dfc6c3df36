"""Start N local ranks as child processes: the job of `mpirun -np N` for the reference's tests
(`tensorflow/contrib/mpi_collectives/mpi_ops_test.py:30-62` reads the launcher's environment).
Used by the launcher module and by the test-suite."""
from __future__ import annotations

import os
import signal
import socket
import subprocess
import sys
import tempfile
import time
from typing import Dict, List, Optional, Sequence


def free_port() -> int:
    """A port for rank 0's rendezvous listener that nothing is bound to right now.

    Ports below the kernel's ephemeral range are tried first: a port of that range can be handed
    to any other socket (a rank's own data listener, the source port of a connection attempt)
    between this call and rank 0's bind, which then fails while the other ranks wait."""
    import random

    low = 32768
    try:
        with open("/proc/sys/net/ipv4/ip_local_port_range") as f:
            low = int(f.read().split()[0])
    except (OSError, ValueError, IndexError):
        pass
    if low > 21000:
        rng = random.Random(os.getpid() * 1000003 + time.monotonic_ns())
        for _ in range(64):
            port = rng.randrange(20000, low)
            with socket.socket() as s:
                try:
                    s.bind(("0.0.0.0", port))
                except OSError:
                    continue
                return port
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class RankResult:
    def __init__(self, rank: int, returncode: Optional[int], stdout: str, stderr: str):
        self.rank, self.returncode, self.stdout, self.stderr = rank, returncode, stdout, stderr

    def __repr__(self):
        return f"RankResult(rank={self.rank}, rc={self.returncode})"


def rank_env(rank: int, size: int, port: int, extra: Optional[Dict[str, str]] = None, gpus: bool = False) -> Dict[str, str]:
    env = dict(os.environ)
    for k in ("TORCHELASTIC_USE_AGENT_STORE", "TORCHELASTIC_RUN_ID", "OMPI_COMM_WORLD_RANK", "PMI_RANK"):
        env.pop(k, None)
    env.update({
        "RANK": str(rank), "WORLD_SIZE": str(size), "LOCAL_RANK": str(rank), "LOCAL_WORLD_SIZE": str(size),
        "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "BC_PORT": str(port),
    })
    if not gpus:
        env.setdefault("CUDA_VISIBLE_DEVICES", "")
    if extra:
        env.update({k: str(v) for k, v in extra.items()})
    return env


def run_ranks(argv: Sequence[str], nranks: int, timeout: float = 120.0, env: Optional[Dict[str, str]] = None,
              per_rank_env: Optional[Dict[int, Dict[str, str]]] = None, gpus: bool = False, cwd: Optional[str] = None,
              dump_stacks: bool = False) -> List[RankResult]:
    """Run `python <argv...>` as `nranks` processes and wait for all of them. A rank still running
    at the deadline is killed (its own process only) and reported with returncode None; with
    `dump_stacks` it is sent SIGUSR1 first (for scripts that registered `faulthandler` on it)."""
    port = free_port()
    procs = []
    files = []
    for r in range(nranks):
        e = rank_env(r, nranks, port, env, gpus=gpus)
        if per_rank_env and r in per_rank_env:
            e.update({k: str(v) for k, v in per_rank_env[r].items()})
        out = tempfile.TemporaryFile(mode="w+")
        err = tempfile.TemporaryFile(mode="w+")
        files.append((out, err))
        procs.append(subprocess.Popen([sys.executable, *argv], env=e, stdout=out, stderr=err, cwd=cwd))
    deadline = time.time() + timeout
    results = []
    for r, p in enumerate(procs):
        rc: Optional[int]
        try:
            rc = p.wait(timeout=max(0.1, deadline - time.time()))
        except subprocess.TimeoutExpired:
            # A script that registered faulthandler on SIGUSR1 leaves its Python stacks in stderr.
            if dump_stacks:
                try:
                    p.send_signal(signal.SIGUSR1)
                    time.sleep(0.5)
                except OSError:
                    pass
            p.kill()
            p.wait()
            rc = None
        out, err = files[r]
        out.seek(0)
        err.seek(0)
        results.append(RankResult(r, rc, out.read(), err.read()))
        out.close()
        err.close()
    return results


def run_script(body: str, nranks: int, **kw) -> List[RankResult]:
    """Run a Python source string as `nranks` ranks (the script sees RANK / WORLD_SIZE / ...)."""
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write(body)
        path = f.name
    try:
        return run_ranks([path], nranks, **kw)
    finally:
        os.unlink(path)
