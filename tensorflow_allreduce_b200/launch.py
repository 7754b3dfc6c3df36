"""`python -m tensorflow_allreduce_b200.launch --nproc N script.py [args...]`

Starts N ranks of `script.py` on this host, one per GPU when CUDA devices are visible, with
RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT set: what `mpirun -np N` does for the
reference. `torchrun` works as well; the library reads the same variables.
"""
from __future__ import annotations

import argparse
import signal
import subprocess
import sys

from .utils.spawn import free_port, rank_env


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tensorflow_allreduce_b200.launch")
    ap.add_argument("--nproc", "-n", type=int, default=1, help="number of ranks to start on this host")
    ap.add_argument("--port", type=int, default=0, help="rendezvous port (default: a free one)")
    ap.add_argument("--cpu", action="store_true", help="hide GPUs from the ranks")
    ap.add_argument("script")
    ap.add_argument("args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    port = a.port or free_port()
    procs = []
    for r in range(a.nproc):
        env = rank_env(r, a.nproc, port, gpus=not a.cpu)
        procs.append(subprocess.Popen([sys.executable, a.script, *a.args], env=env))

    def forward(sig, _frame):
        for p in procs:
            if p.poll() is None:
                p.send_signal(sig)

    signal.signal(signal.SIGINT, forward)
    signal.signal(signal.SIGTERM, forward)
    rc = 0
    for p in procs:
        code = p.wait()
        if code != 0 and rc == 0:
            rc = code
            # one rank failed: the others would only run into their deadlines
            for q in procs:
                if q.poll() is None:
                    q.terminate()
    return rc


if __name__ == "__main__":
    sys.exit(main())
