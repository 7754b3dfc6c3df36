"""`python -m tensorflow_allreduce_b200.launch --nproc N script.py [args...]`

Starts N ranks of `script.py` on this host, one per GPU when CUDA devices are visible, with
RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT set: what `mpirun -np N` does for the
reference. `torchrun` works as well; the library reads the same variables.

A job over several hosts (`mpirun -H a,b` for the reference) is one launcher per host:

    host a:  python -m tensorflow_allreduce_b200.launch --nnodes 2 --node-rank 0 --master-addr a --port 29400 --nproc 8 script.py
    host b:  python -m tensorflow_allreduce_b200.launch --nnodes 2 --node-rank 1 --master-addr a --port 29400 --nproc 8 script.py

Rank = node-rank x nproc + local rank; rank 0 (on node 0) listens on master-addr:port.
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
    ap.add_argument("--nnodes", type=int, default=1, help="hosts of the job (one launcher runs on each)")
    ap.add_argument("--node-rank", type=int, default=0, help="index of this host, 0 .. nnodes-1")
    ap.add_argument("--master-addr", default="127.0.0.1", help="address of the host with node-rank 0")
    ap.add_argument("script")
    ap.add_argument("args", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    if a.nnodes > 1 and not a.port:
        ap.error("--port is required with --nnodes > 1 (every host must name the same one)")
    if not 0 <= a.node_rank < a.nnodes:
        ap.error("--node-rank must lie in 0 .. nnodes-1")
    port = a.port or free_port()
    procs = []
    for r in range(a.nproc):
        env = rank_env(a.node_rank * a.nproc + r, a.nnodes * a.nproc, port, gpus=not a.cpu)
        env.update({"LOCAL_RANK": str(r), "LOCAL_WORLD_SIZE": str(a.nproc), "MASTER_ADDR": a.master_addr,
                    "GROUP_RANK": str(a.node_rank)})
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
