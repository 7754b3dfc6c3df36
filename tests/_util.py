"""Shared helpers for multi-process tests: run a worker script as N ranks and collect one JSON
result line per rank. CPU ranks are forked from a helper process that has torch imported
(`_forkserver.py`; BC_TEST_FORKSERVER=0 starts a fresh interpreter per rank instead, which is
also what GPU ranks always get)."""
import json
import os
import textwrap

from tensorflow_allreduce_b200.utils.spawn import run_script

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

PRELUDE = f"""
import faulthandler, json, os, signal, sys
faulthandler.register(signal.SIGUSR1, all_threads=True)      # the runner asks for the stacks of a rank it is about to kill
sys.path.insert(0, {ROOT!r})
import torch
import tensorflow_allreduce_b200 as bc
RANK = int(os.environ["RANK"]); SIZE = int(os.environ["WORLD_SIZE"])
def emit(**kw):
    print("RESULT " + json.dumps(kw), flush=True)
"""


class _ForkServer:
    """Client of `tests/_forkserver.py`: CPU ranks are forked from a process that has torch imported."""

    def __init__(self):
        import subprocess
        import sys

        env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
        self.proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "_forkserver.py")], stdin=subprocess.PIPE,
                                     stdout=subprocess.PIPE, text=True, env=env, cwd=ROOT)
        if not json.loads(self.proc.stdout.readline()).get("ready"):
            raise RuntimeError("the fork server did not start")

    def ask(self, **req):
        self.proc.stdin.write(json.dumps(req) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline()
        if not line:
            raise RuntimeError("the fork server went away")
        return json.loads(line)

    def close(self):
        try:
            self.proc.stdin.write(json.dumps({"op": "quit"}) + "\n")
            self.proc.stdin.flush()
            self.proc.wait(timeout=10)
        except Exception:
            self.proc.kill()


_server = None


def _fork_server():
    """The shared helper, or None when it is switched off (BC_TEST_FORKSERVER=0) or cannot start."""
    global _server
    if os.environ.get("BC_TEST_FORKSERVER", "1") == "0":
        return None
    if _server is None:
        import atexit

        try:
            _server = _ForkServer()
            atexit.register(_server.close)
        except Exception:
            _server = False
    return _server or None


def _run_forked(server, source: str, nranks: int, timeout: float, env, per_rank_env):
    import tempfile
    import time

    from tensorflow_allreduce_b200.utils.spawn import RankResult, free_port, rank_env

    port = free_port()
    with tempfile.TemporaryDirectory() as tmp:
        script = os.path.join(tmp, "rank.py")
        with open(script, "w") as f:
            f.write(source)
        pids = []
        for r in range(nranks):
            e = rank_env(r, nranks, port, env, gpus=False)
            if per_rank_env and r in per_rank_env:
                e.update({k: str(v) for k, v in per_rank_env[r].items()})
            pids.append(server.ask(op="spawn", script=script, env=e, stdout=os.path.join(tmp, f"out{r}"),
                                   stderr=os.path.join(tmp, f"err{r}"))["pid"])
        deadline = time.time() + timeout
        results = []
        for r, pid in enumerate(pids):
            rc = None
            while rc is None and time.time() < deadline:
                rc = server.ask(op="wait", pid=pid, timeout=min(1.0, max(0.0, deadline - time.time())))["rc"]
            if rc is None:
                server.ask(op="kill", pid=pid, dump=True)       # reported like a rank that subprocess had to kill
            results.append(RankResult(r, rc, open(os.path.join(tmp, f"out{r}")).read(), open(os.path.join(tmp, f"err{r}")).read()))
        return results


def run(body: str, nranks: int = 2, timeout: float = 120.0, env=None, per_rank_env=None, gpus=False, expect_ok=True):
    env = dict(env or {})
    if not gpus:
        # A stuck host-side wait reports itself before the runner's deadline. GPU ranks keep the
        # library's default: context creation and the first launches can take a while on a cold box.
        env.setdefault("BC_TIMEOUT_S", str(max(10, int(timeout * 0.8))))
    source = PRELUDE + textwrap.dedent(body)
    server = None if gpus else _fork_server()
    if server is not None:
        res = _run_forked(server, source, nranks, timeout, env, per_rank_env)
    else:
        res = run_script(source, nranks, timeout=timeout, env=env, per_rank_env=per_rank_env, gpus=gpus, dump_stacks=True)
    out = []
    for r in res:
        rec = None
        for line in r.stdout.splitlines():
            if line.startswith("RESULT "):
                rec = json.loads(line[7:])
        if expect_ok:
            assert r.returncode == 0, f"rank {r.rank} exited with {r.returncode}\nstdout:\n{r.stdout}\nstderr:\n{r.stderr[-4000:]}"
            assert rec is not None, f"rank {r.rank} printed no result\n{r.stdout}\n{r.stderr[-2000:]}"
        out.append((r, rec))
    return out
