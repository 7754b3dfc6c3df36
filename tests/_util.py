"""Shared helpers for multi-process tests: run a worker script as N ranks and collect one JSON
result line per rank."""
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


def run(body: str, nranks: int = 2, timeout: float = 120.0, env=None, per_rank_env=None, gpus=False, expect_ok=True):
    env = dict(env or {})
    if not gpus:
        # A stuck host-side wait reports itself before the runner's deadline. GPU ranks keep the
        # library's default: context creation and the first launches can take a while on a cold box.
        env.setdefault("BC_TIMEOUT_S", str(max(10, int(timeout * 0.8))))
    res = run_script(PRELUDE + textwrap.dedent(body), nranks, timeout=timeout, env=env, per_rank_env=per_rank_env, gpus=gpus,
                     dump_stacks=True)
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
