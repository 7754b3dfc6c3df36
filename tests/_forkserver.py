"""A helper process that has `torch` and the package imported once and forks a child per rank, so
that a CPU test does not pay the interpreter start-up and the imports (about 3.5 s) for every rank
it runs. The helper never computes anything and never touches CUDA: it imports, then waits for
requests on its standard input (one JSON object per line) and answers on its standard output.

    {"op": "spawn", "script": path, "env": {...}, "stdout": path, "stderr": path}  ->  {"pid": n}
    {"op": "wait", "pid": n, "timeout": seconds}       ->  {"rc": code | null}    (null: still running)
    {"op": "kill", "pid": n, "dump": bool}             ->  {"rc": code}
    {"op": "quit"}

A child replaces its environment with the one of the request, points its output at the two files
and runs the script as `__main__`. Exit codes are those a separate interpreter would give (a
signal gives the negative signal number, as `subprocess` reports it).
"""
import json
import os
import signal
import sys
import time
import traceback


def _child(req):
    try:
        os.environ.clear()
        os.environ.update(req["env"])
        for path, fd in ((req["stdout"], 1), (req["stderr"], 2)):
            f = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
            os.dup2(f, fd)
            os.close(f)
        null = os.open(os.devnull, os.O_RDONLY)
        os.dup2(null, 0)
        os.close(null)
        sys.argv = [req["script"]]
        code = 0
        try:
            import runpy

            runpy.run_path(req["script"], run_name="__main__")
        except SystemExit as e:
            code = e.code if isinstance(e.code, int) else (0 if e.code is None else 1)
            if not isinstance(e.code, int) and e.code is not None:
                print(e.code, file=sys.stderr)
        except BaseException:
            traceback.print_exc()
            code = 1
    finally:
        try:
            sys.stdout.flush()
            sys.stderr.flush()
        except Exception:
            pass
    os._exit(code & 0xFF)


def _status_to_rc(status):
    if os.WIFSIGNALED(status):
        return -os.WTERMSIG(status)
    return os.WEXITSTATUS(status)


def main():
    import torch  # noqa: F401

    import tensorflow_allreduce_b200  # noqa: F401

    done = {}
    out = sys.stdout
    out.write(json.dumps({"ready": True}) + "\n")
    out.flush()

    def reap(pid, block_s):
        if pid in done:
            return done[pid]
        deadline = time.time() + block_s
        while True:
            got, status = os.waitpid(pid, os.WNOHANG)
            if got == pid:
                done[pid] = _status_to_rc(status)
                return done[pid]
            if time.time() >= deadline:
                return None
            time.sleep(0.005)

    for line in sys.stdin:
        req = json.loads(line)
        op = req.get("op")
        if op == "quit":
            break
        if op == "spawn":
            pid = os.fork()
            if pid == 0:
                _child(req)
            ans = {"pid": pid}
        elif op == "wait":
            ans = {"rc": reap(req["pid"], float(req.get("timeout", 0)))}
        elif op == "kill":
            pid = req["pid"]
            if reap(pid, 0) is None:
                try:
                    if req.get("dump"):
                        os.kill(pid, signal.SIGUSR1)      # scripts register faulthandler on it
                        time.sleep(0.5)
                    os.kill(pid, signal.SIGKILL)
                except OSError:
                    pass
            ans = {"rc": reap(pid, 10)}
        else:
            ans = {"error": f"unknown request {op!r}"}
        out.write(json.dumps(ans) + "\n")
        out.flush()


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    main()
