"""The bounds-checked build of the kernels (`-DBC_DEBUG`, lib/libbcoll_debug.so, selected with
BC_DEBUG_KERNELS=1): the ordinary emulated-rank tests must pass under it with a clean status
word, and a request whose destination does not fit its segment must be refused with the bounds
status instead of storing out of range."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(code_or_args, timeout=600):
    env = dict(os.environ, BC_DEBUG_KERNELS="1")
    return subprocess.run([sys.executable] + code_or_args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_kernel_tests_pass_under_bounds_checks():
    r = _run(["-m", "pytest", "tests/test_gpu_emulated.py", "-x", "-q", "-k",
              "matches_reference or exhaustive or fused_update or allgatherv or prod_min_max"])
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]


def test_out_of_range_allgather_is_refused_not_executed():
    code = r"""
import sys, torch
sys.path.insert(0, %r)
from tensorflow_allreduce_b200 import _lib
from tensorflow_allreduce_b200.ops.emulated import EmulatedGroup
assert _lib.lib()._name.endswith("libbcoll_debug.so")
g = EmulatedGroup(4, 1 << 20)
ins = [torch.full((128,), float(r), device="cuda") for r in range(4)]      # 2 KiB in total
# 1 KiB before the end of the 1 MiB buffers: the last KiB would land in the guard region that
# follows every buffer (still inside its allocation), so even an unchecked store could not fault.
g.allgatherv(ins, [(1 << 20) - 1024] * 4, blocks=2)
torch.cuda.synchronize()
print("STATUS", hex(g.status), "DAMAGED", g.damaged_guard_bytes())
g.close()
""" % ROOT
    r = _run(["-c", code], timeout=120)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("STATUS")][0].split()
    assert int(line[1], 16) & 0x40000000, line          # kStatusBounds
    assert int(line[3]) == 0                             # nothing was stored past a buffer
