"""The control plane, the CPU ring and the runtime under ThreadSanitizer and AddressSanitizer:
three ranks run as threads of one process (csrc/selftest/host_selftest.cc), once per CPU transport. The reference
configures no sanitizer and its coordinator state has data races
(tensorflow/contrib/mpi_collectives/mpi_ops.cc:593,621,816-821)."""
import os
import subprocess

import pytest

from tensorflow_allreduce_b200 import build
from tensorflow_allreduce_b200.utils.spawn import free_port as _free_port


@pytest.mark.parametrize("transport", ["shm", "ring"])
@pytest.mark.parametrize("sanitizer", ["thread", "address"])
def test_host_runtime_is_clean_under_sanitizer(sanitizer, transport):
    try:
        exe = build.build_selftest(sanitizer)
    except RuntimeError as e:
        if "no C++ compiler" in str(e):
            pytest.skip(str(e))
        raise
    # CPU tensors through the shared-memory segment (small slots: several chunks) or the socket ring;
    # with shared memory the two-level pass cuts its tensors into 1 KiB chunks, so that the step
    # between the hosts runs on its helper thread beside the steps inside the host
    env = dict(os.environ, **({"BC_SHM": "0"} if transport == "ring" else {"BC_SHM_SLOT_KB": "4", "BC_TWO_LEVEL_CHUNK_KB": "1"}))
    # second port: a second pass with 4 ranks on two host names (node groups, rails, two levels)
    r = subprocess.run([str(exe), "3", str(_free_port()), str(_free_port())], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-6000:]
    assert "host_selftest ok" in r.stdout
    assert "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr
