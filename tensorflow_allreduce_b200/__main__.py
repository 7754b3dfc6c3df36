"""`python -m tensorflow_allreduce_b200`: what is installed and how it is configured.

Prints the native library (path, whether it matches the sources), the devices PyTorch sees, the
effective `BC_*` settings and the launcher's variables found in the environment; with `--check`
it also runs a one-rank allreduce on the CPU (and on `cuda:0` when there is one)."""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tensorflow_allreduce_b200")
    ap.add_argument("--check", action="store_true", help="run a one-rank allreduce as a self-check")
    a = ap.parse_args(argv)
    import torch

    import tensorflow_allreduce_b200 as bc
    from tensorflow_allreduce_b200 import build
    from tensorflow_allreduce_b200.config import Config

    info = {
        "version": bc.__version__,
        "library": str(build.LIB),
        "library_built": build.LIB.exists(),
        "library_matches_sources": build.LIB.exists() and not build.needs_build(),
        "debug_library_built": build.LIB_DEBUG.exists(),
        "torch": torch.__version__,
        "cuda_devices": [torch.cuda.get_device_name(i) for i in range(torch.cuda.device_count())] if torch.cuda.is_available() else [],
        "config": dataclasses.asdict(Config.from_env()),
        "environment": {k: v for k, v in sorted(os.environ.items())
                        if k.startswith("BC_") or k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT")
                        or k.startswith("OMPI_COMM_WORLD_") or k.startswith("PMI_")},
    }
    if a.check:
        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            os.environ.pop(k, None)
        devices = ["cpu"] + (["cuda:0"] if torch.cuda.is_available() else [])
        info["check"] = {}
        for dev in devices:
            bc.init(device=dev)
            try:
                x = torch.arange(8.0, device=dev)
                info["check"][dev] = bool(torch.equal(bc.allreduce(x, average=False), x))
            finally:
                bc.shutdown()
    print(json.dumps(info, indent=1))
    return 0 if all(info.get("check", {}).values()) else 1


if __name__ == "__main__":
    sys.exit(main())
