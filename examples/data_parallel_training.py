"""Synchronous data-parallel training in the shape of the reference's usage example
(tensorflow/contrib/mpi_collectives/README.md: `mpi.Session()`, `mpi.DistributedOptimizer(opt)`,
`mpi.rank()`, one process per GPU), on synthetic data.

    python -m tensorflow_allreduce_b200.launch --nproc 2 [--cpu] examples/data_parallel_training.py [--steps 20]
    torchrun --nproc-per-node 8 examples/data_parallel_training.py

Every rank builds the same model, takes its own shard of each batch, and the wrapped optimizer
averages the gradients while backward runs (on GPUs the momentum-SGD update is fused into the
reduction kernel). Rank 0 prints the loss; all ranks end with identical weights.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensorflow_allreduce_b200 as bc


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--batch", type=int, default=32, help="per rank")
    a = ap.parse_args()
    with bc.Session():                                   # init() on entry, shutdown() on exit
        dev = torch.device("cuda", torch.cuda.current_device()) if bc.on_gpu() else torch.device("cpu")
        torch.manual_seed(0)                             # same initial weights everywhere ...
        model = torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10)).to(dev)
        bc.broadcast_parameters(model, root=0)           # ... or make them the same explicitly
        opt = bc.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9))
        gen = torch.Generator().manual_seed(1000 + bc.rank())      # every rank draws its own shard
        w_true = torch.randn(64, 10, generator=torch.Generator().manual_seed(7))
        first = last = None
        for step in range(a.steps):
            x = torch.randn(a.batch, 64, generator=gen)
            y = (x @ w_true).argmax(dim=1)
            loss = opt.minimize(torch.nn.functional.cross_entropy(model(x.to(dev)), y.to(dev)))
            mean_loss = bc.allreduce(loss.reshape(1), average=True).item()
            first = mean_loss if first is None else first
            last = mean_loss
            if bc.rank() == 0 and (step % 5 == 0 or step == a.steps - 1):
                print(f"step {step:3d}  loss {mean_loss:.4f}", flush=True)
        flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
        everyone = bc.allgather(flat.unsqueeze(0))
        same = bool((everyone == everyone[0:1]).all())
        if bc.rank() == 0:
            print(f"ranks {bc.size()}  fused update {opt.fused}  loss {first:.4f} -> {last:.4f}  identical weights {same}", flush=True)
        return 0 if (same and last < first) else 1


if __name__ == "__main__":
    sys.exit(main())
