"""The usage example of the reference's module docstring
(tensorflow/contrib/mpi_collectives/__init__.py:81-111: a linear regression trained with
`mpi.DistributedOptimizer(tf.train.AdamOptimizer())`, the loss averaged with `mpi.allreduce`,
every rank feeding its own batch inside `mpi.Session()`), restated for this library.

    python -m tensorflow_allreduce_b200.launch --nproc 2 [--cpu] examples/linear_regression.py
"""
from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensorflow_allreduce_b200 as mpi          # the reference's users write `mpi.`


def construct_batch_for_rank(rank: int, step: int, device):
    g = torch.Generator().manual_seed(1000 * rank + step)
    x = torch.randn(64, 20, generator=g)
    w_true = torch.arange(20.0).reshape(20, 1) / 10
    return x.to(device), (x @ w_true + 0.5).to(device)


def main() -> int:
    # Use `mpi.Session` where the reference's example uses it instead of `tf.Session`
    with mpi.Session() as session:
        rank = mpi.rank()
        device = torch.device("cuda", torch.cuda.current_device()) if mpi.on_gpu() else torch.device("cpu")
        if rank == 0:
            print("MPI Size:", mpi.size())

        # A simple linear regression model (the same starting point on every rank)
        torch.manual_seed(0)
        W = torch.zeros(20, 1, device=device, requires_grad=True)
        B = torch.zeros(1, 1, device=device, requires_grad=True)

        # Training using allreduce with DistributedOptimizer
        optimizer = mpi.DistributedOptimizer(torch.optim.Adam([W, B], lr=0.05))
        first = last = None
        for step in range(60):
            # On different ranks, feed different input data.
            batch_inputs, batch_outputs = construct_batch_for_rank(rank, step, device)
            loss = 0.5 * ((batch_inputs @ W + B - batch_outputs) ** 2).sum() / batch_inputs.shape[0]
            optimizer.minimize(loss)
            # Average loss over all ranks, for printing.
            avg_loss = session.run(mpi.allreduce, loss.detach().reshape(1)).item()
            first = avg_loss if first is None else first
            last = avg_loss
        if rank == 0:
            print(f"Average Loss: {first:.4f} -> {last:.4f}")
        same = mpi.allgather(torch.cat([W.detach().reshape(-1), B.detach().reshape(-1)]).unsqueeze(0))
        return 0 if (last < 0.2 * first and bool((same == same[0:1]).all())) else 1


if __name__ == "__main__":
    sys.exit(main())
