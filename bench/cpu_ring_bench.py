"""Timed CPU baseline: sum-allreduce and variable allgather of a CPU group, the data path that plays
the role of the reference's `RingAllreduce<CPU>` / `RingAllgather<CPU>`
(tensorflow/contrib/mpi_collectives/ring.h:136-301, ring.cc:36-50). Ranks of one host exchange the
data through shared memory; `BC_SHM=0` times the socket ring (loopback TCP) instead.

    python -m tensorflow_allreduce_b200.launch --nproc 2 --cpu bench/cpu_ring_bench.py [--max-mb 64]
    BC_SHM=0 python -m tensorflow_allreduce_b200.launch --nproc 2 --cpu bench/cpu_ring_bench.py
    ... bench/cpu_ring_bench.py --gloo        (adds torch.distributed's gloo all_reduce, in place, as a comparator)
    ... --nproc 4 --cpu bench/cpu_ring_bench.py --fake-hosts 2      (two made-up hosts of two ranks: two levels)

Wall-clock time per call (host timers, maximum over ranks) through the public, name-keyed API, so
the coordinator round trip is included; `allreduce_inplace_ms` is the same without an output to
allocate, `allreduce_data_phase_ms` the part after the negotiation (from `stats()`). Bus bandwidth
as in the GPU sweep.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

import tensorflow_allreduce_b200 as bc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--gloo", action="store_true", help="also time torch.distributed's gloo backend on the same tensors")
    ap.add_argument("--fake-hosts", type=int, default=1, help="the ranks report this many host names (equal shares): the allreduce "
                    "then runs in two levels, shared memory inside a \"host\" and rails between them (BC_TWO_LEVEL_CHUNK_KB=0: in one piece)")
    ap.add_argument("--min-kb", type=int, default=1)
    a = ap.parse_args()
    if a.fake_hosts > 1:
        rank_, world_ = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        os.environ["BC_HOSTNAME"] = f"host{rank_ // (world_ // a.fake_hosts)}"
        os.environ["LOCAL_RANK"] = "-1"
    bc.init(device="cpu")
    rank, P = bc.rank(), bc.size()
    if a.gloo:
        import torch.distributed as dist

        port = bc.host_allgather(__import__("tensorflow_allreduce_b200.utils.spawn", fromlist=["free_port"]).free_port())[0]
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=P)
    s = a.min_kb << 10
    while s <= a.max_mb << 20:
        n = s // 4
        x = torch.full((n,), float(rank + 1))
        want = float(P * (P + 1) // 2)
        times = []
        for it in range(a.iters + 2):
            bc.barrier()
            t0 = time.perf_counter()
            y = bc.allreduce(x, average=False, name=f"ar.{s}.{it}")
            t1 = time.perf_counter()
            if it >= 2:
                times.append(t1 - t0)
        ok = bool(y[0] == want and y[-1] == want)
        sec = max(bc.host_allgather(sorted(times)[len(times) // 2]))
        # in place (no output to allocate and fault in), and the data phase alone from the library's records
        z = torch.zeros(n)
        bc.clear_stats()
        tin = []
        for it in range(a.iters + 2):
            bc.barrier()
            t0 = time.perf_counter()
            bc.allreduce_(z, average=False, name=f"ip.{s}.{it}")
            t1 = time.perf_counter()
            if it >= 2:
                tin.append(t1 - t0)
        sec_in = max(bc.host_allgather(sorted(tin)[len(tin) // 2]))
        recs = [e for e in bc.stats() if e["name"].startswith("ip.")][2:]
        data = sorted(e["t_done"] - e["t_negotiated"] for e in recs)[len(recs) // 2]
        sec_data = max(bc.host_allgather(data))
        gloo_ms = None
        if a.gloo:
            w = torch.zeros(n)
            tg = []
            for it in range(a.iters + 2):
                bc.barrier()
                t0 = time.perf_counter()
                dist.all_reduce(w)
                t1 = time.perf_counter()
                if it >= 2:
                    tg.append(t1 - t0)
            gloo_ms = round(max(bc.host_allgather(sorted(tg)[len(tg) // 2])) * 1e3, 4)
        rows = max(1, n // 256 // (P * (P + 1) // 2))
        t = torch.full(((rank + 1) * rows, 256), float(rank))
        gt = []
        for it in range(a.iters + 2):
            bc.barrier()
            t0 = time.perf_counter()
            g = bc.allgather(t, name=f"ag.{s}.{it}")
            t1 = time.perf_counter()
            if it >= 2:
                gt.append(t1 - t0)
        gsec = max(bc.host_allgather(sorted(gt)[len(gt) // 2]))
        total = g.numel() * 4
        if rank == 0:
            print(json.dumps({"bytes": s, "world": P, "transport": [e["algo"] for e in bc.stats() if e["op"] == "allreduce"][-1], "allreduce_ms": round(sec * 1e3, 4), "allreduce_busbw_gbs": round(s / sec * 2 * (P - 1) / P / 1e9, 3),
                              "allreduce_inplace_ms": round(sec_in * 1e3, 4), "allreduce_data_phase_ms": round(sec_data * 1e3, 4),
                              "gloo_allreduce_inplace_ms": gloo_ms,
                              "correct": ok, "allgather_total_bytes": total, "allgather_ms": round(gsec * 1e3, 4),
                              "allgather_busbw_gbs": round(total / gsec * (P - 1) / P / 1e9, 3)}), flush=True)
        s *= 4
    if a.gloo:
        dist.destroy_process_group()
    bc.shutdown()


if __name__ == "__main__":
    main()
