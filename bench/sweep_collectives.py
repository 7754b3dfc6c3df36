"""Bandwidth sweep of allreduce and variable allgather on 2/4/8 GPUs, with NCCL
(`torch.distributed`) and a restatement of the reference's ring as comparators.

    python -m torch.distributed.run --nproc-per-node N bench/sweep_collectives.py [--max-mb 1024] [--out file.json]

Message sizes are powers of two from 1 KiB; payloads fp32 and bf16 filled with U(-1,1), seed = rank.
Every number is device time (CUDA events) over several iterations, maximum over ranks.
Bus bandwidth: allreduce  busbw = bytes/time * 2(P-1)/P ;  allgather busbw = total_bytes/time * (P-1)/P.

Arms:
  ours_direct in-place allreduce on a tensor in symmetric memory, ordered launch without negotiation
              (zero-copy; the path gradient buckets take)
  ours_symm   the same through the name-keyed negotiated API (adds the coordinator round trip)
  ours_staged allreduce of an ordinary tensor (copied through the staging area)
  nccl        torch.distributed.all_reduce / all_gather on the same sizes
  (--fake-hosts H: the ranks report H host names, so ours_staged runs in two levels: NVLink kernels
   inside a "host", pinned memory and socket rings between them)
  ref_ring    the reference's algorithm (tensorflow/contrib/mpi_collectives/ring.h:136-228, ring.cu.cc:41-69):
              N-1 reduce-scatter steps of peer copy + a separate 32x256 accumulate launch + a
              stream synchronise after each, then N-1 allgather steps; a restatement over NCCL
              send/recv, not the original MPI binary.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch
import torch.distributed as dist

import tensorflow_allreduce_b200 as bc
from tensorflow_allreduce_b200.ops import symmetric


def timed(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    bc.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return max(bc.host_allgather(ms))


def ref_ring_allreduce(buf, tmp, rank, world):
    """Host-driven ring with a sync after every step, as the reference's GPU path does."""
    n = buf.numel()
    q, rem = divmod(n, world)
    starts = [i * q + min(i, rem) for i in range(world + 1)]
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for k in range(world - 1):
        si, ri = (rank - k) % world, (rank - k - 1) % world
        ops = [dist.P2POp(dist.isend, buf[starts[si]:starts[si + 1]], nxt), dist.P2POp(dist.irecv, tmp[:starts[ri + 1] - starts[ri]], prv)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        torch.cuda.current_stream().synchronize()
        buf[starts[ri]:starts[ri + 1]].add_(tmp[:starts[ri + 1] - starts[ri]])
        torch.cuda.current_stream().synchronize()
    for k in range(world - 1):
        si, ri = (rank - k + 1) % world, (rank - k) % world
        ops = [dist.P2POp(dist.isend, buf[starts[si]:starts[si + 1]], nxt), dist.P2POp(dist.irecv, buf[starts[ri]:starts[ri + 1]], prv)]
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        torch.cuda.current_stream().synchronize()


def main():
    if os.environ.get("BC_SWEEP_WATCHDOG_S"):
        import faulthandler
        faulthandler.dump_traceback_later(float(os.environ["BC_SWEEP_WATCHDOG_S"]), exit=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--min-kb", type=int, default=1)
    ap.add_argument("--out", default="")
    ap.add_argument("--arms", default="ours_direct,ours_symm,ours_staged,nccl,ref_ring")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--no-allgather", action="store_true")
    ap.add_argument("--no-allreduce", action="store_true")
    ap.add_argument("--fake-hosts", type=int, default=1,
                    help="report this many host names (consecutive ranks share one): times the two-level path on one box")
    a = ap.parse_args()
    arms = a.arms.split(",")
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if a.fake_hosts > 1:
        if world % a.fake_hosts:
            raise SystemExit("--fake-hosts must divide the number of ranks")
        os.environ["BC_HOSTNAME"] = f"host{rank // (world // a.fake_hosts)}"
        # tensors in symmetric memory and ordered launches need all ranks on one host
        arms = [x for x in arms if x in ("ours_staged", "nccl", "ref_ring")]
    torch.cuda.set_device(local)
    cfg = bc.Config.from_env(heap_mb=max(6 * a.max_mb + 64, 256), staging_mb=64)
    bc.init(device=local, config=cfg)
    use_nccl = ("nccl" in arms or "ref_ring" in arms) and world > 1
    if use_nccl:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rows = []
    sizes = []
    s = a.min_kb << 10
    while s <= a.max_mb << 20:
        sizes.append(s)
        s *= 2
    P = world
    for dname in a.dtypes.split(","):
        dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dname]
        es = 4 if dtype == torch.float32 else 2
        for nbytes in ([] if a.no_allreduce else sizes):
            n = nbytes // es
            iters = 50 if nbytes <= (1 << 20) else (20 if nbytes <= (64 << 20) else 5)
            g = torch.Generator(device="cuda").manual_seed(rank)
            x = (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
            row = {"op": "allreduce", "dtype": dname, "bytes": nbytes, "world": P}
            factor = 2 * (P - 1) / P if P > 1 else 1.0
            if "ours_direct" in arms:
                from tensorflow_allreduce_b200.ops.direct import allreduce_direct_
                sx = symmetric.empty((n,), dtype)
                sx.copy_(x)
                want = bc.allreduce(x, average=False, name=f"dchk.{dname}.{nbytes}")
                allreduce_direct_(sx)
                row["direct_correct"] = bool(torch.equal(sx, want))
                sx.zero_()
                ms = timed(lambda: allreduce_direct_(sx), iters)
                row["ours_direct_ms"] = ms
                row["ours_direct_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
                del sx
            if "ours_symm" in arms and nbytes <= (16 << 20):
                sx = symmetric.empty((n,), dtype)
                sx.copy_(x)
                # correctness once (sum), then time the in-place op (values grow; zeros avoid overflow)
                want = bc.allreduce(x, average=False, name=f"chk.{dname}.{nbytes}")
                bc.allreduce_(sx, average=False, name=f"chk2.{dname}.{nbytes}")
                row["symm_correct"] = bool(torch.equal(sx, want))
                sx.zero_()
                i = [0]

                def f():
                    i[0] += 1
                    bc.allreduce_(sx, average=False, name=f"s.{dname}.{nbytes}.{i[0]}")
                ms = timed(f, iters)
                row["ours_symm_ms"] = ms
                row["ours_symm_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
                row["ours_symm_algo"] = [e for e in bc.stats() if e["device"] == 1][-1]["algo"]
                del sx
            if "ours_staged" in arms:
                i = [0]

                def f2():
                    i[0] += 1
                    bc.allreduce(x, average=False, name=f"t.{dname}.{nbytes}.{i[0]}")
                ms = timed(f2, iters)
                row["ours_staged_ms"] = ms
                row["ours_staged_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
            if "nccl" in arms and use_nccl:
                y = x.clone()
                ms = timed(lambda: dist.all_reduce(y), iters)
                row["nccl_ms"] = ms
                row["nccl_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
            if "ref_ring" in arms and use_nccl and nbytes >= (1 << 12) and nbytes <= (256 << 20):
                y = x.clone()
                tmp = torch.empty(n // P + 1, dtype=dtype, device="cuda")
                ms = timed(lambda: ref_ring_allreduce(y, tmp, rank, P), max(2, iters // 5), warmup=1)
                row["ref_ring_ms"] = ms
                row["ref_ring_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
            rows.append(row)
            bc.clear_stats()
            if rank == 0:
                print(json.dumps(row), flush=True)
        if a.no_allgather:
            continue
        for nbytes in sizes:
            # rank r contributes (r+1)*k rows of 256 elements; total = nbytes
            cols = 256
            k = max(1, nbytes // (es * cols * (P * (P + 1) // 2)))
            t = (torch.ones((rank + 1) * k, cols, device="cuda") * rank).to(dtype)
            total = es * cols * k * (P * (P + 1) // 2)
            if total > (a.max_mb << 20):
                continue
            iters = 50 if total <= (1 << 20) else (20 if total <= (64 << 20) else 5)
            row = {"op": "allgather", "dtype": dname, "bytes": total, "world": P}
            out = bc.allgather(t, name=f"agchk.{dname}.{nbytes}")
            lo, ok = 0, True
            for r in range(P):
                ok = ok and bool((out[lo:lo + (r + 1) * k] == r).all())
                lo += (r + 1) * k
            row["correct"] = ok
            del out
            i = [0]

            def f3():
                i[0] += 1
                bc.allgather(t, name=f"ag.{dname}.{nbytes}.{i[0]}")
            ms = timed(f3, iters)
            factor = (P - 1) / P if P > 1 else 1.0
            row["ours_ms"] = ms
            row["ours_busbw"] = total / (ms * 1e-3) * factor / 1e9
            from tensorflow_allreduce_b200.ops.direct import allgatherv_direct
            # results of the timed calls above live in the symmetric heap until they are collected
            torch.cuda.synchronize()
            gc.collect()
            sym_out = symmetric.try_empty((total // (es * cols), cols), dtype, torch.device("cuda", local))
            if not all(bc.host_allgather(sym_out is not None)):
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
                continue
            szs = torch.zeros(P, dtype=torch.int64, device="cuda")
            sym_out.zero_()
            allgatherv_direct(t, sym_out, szs)
            lo, ok = 0, True
            for r in range(P):
                ok = ok and bool((sym_out[lo:lo + (r + 1) * k] == r).all()) and int(szs[r]) == (r + 1) * k * cols * es
                lo += (r + 1) * k
            row["direct_correct"] = ok
            ms = timed(lambda: allgatherv_direct(t, sym_out, szs), iters)
            row["ours_direct_ms"] = ms
            row["ours_direct_busbw"] = total / (ms * 1e-3) * factor / 1e9
            del sym_out
            if use_nccl and "nccl" in arms:
                # the usual workaround for a variable first dimension: pad to the largest slab
                pad = torch.zeros(P * k, cols, dtype=dtype, device="cuda")
                pad[:(rank + 1) * k] = t
                outp = torch.empty(P * P * k, cols, dtype=dtype, device="cuda")
                ms = timed(lambda: dist.all_gather_into_tensor(outp, pad), iters)
                row["nccl_padded_ms"] = ms
                row["nccl_padded_busbw"] = total / (ms * 1e-3) * factor / 1e9
            rows.append(row)
            bc.clear_stats()
            if rank == 0:
                print(json.dumps(row), flush=True)
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump({"world": P, "symm": symmetric.describe(), "rows": rows}, f, indent=1)
    if use_nccl:
        dist.destroy_process_group()
    bc.shutdown()


if __name__ == "__main__":
    main()
