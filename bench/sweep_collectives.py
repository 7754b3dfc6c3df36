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
  ours_staged allreduce of an ordinary tensor through the name-keyed API (negotiation + staging area)
  ours_private the same ordinary tensor with an ordered launch (`allreduce_direct_`): staging without negotiation,
              which is what NCCL's ordered `all_reduce` is comparable with
  ours_pipeline (not in the default list) ours_private with the staged pipeline kernel forced from 4 MiB on (the
              library uses it from 96 MiB): one launch whose copier blocks and reducer blocks work on different
              chunks of a ring in the staging area
  ours_nopipeline (not in the default list) ours_private with that kernel switched off: one kernel that copies in,
              reduces and copies out up to a quarter of the staging slice, a pipeline of kernels on three streams above
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


def timed(fn, iters=0, warmup=3):
    """Device time of one call of `fn` in ms (CUDA events around a loop, maximum over ranks).

    `iters` = 0 sizes the loop for about 30 ms of device time (10 to 200 calls, the same number on
    every rank). One more call runs between the host barrier and the first event: the collective
    itself lines the GPUs up, so the clock does not start while a rank is still on its way out of
    the barrier (with 5 calls of 0.2 ms such a skew was a tenth of the measurement)."""
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if iters <= 0:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            fn()
        e1.record()
        torch.cuda.synchronize()
        est = max(bc.host_allgather(e0.elapsed_time(e1) / 3))
        iters = int(min(200, max(10, 30.0 / max(est, 1e-3))))
    torch.cuda.synchronize()
    bc.barrier()
    fn()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return max(bc.host_allgather(ms))


def phases_of(fn):
    """Time stamps of block 0 inside the reduction kernel of one call of `fn` (%globaltimer at kernel entry, after
    the first barrier, after phase 1, after the second barrier, at the end), as durations in microseconds:
    [barrier 1, phase 1, barrier 2, phase 2]; maximum over ranks of each."""
    import ctypes as C

    from tensorflow_allreduce_b200 import _lib

    stamps = torch.zeros(8, dtype=torch.int64, device="cuda")
    lib = _lib.lib()
    fn()
    torch.cuda.synchronize()
    bc.barrier()
    # Two calls queued back to back: the first lines the GPUs up (the ranks leave a host barrier
    # tens of microseconds apart, and the first barrier of a kernel would show that skew), the
    # second is the one that writes the stamps.
    fn()
    lib.bc_set_allreduce_profile(C.c_void_p(stamps.data_ptr()))
    fn()
    lib.bc_set_allreduce_profile(None)
    torch.cuda.synchronize()
    t = stamps.tolist()
    d = [(t[i + 1] - t[i]) / 1e3 for i in range(4)]
    allv = bc.host_allgather(d)
    return [round(max(v[i] for v in allv), 2) for i in range(4)]


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


def _size(n):
    for unit, sh in (("GiB", 30), ("MiB", 20), ("KiB", 10)):
        if n >= (1 << sh):
            v = n / (1 << sh)
            return f"{v:.0f} {unit}" if v == int(v) else f"{v:.1f} {unit}"
    return f"{n} B"


def markdown(rows, world, link_measured=764.0, link_nominal=900.0):
    """The rows of one run as markdown tables (one per operation and dtype): time, bus GB/s per arm, the best of
    this library's arms as a fraction of the measured and of the nominal link rate, correctness flags."""
    out = []
    for op in ("allreduce", "allgather"):
        for dname in ("fp32", "bf16"):
            sel = [r for r in rows if r["op"] == op and r["dtype"] == dname]
            if not sel:
                continue
            arms = [k[:-6] for k in ("ours_direct_busbw", "ours_symm_busbw", "ours_staged_busbw", "ours_private_busbw", "ours_pipeline_busbw", "ours_nopipeline_busbw", "ours_busbw", "nccl_busbw",
                                      "nccl_padded_busbw", "ref_ring_busbw") if any(k in r for r in sel)]
            out.append(f"\n### {op}, {world} GPUs, {dname}\n")
            head = ["bytes"] + [f"{a_} ms" for a_ in arms if a_.startswith("ours")] + [f"{a_} GB/s" for a_ in arms]
            head += [f"ours / {link_measured:.0f}", f"ours / {link_nominal:.0f}", "correct"]
            if any("direct_phases_us" in r for r in sel):
                head.append("direct: barrier 1 / phase 1 / barrier 2 / phase 2 (us)")
            out.append("| " + " | ".join(head) + " |")
            out.append("|" + "---|" * len(head))
            for r in sel:
                cells = [_size(r["bytes"])]
                cells += [f'{r[a_ + "_ms"]:.4f}' if a_ + "_ms" in r else "-" for a_ in arms if a_.startswith("ours")]
                cells += [f'{r[a_ + "_busbw"]:.1f}' if a_ + "_busbw" in r else "-" for a_ in arms]
                best = max([r[a_ + "_busbw"] for a_ in arms if a_.startswith("ours") and a_ + "_busbw" in r] or [0.0])
                cells += [f"{best / link_measured:.2f}", f"{best / link_nominal:.2f}"]
                flags = [k.split("_")[0] + ("=ok" if r[k] else "=WRONG") for k in ("direct_correct", "symm_correct", "staged_correct", "private_correct", "pipeline_correct", "nopipeline_correct", "correct") if k in r]
                cells.append(" ".join(flags) or "-")
                if any("direct_phases_us" in x for x in sel):
                    cells.append(" / ".join(f"{v:.1f}" for v in r["direct_phases_us"]) if "direct_phases_us" in r else "-")
                out.append("| " + " | ".join(cells) + " |")
    return "\n".join(out) + "\n"


def main():
    if os.environ.get("BC_SWEEP_WATCHDOG_S"):
        import faulthandler
        faulthandler.dump_traceback_later(float(os.environ["BC_SWEEP_WATCHDOG_S"]), exit=True)
    ap = argparse.ArgumentParser()
    ap.add_argument("--max-mb", type=int, default=1024)
    ap.add_argument("--min-kb", type=int, default=1)
    ap.add_argument("--out", default="")
    ap.add_argument("--arms", default="ours_direct,ours_symm,ours_staged,ours_private,nccl,ref_ring")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--no-allgather", action="store_true")
    ap.add_argument("--no-allreduce", action="store_true")
    ap.add_argument("--phases", action="store_true", help="ours_direct: also record the kernel's phase times (block 0 time stamps)")
    ap.add_argument("--phases-min-kb", type=int, default=1024)
    ap.add_argument("--pipeline-mode", type=int, default=2, help="arm ours_pipeline: 1 = only where the switch reduces, 2 = always")
    ap.add_argument("--staging-mb", type=int, default=0, help="size of the staging area (0 = the library's default)")
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
        arms = [x for x in arms if x in ("ours_staged", "nccl", "ref_ring")]   # ours_private is an ordered launch as well
    torch.cuda.set_device(local)
    cfg = bc.Config.from_env(heap_mb=max(6 * a.max_mb + 64, 256), staging_mb=a.staging_mb or None)
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
            iters = 0
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
                if a.phases and nbytes >= (a.phases_min_kb << 10) and nbytes <= (512 << 20):
                    row["direct_phases_us"] = phases_of(lambda: allreduce_direct_(sx))
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
                got = bc.allreduce(x, average=False, name=f"tchk.{dname}.{nbytes}")
                ref = x.clone()
                if use_nccl:
                    dist.all_reduce(ref)
                    # NCCL's summation order differs: equal within the rounding of a P-term sum
                    tol = 1e-5 * P if dtype == torch.float32 else 1e-2 * P
                    row["staged_correct"] = bool(torch.allclose(got.float(), ref.float(), rtol=tol, atol=tol))
                del got, ref
                ms = timed(f2, iters)
                row["ours_staged_ms"] = ms
                row["ours_staged_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
            if "ours_private" in arms:
                from tensorflow_allreduce_b200.ops.direct import allreduce_direct_
                y = x.clone()
                allreduce_direct_(y)
                ref = x.clone()
                if use_nccl:
                    dist.all_reduce(ref)
                    tol = 1e-5 * P if dtype == torch.float32 else 1e-2 * P
                    row["private_correct"] = bool(torch.allclose(y.float(), ref.float(), rtol=tol, atol=tol))
                y.zero_()
                del ref
                ms = timed(lambda: allreduce_direct_(y), iters)
                row["ours_private_ms"] = ms
                row["ours_private_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
                del y
            for arm, mode, min_mb in (("ours_pipeline", a.pipeline_mode, 4), ("ours_nopipeline", 0, 0)):
                # the same ordered launch with the staged pipeline kernel forced from 4 MiB on / switched off for this arm
                if arm not in arms:
                    continue
                from tensorflow_allreduce_b200 import _lib
                from tensorflow_allreduce_b200.ops.direct import allreduce_direct_
                _lib.lib().bc_set_option(b"staged_pipeline", mode)
                _lib.lib().bc_set_option(b"pipeline_min_bytes", max(min_mb, 1) << 20)
                y = x.clone()
                allreduce_direct_(y)
                ref = x.clone()
                if use_nccl:
                    dist.all_reduce(ref)
                    tol = 1e-5 * P if dtype == torch.float32 else 1e-2 * P
                    row[arm[5:] + "_correct"] = bool(torch.allclose(y.float(), ref.float(), rtol=tol, atol=tol))
                y.zero_()
                del ref
                ms = timed(lambda: allreduce_direct_(y), iters)
                row[arm + "_ms"] = ms
                row[arm + "_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
                del y
                _lib.lib().bc_set_option(b"staged_pipeline", cfg.staged_pipeline)
                _lib.lib().bc_set_option(b"pipeline_min_bytes", cfg.pipeline_min_mb << 20)
                bc.check_device_status()
            if "nccl" in arms and use_nccl:
                y = x.clone()
                ms = timed(lambda: dist.all_reduce(y), iters)
                row["nccl_ms"] = ms
                row["nccl_busbw"] = nbytes / (ms * 1e-3) * factor / 1e9
            if "ref_ring" in arms and use_nccl and nbytes >= (1 << 12) and nbytes <= (256 << 20):
                y = x.clone()
                tmp = torch.empty(n // P + 1, dtype=dtype, device="cuda")
                ms = timed(lambda: ref_ring_allreduce(y, tmp, rank, P), 3 if nbytes <= (64 << 20) else 2, warmup=1)
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
            iters = 0
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
            # ordered launches need all ranks on one host
            sym_out = None if a.fake_hosts > 1 else symmetric.try_empty((total // (es * cols), cols), dtype, torch.device("cuda", local))
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
        with open(os.path.splitext(a.out)[0] + ".md", "w") as f:
            f.write(markdown(rows, P))
    if use_nccl:
        dist.destroy_process_group()
    bc.shutdown()


if __name__ == "__main__":
    main()
