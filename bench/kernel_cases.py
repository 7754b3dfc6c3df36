"""Small, self-contained cases of the library's own kernels, for timing and for profiler captures.

    python bench/kernel_cases.py --case fused_sgd        [--mb 256] [--iters 10]
    python bench/kernel_cases.py --case fused_adamw_bf16
    python bench/kernel_cases.py --case emu_allreduce    (8 emulated ranks on one GPU, two-shot, fp32)
    python bench/kernel_cases.py --case emu_one_shot --kb 256   (8 emulated ranks, one-shot, small message)
    python bench/kernel_cases.py --case emu_allgatherv
    python bench/kernel_cases.py --case gru [--T 350]    (one bidirectional GRU layer 2048 -> 1024, batch 32: persistent kernels vs cuDNN)
    python bench/kernel_cases.py --case bn_clip          (batch norm + clipped ReLU on [32, 32, 81, 350], the speech model's first block: fused kernels vs torch)

Each case prints one JSON line with the CUDA-event time per launch, the algorithmic bytes moved and
the resulting GB/s next to the measured copy bandwidth (`MEASURED_PEAKS.json` when present).
Inputs are larger than the 126 MB L2.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch


def peak_hbm():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return json.load(open(p))["hbm_gbs"], "measured"
    except Exception:
        return 6650.0, "fallback"


def timed(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True, choices=["fused_sgd", "fused_adamw_bf16", "emu_allreduce", "emu_one_shot", "emu_allgatherv", "gru", "bn_clip"])
    ap.add_argument("--mb", type=int, default=256, help="gradient / message size in MiB")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--blocks", type=int, default=0)
    ap.add_argument("--T", type=int, default=350, help="gru: time steps")
    ap.add_argument("--kb", type=int, default=256, help="emu_one_shot: message size in KiB")
    a = ap.parse_args()
    torch.cuda.set_device(0)
    hbm, src = peak_hbm()
    out = {"case": a.case, "mb": a.mb}

    if a.case == "bn_clip":
        import torch.nn.functional as F

        from tensorflow_allreduce_b200.ops.bn_clip import bn_clip

        n, c, h, w = 32, 32, 81, 350
        torch.manual_seed(0)
        x = torch.randn(n, c, h, w, device="cuda").requires_grad_(True)
        wt = (torch.rand(c, device="cuda") + 0.5).requires_grad_(True)
        b = torch.randn(c, device="cuda").requires_grad_(True)
        rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
        dy = torch.randn(n, c, h, w, device="cuda")
        res = {}
        for name, fn in (("fused", lambda: bn_clip(x, wt, b, rm, rv, 1e-5, 0.1, 20.0)),
                         ("torch", lambda: F.hardtanh(F.batch_norm(x, rm, rv, wt, b, True, 0.1, 1e-5), 0.0, 20.0))):
            f, bw = [], []
            for it in range(a.iters + 3):
                x.grad = wt.grad = b.grad = None
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                torch.cuda.synchronize()
                e0.record(); y = fn(); e1.record(); y.backward(dy); e2.record()
                torch.cuda.synchronize()
                if it >= 3:
                    f.append(e0.elapsed_time(e1)); bw.append(e1.elapsed_time(e2))
            res[name] = {"fwd_ms": sum(f) / len(f), "bwd_ms": sum(bw) / len(bw)}
        nbytes = x.numel() * 4
        # forward: x read twice, y written; backward: x and dy read twice, dx written
        out.update(shape=[n, c, h, w], tensor_mb=round(nbytes / 2 ** 20, 1),
                   **{k + "_" + kk: round(vv, 4) for k, v in res.items() for kk, vv in v.items()},
                   fused_fwd_gbs=3 * nbytes / res["fused"]["fwd_ms"] / 1e6, fused_bwd_gbs=5 * nbytes / res["fused"]["bwd_ms"] / 1e6)
        out["hbm_peak_gbs"] = hbm
        out["fwd_frac_of_hbm_copy_" + src] = out["fused_fwd_gbs"] / hbm
        out["bwd_frac_of_hbm_copy_" + src] = out["fused_bwd_gbs"] / hbm
        print(json.dumps(out))
        return
    if a.case == "gru":
        from tensorflow_allreduce_b200.ops import persistent_gru as pg

        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
        T, B, I, H = a.T, 32, 2048, 1024
        torch.manual_seed(0)
        rnn = torch.nn.GRU(I, H, num_layers=1, bidirectional=True).cuda()
        x = torch.randn(T, B, I, device="cuda", requires_grad=True)
        res = {}
        for name, fn in (("persistent", lambda: pg.gru_forward(rnn, x)), ("cudnn", lambda: rnn(x)[0])):
            f, b = [], []
            for it in range(a.iters + 2):
                e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
                torch.cuda.synchronize()
                e0.record(); y = fn(); e1.record(); y.sum().backward(); e2.record()
                torch.cuda.synchronize()
                if it >= 2:
                    f.append(e0.elapsed_time(e1)); b.append(e1.elapsed_time(e2))
            res[name] = {"fwd_ms": sum(f) / len(f), "bwd_ms": sum(b) / len(b)}
        pg.check_status()
        # recurrent work of one layer: 2 directions x T steps x (B x H x 3H) MACs forward, the same again backward
        flop = 2 * 2 * T * B * H * 3 * H
        out.update(T=T, batch=B, hidden=H, **{k + "_" + kk: round(vv, 3) for k, v in res.items() for kk, vv in v.items()},
                   recurrent_gflop_per_pass=flop / 1e9)
        print(json.dumps(out))
        return
    if a.case.startswith("fused"):
        import tensorflow_allreduce_b200 as bc
        from tensorflow_allreduce_b200 import _lib
        from tensorflow_allreduce_b200.ops import fused_optim as fo

        for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
            os.environ.pop(k, None)
        if a.blocks:
            os.environ["BC_MAX_BLOCKS"] = str(a.blocks)
        bc.init(device=0)
        lib = _lib.lib()
        bf16 = a.case == "fused_adamw_bf16"
        dtype = torch.bfloat16 if bf16 else torch.float32
        n = (a.mb << 20) // (2 if bf16 else 4)
        grad = torch.randn(n, device="cuda").to(dtype)
        param = torch.randn(n, device="cuda").to(dtype)
        master = param.float() if bf16 else None
        s1 = torch.zeros(n, device="cuda")
        s2 = torch.zeros(n, device="cuda") if bf16 else None
        h = fo.adam_hyper(1e-3, 3, weight_decay=0.01, zero_grad=True) if bf16 else fo.sgd_hyper(3e-4, momentum=0.9, zero_grad=True)
        stream = torch.cuda.current_stream()
        ev0, ev1 = torch.cuda.Event(), torch.cuda.Event()
        ev0.record(); ev1.record()

        def fn():
            ev0.record(stream)
            rc = lib.bc_fused_step(1, C.c_void_p(grad.data_ptr()), n, 3 if bf16 else 0, C.c_void_p(param.data_ptr()),
                                   C.c_void_p(master.data_ptr()) if bf16 else None, C.c_void_p(s1.data_ptr()),
                                   C.c_void_p(s2.data_ptr()) if bf16 else None, C.byref(h), 1.0, C.c_void_p(ev0.cuda_event),
                                   C.c_void_p(ev1.cuda_event), 0)
            assert rc >= 0, _lib.last_error()
            stream.wait_event(ev1)

        ms = timed(fn, a.iters)
        # bytes: grad read + grad zeroed, param (and master) read+write, state read+write
        es = 2 if bf16 else 4
        nbytes = n * (es + es) + (n * (2 + 4 + 4) if bf16 else n * 8) + n * 8 * (2 if bf16 else 1)
        out.update(ms=ms, bytes=nbytes, gbs=nbytes / ms / 1e6)
        bc.shutdown()
    else:
        from tensorflow_allreduce_b200.ops.emulated import EmulatedGroup

        P = 8
        per_rank = max(a.mb, 8) << 20
        g = EmulatedGroup(P, per_rank)
        blocks = a.blocks or g.max_blocks()
        if a.case == "emu_one_shot":
            n = (a.kb << 10) // 4
            for r in range(P):
                g.buffer(r, torch.float32, n).fill_(float(r))
            outs = [torch.empty(n, device="cuda") for _ in range(P)]
            blocks = a.blocks or max(1, min(blocks, (a.kb + 31) // 32))
            ms = timed(lambda: g.allreduce(n, torch.float32, "one_shot", outs=outs, blocks=blocks, scale=1.0 / P), a.iters)
            nbytes = P * (P * n * 4 + n * 4)     # every rank reads all P copies and writes one result
            out.update(ms=ms, bytes=nbytes, gbs=nbytes / ms / 1e6, blocks=blocks, ok=bool(g.status == 0 and float(outs[3][5]) == 3.5))
        elif a.case == "emu_allreduce":
            n = (a.mb << 20) // 4
            for r in range(P):
                g.buffer(r, torch.float32, n).fill_(float(r))
            ms = timed(lambda: g.allreduce(n, torch.float32, "two_shot", blocks=blocks, scale=1.0 / P), a.iters)
            # per rank: reads P slices of n/P and writes P copies of n/P; in total over the GPU:
            nbytes = P * (n * 4 + n * 4)
            out.update(ms=ms, bytes=nbytes, gbs=nbytes / ms / 1e6, blocks=blocks, ok=bool(g.status == 0))
        else:
            rows = (a.mb << 20) // (4 * 256) // (P * (P + 1) // 2)
            ins = [torch.full(((r + 1) * rows, 256), float(r), device="cuda") for r in range(P)]
            total = sum(t.numel() for t in ins) * 4
            blocks = min(blocks, 48)
            ms = timed(lambda: g.allgatherv(ins, [0] * P, blocks=blocks), a.iters)
            nbytes = total + P * total      # every slab read once, written into P outputs
            out.update(ms=ms, bytes=nbytes, gbs=nbytes / ms / 1e6, blocks=blocks, ok=bool(g.status == 0))
        g.close()
    out["hbm_peak_gbs"] = hbm
    out["frac_of_hbm_copy_" + src] = out["gbs"] / hbm
    print(json.dumps(out))


if __name__ == "__main__":
    main()
