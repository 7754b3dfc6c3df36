"""Headline benchmark: DeepSpeech2-style data-parallel training throughput (samples/s).

    python bench.py --gpus N --steps K --warmup W            (N > 1: started by torchrun, one rank per GPU)

Configuration: log-spectrograms 161 x 700 from N(0,1), batch 32 per GPU, two conv layers + BN +
clipped ReLU, 5 bidirectional GRU layers of 1024, FC to 29 classes, CTC loss on 100 random labels
per utterance, fp32 parameters with TF32 math, momentum-SGD lr 3e-4 whose update is fused into the
gradient allreduce kernel of this library. Synthetic data, random-initialised weights.

Prints ONE JSON line (rank 0). `value` is the whole-job samples/s over the K timed steps, timed
with CUDA events between barriers, maximum over ranks. `e2e` repeats the measurement through the
public API with the per-step host->device copy of the inputs from pinned memory (on a copy stream,
issued one step ahead so that it overlaps the previous step's compute; K + 1 copies for K steps,
all inside the timed region) and the device->host read of the loss inside the timed region.

After its own numbers an `--impl ours` run measures, in the same process and with the same steps
and warm-up, torch DistributedDataParallel + NCCL + the plain torch optimizer on the same model:
once with the same model kernels (`ddp_nccl_same_kernels`: the persistent GRU and the fused batch
norm, which isolates what the collectives library is worth) and once with the stock model
(`ddp_nccl_cudnn`: cuDNN's GRU and batch norm). They go under `comparators` and are
labelled as what they are: not the reference. `--no-comparators` skips them.

Other arms: `--impl reference` reports the reference's own build (unavailable on this image);
`--impl ddp` runs only the torch DDP comparator. `--model gpt2|resnet50` run the other two
data-parallel configurations.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "ddp"])
    ap.add_argument("--model", default="ds2", choices=["ds2", "gpt2", "resnet50"])
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (0 = the configuration's value)")
    ap.add_argument("--rnn", default="auto", choices=["auto", "persistent", "cudnn"],
                    help="ds2: GRU stack and batch norm on the library's kernels (auto: ours yes, ddp no) or the stock cuDNN model")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-comparators", action="store_true",
                    help="skip the torch DDP + NCCL arms that an `--impl ours` run measures after its own numbers")
    return ap.parse_args()


def reference_unavailable():
    if int(os.environ.get("RANK", "0")) != 0:      # under torchrun every rank runs this; one line is enough
        return 0
    print(json.dumps({
        "impl": "reference",
        "unavailable": "the reference is a TensorFlow 1.3 fork: pip reports that its tree is not installable "
                       "(neither setup.py nor pyproject.toml); its build needs Bazel, an MPI install and CUDA 8/cuDNN 6, none present offline",
    }))
    return 0


def build_model(name: str, device, batch: int, persistent_rnn: bool = True, fused_norm: bool = True):
    import torch

    if name == "ds2":
        from tensorflow_allreduce_b200.models import ds2

        cfg = ds2.DS2Config(persistent_rnn=persistent_rnn, fused_norm=fused_norm)
        model = ds2.DeepSpeech2(cfg).to(device)
        model.rnn.flatten_parameters()
        b = batch or 32

        def make(pin):
            return ds2.synthetic_batch(cfg, b, device, pin=pin)

        def loss_fn(fwd, batch_):
            import torch.nn.functional as F

            spect, labels, lens = batch_
            logp = fwd(spect)
            t, nb, _ = logp.shape
            in_len = torch.full((nb,), t, dtype=torch.long, device=logp.device)
            return F.ctc_loss(logp, labels, in_len, lens, blank=0, reduction="mean", zero_infinity=True)

        meta = {"model": "deepspeech2-style (2 conv + 5 biGRU-1024 + FC-29 + CTC)", "seq_len": cfg.n_frames, "dtype": "tf32",
                "optimizer": "momentum-SGD lr 3e-4 momentum 0.9"}
        opt = torch.optim.SGD(model.parameters(), lr=3e-4, momentum=0.9)
        return model, opt, make, loss_fn, b, meta
    if name == "gpt2":
        from tensorflow_allreduce_b200.models import gpt2

        cfg = gpt2.GPT2Config()
        model = gpt2.GPT2(cfg).to(device).to(torch.bfloat16)
        b = batch or 8

        def make(pin):
            return gpt2.synthetic_batch(cfg, b, device, pin=pin)

        def loss_fn(fwd, batch_):
            import torch.nn.functional as F

            (idx,) = batch_
            logits = fwd(idx[:, :-1])
            return F.cross_entropy(logits.float().view(-1, logits.size(-1)), idx[:, 1:].reshape(-1))

        meta = {"model": "gpt2-medium (24L d1024 h16 ffn4096 vocab50257)", "seq_len": cfg.seq_len, "dtype": "bf16",
                "optimizer": "AdamW lr 1e-4 wd 0.01 (fp32 master weights)"}
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
        return model, opt, make, loss_fn, b, meta
    from tensorflow_allreduce_b200.models import resnet50

    model = resnet50.ResNet50().to(device).to(torch.bfloat16).to(memory_format=torch.channels_last)
    b = batch or 256

    def make(pin):
        return resnet50.synthetic_batch(b, device, pin=pin)

    def loss_fn(fwd, batch_):
        import torch.nn.functional as F

        x, y = batch_
        if x.dim() == 4 and not x.is_contiguous(memory_format=torch.channels_last):
            x = x.contiguous(memory_format=torch.channels_last)
        return F.cross_entropy(fwd(x).float(), y)

    meta = {"model": "resnet50", "seq_len": 224, "dtype": "bf16", "optimizer": "momentum-SGD lr 0.1 momentum 0.9 wd 1e-4"}
    opt = torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9, weight_decay=1e-4)
    return model, opt, make, loss_fn, b, meta


# Recorded same-box comparators (torch DDP + NCCL + torch.optim.SGD + cuDNN GRU on the DeepSpeech2-style
# configuration, samples/s by number of GPUs, on this pool's B200 boxes). They are NOT the reference's own build,
# which cannot be installed on this image; they are the only recorded figures that `vs_baseline` can be taken against.
RECORDED_DS2_DDP_CUDNN = {1: 376.1, 2: 698.6, 4: 1285.4}


def run_arm(a, impl: str, rnn: str, device, rank: int, world: int, local: int, with_e2e: bool):
    """Build the model and its optimizer for one arm, run warm-up and the timed steps, and return the
    measurements. `impl`: "ours" (DistributedOptimizer of this library) or "ddp" (torch DistributedDataParallel over
    NCCL with the plain torch optimizer; a single process without DDP when world == 1)."""
    import torch

    import tensorflow_allreduce_b200 as bc
    from tensorflow_allreduce_b200.ops import persistent_gru
    from tensorflow_allreduce_b200.utils.clocks import ClockSampler

    torch.manual_seed(1234)          # same initial weights on every rank, as the reference requires
    persistent = rnn == "persistent"
    # "cudnn" is the stock model: cuDNN's GRU and cuDNN's batch norm + a separate clipped ReLU
    model, base_opt, make, loss_fn, per_gpu_batch, meta = build_model(a.model, device, a.batch, persistent, fused_norm=persistent)
    ddp = None
    fwd = model
    if impl == "ddp":
        import torch.distributed as dist
        from torch.nn.parallel import DistributedDataParallel

        if world > 1:
            if not dist.is_initialized():
                dist.init_process_group("nccl", device_id=device)
            ddp = DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True)
            fwd = ddp
        opt = base_opt
    else:
        opt = bc.DistributedOptimizer(base_opt)

    torch.manual_seed(100 + rank)
    dev_batch = make(False)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)   # > 126 MB L2

    def step(batch_):
        flush.zero_()
        opt.zero_grad()
        loss = loss_fn(fwd, batch_)
        loss.backward()
        opt.step()
        return loss

    def max_over_ranks(x):
        return max(bc.host_allgather(float(x)))

    for _ in range(a.warmup):
        step(dev_batch)
    torch.cuda.synchronize()
    from tensorflow_allreduce_b200.ops import bn_clip

    def own_launches():
        # kernels of this library launched so far: bucket reductions / fused updates, persistent GRU layers, fused batch norms
        return getattr(opt, "launch_count", 0) + persistent_gru.launch_count + 2 * bn_clip.launch_count

    launches0 = own_launches()
    bc.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        torch.cuda.synchronize()
        e0.record()
        for _ in range(a.steps):
            loss = step(dev_batch)
        e1.record()
        torch.cuda.synchronize()
    bc.barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    launches = own_launches() - launches0
    persistent_gru.check_status()
    bc.check_device_status()
    res = {
        "impl": impl, "rnn": rnn, "ms": ms, "per_gpu_batch": per_gpu_batch, "meta": meta, "launches": launches,
        "value": world * per_gpu_batch * a.steps / (ms / 1e3), "final_loss": float(loss.detach()), "clocks": clk.summary(),
        "n_params": sum(p.numel() for p in model.parameters()), "grad_buckets": len(getattr(opt, "buckets", [])),
        "fused": bool(getattr(opt, "fused", False)), "e2e": None,
    }
    if with_e2e:
        pinned = make(True)
        h2d = sum(t.numel() * t.element_size() for t in pinned)
        loss_host = 0.0
        copy_stream = torch.cuda.Stream(device)

        def fetch():
            # host -> device copy of one step's inputs from pinned memory, on a stream of its own
            with torch.cuda.stream(copy_stream):
                b_ = tuple(t.to(device, non_blocking=True) for t in pinned)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
            return b_, ev

        for _ in range(2):
            b_, ev = fetch()
            torch.cuda.current_stream().wait_event(ev)
            step(b_)
        torch.cuda.synchronize()
        bc.barrier()
        t0 = time.perf_counter()
        nxt = fetch()
        for _ in range(a.steps):
            batch_, ev = nxt
            torch.cuda.current_stream().wait_event(ev)
            for t in batch_:                          # allocated on the copy stream, read on this one
                t.record_stream(torch.cuda.current_stream())
            loss = step(batch_)
            nxt = fetch()                            # the next step's inputs travel while this step computes
            loss_host = loss.item()                  # device -> host read of the step's result
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        del nxt
        bc.barrier()
        e2e_s = max_over_ranks(t1 - t0)
        res["e2e"] = {"value": round(world * per_gpu_batch * a.steps / e2e_s, 3), "unit": "samples/s", "h2d_bytes_per_step": h2d,
                      "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_s * 1e3 / a.steps, 3), "last_loss": loss_host}
    # free this arm's memory before the next one
    del opt, fwd, ddp, model, base_opt, dev_batch, flush
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    return res


def main():
    a = parse()
    if a.impl == "reference":
        return reference_unavailable()

    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            # convenience: start the ranks ourselves when not launched by torchrun
            from tensorflow_allreduce_b200 import launch
            return launch.main(["--nproc", str(a.gpus), os.path.abspath(__file__)] + sys.argv[1:])
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.benchmark = True

    import tensorflow_allreduce_b200 as bc

    bc.init(device=local)
    persistent = a.rnn == "persistent" or (a.rnn == "auto" and a.impl == "ours")
    main_rnn = ("persistent" if persistent else "cudnn") if a.model == "ds2" else "none"
    r = run_arm(a, a.impl, main_rnn, device, rank, world, local, with_e2e=not a.no_e2e)

    # Comparators in the same process, on the same model, with the same steps and warm-up. They are torch's own
    # data-parallel stack (DDP over NCCL, torch.optim), not the reference: its build is unavailable here.
    comps = None
    if a.impl == "ours" and not a.no_comparators:
        comps = {"note": "same-box comparators measured in this invocation; torch DDP + NCCL + torch.optim, NOT the reference"}
        arms = [("ddp_nccl_same_kernels", "persistent"), ("ddp_nccl_cudnn", "cudnn")] if a.model == "ds2" else [("ddp_nccl", "none")]
        if a.model == "ds2" and main_rnn != "persistent":
            arms = [("ddp_nccl_cudnn", "cudnn")]
        for key, rnn in arms:
            c = run_arm(a, "ddp", rnn, device, rank, world, local, with_e2e=not a.no_e2e)
            comps[key] = {"value": round(c["value"], 3), "ms_per_step": round(c["ms"] / a.steps, 3),
                          "e2e": c["e2e"]["value"] if c["e2e"] else None}
        same = comps.get("ddp_nccl_same_kernels") or comps.get("ddp_nccl")
        if same:
            comps["ratio_same_kernels"] = round(r["value"] / same["value"], 4)
            if r["e2e"] and same["e2e"]:
                comps["e2e_ratio_same_kernels"] = round(r["e2e"]["value"] / same["e2e"], 4)
        if "ddp_nccl_cudnn" in comps:
            comps["ratio_cudnn"] = round(r["value"] / comps["ddp_nccl_cudnn"]["value"], 4)

    if rank == 0:
        meta, clocks, ms = r["meta"], r["clocks"], r["ms"]
        base = RECORDED_DS2_DDP_CUDNN.get(world) if (a.model == "ds2" and not a.batch) else None
        out = {
            "metric": f"{a.model}_train_samples_per_sec",
            "value": round(r["value"], 3),
            "unit": "samples/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": round(ms / a.steps, 3),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": round(r["value"] / base, 4) if base else None,
            "vs_baseline_of": ("torch DDP + NCCL + torch.optim.SGD + cuDNN GRU recorded earlier on the same B200 boxes; "
                               "the reference publishes no number and its own build is unavailable") if base else None,
            "dtype": meta["dtype"], "data": "synthetic (random inputs and labels, random-init weights)",
            "impl": a.impl,
            "config": {"model": meta["model"], "global_batch": world * r["per_gpu_batch"], "seq_len": meta["seq_len"],
                       "parallelism": f"dp{world}", "optimizer": meta["optimizer"], "params_m": round(r["n_params"] / 1e6, 2),
                       "l2": "256 MB buffer written between steps (L2 flush); working set exceeds L2 anyway",
                       "grad_buckets": r["grad_buckets"], "fused_update": r["fused"],
                       "rnn": ("persistent tcgen05 kernels" if persistent else "cudnn") if a.model == "ds2" else None,
                       "norm": ("fused batch norm + clipped ReLU kernels" if persistent else "cudnn") if a.model == "ds2" else None},
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons", []),
                       "power_w_max": clocks.get("power_w_max"), "samples": clocks.get("samples"), "source": clocks.get("source")},
            "gpu_launches": r["launches"],
            "final_loss": r["final_loss"],
        }
        if r["e2e"] is not None:
            out["e2e"] = r["e2e"]
        if comps is not None:
            out["comparators"] = comps
        print(json.dumps(out), flush=True)
    import torch.distributed as dist

    if dist.is_initialized():
        dist.destroy_process_group()
    bc.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
