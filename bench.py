"""Headline benchmark: DeepSpeech2-style data-parallel training throughput (samples/s).

    python bench.py --gpus N --steps K --warmup W            (N > 1: started by torchrun, one rank per GPU)

Configuration: log-spectrograms 161 x 700 from N(0,1), batch 32 per GPU, two conv layers + BN +
clipped ReLU, 5 bidirectional GRU layers of 1024, FC to 29 classes, CTC loss on 100 random labels
per utterance, fp32 parameters with TF32 math, momentum-SGD lr 3e-4 whose update is fused into the
gradient allreduce kernel of this library. Synthetic data, random-initialised weights.

Prints ONE JSON line (rank 0). `value` is the whole-job samples/s over the K timed steps, timed
with CUDA events between barriers, maximum over ranks. `e2e` repeats the measurement through the
public API with the per-step host->device copy of the inputs from pinned memory and the
device->host read of the loss inside the timed region.

Other arms: `--impl reference` reports the reference's own build (unavailable on this image);
`--impl ddp` runs torch DistributedDataParallel + NCCL + torch.optim.SGD on the same model as a
same-box comparator. `--model gpt2|resnet50` run the other two data-parallel configurations.
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
                    help="ds2: GRU stack on the library's persistent tcgen05 kernels (auto: ours yes, ddp no) or on cuDNN")
    ap.add_argument("--no-e2e", action="store_true")
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


def build_model(name: str, device, batch: int, persistent_rnn: bool = True):
    import torch

    if name == "ds2":
        from tensorflow_allreduce_b200.models import ds2

        cfg = ds2.DS2Config(persistent_rnn=persistent_rnn)
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
    torch.manual_seed(1234)          # same initial weights on every rank, as the reference requires

    import tensorflow_allreduce_b200 as bc
    from tensorflow_allreduce_b200.utils.clocks import ClockSampler

    bc.init(device=local)
    persistent = a.rnn == "persistent" or (a.rnn == "auto" and a.impl == "ours")
    model, base_opt, make, loss_fn, per_gpu_batch, meta = build_model(a.model, device, a.batch, persistent)
    from tensorflow_allreduce_b200.ops import persistent_gru

    ddp = None
    fwd = model
    if a.impl == "ddp":
        import torch.distributed as dist
        from torch.nn.parallel import DistributedDataParallel

        if world > 1:
            dist.init_process_group("nccl", device_id=device)
            ddp = DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True)
            fwd = ddp
        opt = base_opt
    else:
        opt = bc.DistributedOptimizer(base_opt)

    def loss_call(batch_):
        return loss_fn(fwd, batch_)

    torch.manual_seed(100 + rank)
    dev_batch = make(False)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)   # > 126 MB L2

    def step(batch_):
        flush.zero_()
        opt.zero_grad()
        loss = loss_call(batch_)
        loss.backward()
        opt.step()
        return loss

    def max_over_ranks(x):
        return max(bc.host_allgather(float(x)))

    for _ in range(a.warmup):
        step(dev_batch)
    torch.cuda.synchronize()
    launches0 = getattr(opt, "launch_count", 0) + persistent_gru.launch_count
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
    launches = getattr(opt, "launch_count", 0) + persistent_gru.launch_count - launches0
    persistent_gru.check_status()
    final_loss = float(loss.detach())
    clocks = clk.summary()
    bc.check_device_status()

    e2e = None
    if not a.no_e2e:
        pinned = make(True)
        h2d = sum(t.numel() * t.element_size() for t in pinned)
        loss_host = 0.0
        for _ in range(2):
            step(tuple(t.to(device, non_blocking=True) for t in pinned))
        torch.cuda.synchronize()
        bc.barrier()
        t0 = time.perf_counter()
        for _ in range(a.steps):
            batch_ = tuple(t.to(device, non_blocking=True) for t in pinned)
            loss_host = step(batch_).item()          # device -> host read of the step's result
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        bc.barrier()
        e2e_s = max_over_ranks(t1 - t0)
        e2e = {"value": round(world * per_gpu_batch * a.steps / e2e_s, 3), "unit": "samples/s", "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_s * 1e3 / a.steps, 3), "last_loss": loss_host}

    if rank == 0:
        n_params = sum(p.numel() for p in model.parameters())
        out = {
            "metric": f"{a.model}_train_samples_per_sec",
            "value": round(world * per_gpu_batch * a.steps / (ms / 1e3), 3),
            "unit": "samples/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup,
            "ms_per_step": round(ms / a.steps, 3),
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,
            "dtype": meta["dtype"], "data": "synthetic (random inputs and labels, random-init weights)",
            "impl": a.impl,
            "config": {"model": meta["model"], "global_batch": world * per_gpu_batch, "seq_len": meta["seq_len"],
                       "parallelism": f"dp{world}", "optimizer": meta["optimizer"], "params_m": round(n_params / 1e6, 2),
                       "l2": "256 MB buffer written between steps (L2 flush); working set exceeds L2 anyway",
                       "grad_buckets": len(getattr(opt, "buckets", [])), "fused_update": bool(getattr(opt, "fused", False)),
                       "rnn": ("persistent tcgen05 kernels" if persistent else "cudnn") if a.model == "ds2" else None},
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons", []),
                       "power_w_max": clocks.get("power_w_max"), "samples": clocks.get("samples"), "source": clocks.get("source")},
            "gpu_launches": launches,
            "final_loss": final_loss,
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out), flush=True)
    if ddp is not None:
        import torch.distributed as dist
        dist.destroy_process_group()
    bc.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
