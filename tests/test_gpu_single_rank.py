"""The full stack on one GPU with a group of size 1: runtime, symmetric memory, negotiated
collectives, and DistributedOptimizer (fused and generic) against torch.optim."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def group():
    import tensorflow_allreduce_b200 as bc

    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        import os
        os.environ.pop(k, None)
    bc.init(device=0)
    yield bc
    bc.shutdown()


def test_group_basics(group):
    bc = group
    assert (bc.rank(), bc.size(), bc.local_rank()) == (0, 1, 0)
    assert bc.on_gpu()
    from tensorflow_allreduce_b200.ops import symmetric
    assert symmetric.describe() in ("vmm", "vmm+multicast", "ipc")


def test_allreduce_allgather_cuda(group):
    bc = group
    for dtype in (torch.float32, torch.bfloat16, torch.int32, torch.int64):
        x = (torch.arange(1000, device="cuda") % 13).to(dtype)
        assert torch.equal(bc.allreduce(x, average=False), x)
        assert torch.equal(bc.allreduce(x, average=True), x)
    x = torch.randn(33, 7, device="cuda")
    g = bc.allgather(x)
    assert torch.equal(g, x)
    from tensorflow_allreduce_b200.ops import symmetric
    assert symmetric.is_symmetric(g)          # gathered straight into the symmetric heap
    y = x[1:]                                  # misaligned view
    assert torch.equal(bc.allreduce(y, average=False), y)
    s = symmetric.empty((1024,), torch.float32)
    s.fill_(3.0)
    bc.allreduce_(s, average=True)
    assert float(s.sum()) == 3.0 * 1024
    # CPU tensors are accepted by a CUDA group too
    c = torch.arange(5.)
    assert torch.equal(bc.allreduce(c), c)
    assert any(e["device"] == 1 for e in bc.stats())


def _mlp(dtype=torch.float32):
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(37, 64), torch.nn.ReLU(), torch.nn.Linear(64, 64), torch.nn.Tanh(),
                            torch.nn.Linear(64, 5)).cuda().to(dtype)
    return m


@pytest.mark.parametrize("opt_name", ["sgd", "sgd_mom", "sgd_nesterov", "adam", "adamw"])
def test_fused_optimizer_matches_torch(group, opt_name):
    bc = group
    mk = {
        "sgd": lambda ps: torch.optim.SGD(ps, lr=0.05),
        "sgd_mom": lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, weight_decay=1e-3),
        "sgd_nesterov": lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, nesterov=True, dampening=0.0),
        "adam": lambda ps: torch.optim.Adam(ps, lr=1e-2, weight_decay=1e-2),
        "adamw": lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=1e-1),
    }[opt_name]
    ref = _mlp()
    mine = copy.deepcopy(ref)
    o_ref = mk(ref.parameters())
    o_mine = bc.DistributedOptimizer(mk(mine.parameters()), bucket_mb=0.01)
    assert o_mine.fused and len(o_mine.buckets) > 1
    torch.manual_seed(1)
    for it in range(5):
        x = torch.randn(16, 37, device="cuda")
        y = torch.randn(16, 5, device="cuda")
        for m, o in ((ref, o_ref), (mine, o_mine)):
            o.zero_grad()
            torch.nn.functional.mse_loss(m(x), y).backward()
            o.step()
    for a, b in zip(ref.parameters(), mine.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=5e-6)
    # optimizer state is visible under torch's keys and survives a state_dict round trip
    sd = o_mine.state_dict()
    sd_ref = o_ref.state_dict()
    assert set(sd["state"].keys()) == set(sd_ref["state"].keys()) or opt_name == "sgd"
    for k, st in sd_ref["state"].items():
        for kk, vv in st.items():
            if isinstance(vv, torch.Tensor) and vv.dim() > 0:
                torch.testing.assert_close(sd["state"][k][kk], vv, rtol=1e-5, atol=1e-6)
            elif kk == "step":
                assert float(sd["state"][k][kk]) == float(vv)
    o_mine.load_state_dict(copy.deepcopy(sd))
    o_ref.load_state_dict(copy.deepcopy(sd_ref))
    x = torch.randn(16, 37, device="cuda")
    y = torch.randn(16, 5, device="cuda")
    for m, o in ((ref, o_ref), (mine, o_mine)):
        o.zero_grad()
        torch.nn.functional.mse_loss(m(x), y).backward()
        o.step()
    for a, b in zip(ref.parameters(), mine.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=5e-6)


def test_generic_optimizer_path(group):
    bc = group
    ref = _mlp()
    mine = copy.deepcopy(ref)
    o_ref = torch.optim.RMSprop(ref.parameters(), lr=1e-3)
    o_mine = bc.DistributedOptimizer(torch.optim.RMSprop(mine.parameters(), lr=1e-3))
    assert not o_mine.fused
    sched = torch.optim.lr_scheduler.StepLR(o_mine, step_size=2, gamma=0.5)   # wrapper is a real Optimizer
    sched_ref = torch.optim.lr_scheduler.StepLR(o_ref, step_size=2, gamma=0.5)
    for it in range(4):
        x = torch.randn(8, 37, device="cuda")
        y = torch.randn(8, 5, device="cuda")
        for m, o, s in ((ref, o_ref, sched_ref), (mine, o_mine, sched)):
            o.zero_grad()
            torch.nn.functional.mse_loss(m(x), y).backward()
            o.step()
            s.step()
    for a, b in zip(ref.parameters(), mine.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=5e-6)


def test_bf16_master_weights(group):
    bc = group
    ref = _mlp()                      # fp32 reference of the master weights
    mine = _mlp(torch.bfloat16)
    with torch.no_grad():
        for a, b in zip(ref.parameters(), mine.parameters()):
            a.copy_(b.float())
    o_ref = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.1)
    # gradients are read back below, so neither overlap with backward nor in-kernel zeroing here
    o_mine = bc.DistributedOptimizer(torch.optim.AdamW(mine.parameters(), lr=1e-2, weight_decay=0.1), fused_zero_grad=False)
    for it in range(3):
        x = torch.randn(16, 37, device="cuda")
        y = torch.randn(16, 5, device="cuda")
        o_mine.zero_grad()
        with o_mine.no_sync():
            torch.nn.functional.mse_loss(mine(x.bfloat16()).float(), y).backward()
        # feed the reference the same (bf16-rounded) gradients
        grads = [p.grad.float().clone() for p in mine.parameters()]
        o_mine.step()
        for p, gr in zip(ref.parameters(), grads):
            p.grad = gr
        o_ref.step()
    for a, b in zip(ref.parameters(), mine.parameters()):
        assert torch.equal(a.to(torch.bfloat16), b) or torch.allclose(a, b.float(), rtol=1e-2, atol=1e-2)


def test_cudnn_rnn_weights_stay_flat(group):
    # nn.GRU keeps its weights in one cuDNN-ordered buffer; the bucket builder must preserve the
    # relative layout, otherwise every forward re-packs the weights (and warns).
    import warnings

    bc = group
    torch.manual_seed(0)
    gru = torch.nn.GRU(8, 16, num_layers=2, bidirectional=True).cuda()
    gru.flatten_parameters()
    opt = bc.DistributedOptimizer(torch.optim.SGD(gru.parameters(), lr=0.1, momentum=0.9))
    x = torch.randn(5, 3, 8, device="cuda")
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        for _ in range(2):
            out, _ = gru(x)
            out.sum().backward()
            opt.step()
    assert torch.isfinite(out).all()


def test_flattened_rnn_weights_split_into_buckets_match_torch(group):
    # The flat cuDNN weight buffer is cut into several launch ranges; a reference GRU with
    # separate weights and plain torch SGD must see the same parameters after a few steps, and
    # the module must still own one flat buffer (no re-packing warning).
    import warnings

    bc = group
    torch.manual_seed(0)
    ref = torch.nn.GRU(24, 32, num_layers=3, bidirectional=True).cuda()
    mine = copy.deepcopy(ref)
    mine.flatten_parameters()
    o_ref = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3)
    o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3), bucket_mb=0.02)
    assert o_mine.fused and len(o_mine.buckets) >= 4, o_mine.buckets
    covered = [p for ps in o_mine.bucket_parameters for p in ps]
    assert len(covered) == len(list(mine.parameters())) == len({id(p) for p in covered})
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        for it in range(4):
            x = torch.randn(6, 5, 24, device="cuda")
            for m, o in ((ref, o_ref), (mine, o_mine)):
                o.zero_grad()
                m(x)[0].square().mean().backward()
                o.step()
    for a, b in zip(ref.parameters(), mine.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=5e-6)
    storages = {p.untyped_storage().data_ptr() for p in mine.parameters()}
    assert len(storages) == 1


def test_restored_momentum_is_continued_with_dampening(group):
    # With dampening torch seeds a NEW momentum buffer with the gradient itself; a buffer that
    # comes from a state dict must be continued with the recurrence instead.
    bc = group
    mk = lambda ps: torch.optim.SGD(ps, lr=0.05, momentum=0.9, dampening=0.5)
    ref = _mlp()
    mine = copy.deepcopy(ref)
    o_ref = mk(ref.parameters())
    o_mine = bc.DistributedOptimizer(mk(mine.parameters()))
    torch.manual_seed(3)
    data = [(torch.randn(16, 37, device="cuda"), torch.randn(16, 5, device="cuda")) for _ in range(4)]
    for x, y in data[:2]:
        for m, o in ((ref, o_ref), (mine, o_mine)):
            o.zero_grad()
            torch.nn.functional.mse_loss(m(x), y).backward()
            o.step()
    # a fresh wrapper around a fresh optimizer, restored from the state dict
    sd = copy.deepcopy(o_mine.state_dict())
    again = copy.deepcopy(mine)
    o_again = bc.DistributedOptimizer(mk(again.parameters()))
    o_again.load_state_dict(sd)
    for x, y in data[2:]:
        for m, o in ((ref, o_ref), (again, o_again)):
            o.zero_grad()
            torch.nn.functional.mse_loss(m(x), y).backward()
            o.step()
    for a, b in zip(ref.parameters(), again.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=5e-6)


def test_device_time_of_every_bucket_in_sampled_steps(group):
    # timing_every=2: in steps 0 and 2 every bucket launch is bracketed by CUDA events; stats()
    # then holds one record per bucket and sampled step with the time on the device.
    bc = group
    model = _mlp()
    opt = bc.DistributedOptimizer(torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9), bucket_mb=0.01, timing_every=2)
    nb = len(opt.buckets)
    assert nb > 1
    torch.cuda.synchronize()
    bc.clear_stats()
    for it in range(3):
        x = torch.randn(16, 37, device="cuda")
        y = torch.randn(16, 5, device="cuda")
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(x), y).backward()
        opt.step()
    torch.cuda.synchronize()
    recs = [e for e in bc.stats() if e["name"] == "fused_step"]
    assert len(recs) == 2 * nb, (len(recs), nb)
    assert all(e["device_us"] > 0 and e["channel"] == 1 and e["bytes"] > 0 and e["blocks"] >= 1 for e in recs)
    assert sorted(e["bytes"] for e in recs[:nb]) == sorted(n * 4 for _, n in opt.buckets)
    # the switch also covers the other ordered launches and the negotiated GPU allreduce
    from tensorflow_allreduce_b200.ops import symmetric
    from tensorflow_allreduce_b200.ops.direct import allreduce_direct_

    bc.clear_stats()
    bc.set_device_timing(True)
    s = symmetric.empty((1 << 16,), torch.float32)
    s.fill_(1.0)
    allreduce_direct_(s, average=True)
    bc.allreduce(torch.ones(1 << 16, device="cuda"), name="timed.negotiated")
    bc.set_device_timing(False)
    bc.allreduce(torch.ones(1 << 16, device="cuda"), name="untimed")
    torch.cuda.synchronize()
    by_name = {e["name"]: e for e in bc.stats()}
    assert by_name["allreduce_direct"]["device_us"] >= 0 and by_name["timed.negotiated"]["device_us"] > 0
    assert "device_us" not in by_name["untimed"]
    from tensorflow_allreduce_b200.utils import timeline
    assert any(e["cat"] == "allreduce.device" for e in timeline.chrome_trace())
