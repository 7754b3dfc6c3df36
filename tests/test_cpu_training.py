"""CPU groups: the parameter / optimizer-state broadcast helpers, the gradient-averaging optimizer
wrapper against a single-process large-batch run (the reference's `DistributedOptimizer`,
tensorflow/contrib/mpi_collectives/__init__.py:167-234, has no test of its own), and the
benchmark models' CPU paths."""
import torch

from _util import run


def test_broadcast_parameters_and_optimizer_state():
    res = run("""
    bc.init(device="cpu")
    torch.manual_seed(100 + RANK)                      # every rank starts differently
    model = torch.nn.Sequential(torch.nn.Linear(7, 5), torch.nn.BatchNorm1d(5), torch.nn.Linear(5, 3))
    opt = torch.optim.Adam(model.parameters(), lr=1e-2 * (RANK + 1))
    for _ in range(2):
        opt.zero_grad(); model(torch.randn(4, 7)).sum().backward(); opt.step()
    bc.broadcast_parameters(model, root=1)
    bc.broadcast_optimizer_state(opt, root=1)
    flat = torch.cat([t.reshape(-1).double() for t in model.state_dict().values()])
    st = opt.state_dict()
    sflat = torch.cat([v.reshape(-1).double() for s in st["state"].values() for v in s.values() if isinstance(v, torch.Tensor)])
    allp = bc.allgather(flat.unsqueeze(0)); alls = bc.allgather(sflat.unsqueeze(0))
    emit(same_p=bool((allp == allp[1:2]).all()), same_s=bool((alls == alls[1:2]).all()), lr=st["param_groups"][0]["lr"],
         nb=int(model[1].num_batches_tracked))
    bc.shutdown()
    """, nranks=3)
    for _, rec in res:
        assert rec["same_p"] and rec["same_s"]
        assert abs(rec["lr"] - 2e-2) < 1e-12 and rec["nb"] == 2


def test_distributed_optimizer_cpu_equals_large_batch_and_round_trips_state():
    res = run("""
    bc.init(device="cpu")
    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))
    mine, ref = make(), make()
    o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.05, momentum=0.9))
    o_ref = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    g = torch.Generator().manual_seed(5)
    X = torch.randn(4, 8 * SIZE, 16, generator=g); Y = torch.randn(4, 8 * SIZE, 4, generator=g)
    for it in range(4):
        o_ref.zero_grad(); torch.nn.functional.mse_loss(ref(X[it]), Y[it]).backward(); o_ref.step()
        sl = slice(RANK * 8, (RANK + 1) * 8)
        o_mine.zero_grad(); torch.nn.functional.mse_loss(mine(X[it][sl]), Y[it][sl]).backward(); o_mine.step()
        if it == 1:
            saved = o_mine.state_dict()
            o_mine.load_state_dict(saved)               # round trip in the middle of training
    worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
    emit(worst=worst, name=o_mine.name, fused=o_mine.fused, keys=sorted(o_mine.state_dict().keys()))
    bc.shutdown()
    """, nranks=2)
    for _, rec in res:
        assert rec["worst"] < 1e-6
        assert rec["name"] == "DistributedSGD" and not rec["fused"]
        assert rec["keys"] == ["param_groups", "state"]


CLIP = """
bc.init(%s)
DEV = "%s"
def make():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4)).to(DEV)
mine, ref = make(), make()
o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.5, momentum=0.9), fused=False)
o_ref = torch.optim.SGD(ref.parameters(), lr=0.5, momentum=0.9)
g = torch.Generator().manual_seed(5)
X = (torch.randn(4, 8 * SIZE, 16, generator=g) * 3).to(DEV); Y = (torch.randn(4, 8 * SIZE, 4, generator=g) * 3).to(DEV)
norms = []
for it in range(4):
    o_ref.zero_grad(); torch.nn.functional.mse_loss(ref(X[it]), Y[it]).backward()
    torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.1); o_ref.step()
    sl = slice(RANK * 8, (RANK + 1) * 8)
    o_mine.zero_grad(); torch.nn.functional.mse_loss(mine(X[it][sl]), Y[it][sl]).backward()
    o_mine.synchronize()                                   # p.grad now holds the average over the ranks
    norms.append(float(torch.nn.utils.clip_grad_norm_(mine.parameters(), 0.1)))
    o_mine.step()
worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
fused_refuses = False
try:
    bc.DistributedOptimizer(torch.optim.SGD(make().parameters(), lr=0.1)).synchronize()
except RuntimeError:
    fused_refuses = True
emit(worst=worst, clipped=all(n > 0.1 for n in norms), fused_refuses=fused_refuses)
bc.shutdown()
"""


def test_synchronize_allows_clipping_before_step():
    res = run(CLIP % ('device="cpu"', "cpu"), nranks=2)
    for _, rec in res:
        assert rec["worst"] < 1e-6 and rec["clipped"]


def test_models_run_on_cpu():
    from tensorflow_allreduce_b200.models import ds2, gpt2
    from tensorflow_allreduce_b200.ops import persistent_gru

    assert not persistent_gru.supported(10, 4, 128, 2, "cpu") or torch.cuda.is_available()
    cfg = ds2.DS2Config(n_frames=32, rnn_hidden=16, rnn_layers=1, label_len=3)
    m = ds2.DeepSpeech2(cfg)
    loss = m.loss(*ds2.synthetic_batch(cfg, 2, "cpu"))
    loss.backward()
    assert torch.isfinite(loss)
    gcfg = gpt2.GPT2Config(n_layer=1, d_model=32, n_head=2, d_ff=64, vocab=101, seq_len=16)
    g = gpt2.GPT2(gcfg)
    loss = g.loss(*gpt2.synthetic_batch(gcfg, 2, "cpu"))
    loss.backward()
    assert torch.isfinite(loss)


def test_minimize_and_compute_apply_gradients():
    # The reference's spelling of a step: opt.minimize(loss), or compute_gradients -> (edit) ->
    # apply_gradients (mpi_collectives/__init__.py:195-236). Both equal the large-batch run.
    res = run("""
    bc.init(device="cpu")
    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 2))
    mine, ref = make(), make()
    o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.1, momentum=0.9))
    o_ref = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(3)
    X = torch.randn(4, 6 * SIZE, 8, generator=g); Y = torch.randn(4, 6 * SIZE, 2, generator=g)
    sl = slice(RANK * 6, (RANK + 1) * 6)
    grads_match = True
    for it in range(4):
        o_ref.zero_grad(); torch.nn.functional.mse_loss(ref(X[it]), Y[it]).backward()
        if it % 2 == 0:
            o_ref.step()
            o_mine.minimize(torch.nn.functional.mse_loss(mine(X[it][sl]), Y[it][sl]))
        else:
            pairs = o_mine.compute_gradients(torch.nn.functional.mse_loss(mine(X[it][sl]), Y[it][sl]))
            for (gr, p), q in zip(pairs, ref.parameters()):
                grads_match = grads_match and torch.allclose(gr, q.grad, atol=1e-6)
                gr.mul_(0.5); q.grad.mul_(0.5)                 # edit the averaged gradients before the update
            o_ref.step()
            o_mine.apply_gradients(pairs)
    worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
    try:
        o_mine.apply_gradients([(torch.zeros(1), next(mine.parameters()))])
        refused = False
    except ValueError:
        refused = True
    emit(worst=worst, grads_match=bool(grads_match), refused=refused)
    bc.shutdown()
    """, nranks=2)
    for _, rec in res:
        assert rec["worst"] < 1e-6 and rec["grads_match"] and rec["refused"]


def test_example_scripts_train_on_two_cpu_ranks():
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    launch = [sys.executable, "-m", "tensorflow_allreduce_b200.launch", "--nproc", "2", "--cpu"]
    r = subprocess.run(launch + [os.path.join(root, "examples", "data_parallel_training.py"), "--steps", "12"],
                       cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    assert "identical weights True" in r.stdout
    # the example of the reference's module docstring (mpi_collectives/__init__.py:81-111)
    r = subprocess.run(launch + [os.path.join(root, "examples", "linear_regression.py")], cwd=root, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2000:]
    assert "MPI Size: 2" in r.stdout and "Average Loss:" in r.stdout
