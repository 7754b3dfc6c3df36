"""Real multi-process groups, one rank per GPU (2 ranks, and 4/8 when the box has them):
symmetric memory across processes, every allreduce variant, the variable allgather, the
DistributedOptimizer against a single-process large-batch run, and the stress chain of the
reference (tensorflow/contrib/mpi_collectives/mpi_allreduce_test.py:35-128)."""
import pytest
import torch

from _util import run

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _worlds():
    n = _ngpu()
    return [w for w in (2, 4, 8) if w <= n] or [2]


COLLECTIVES = """
bc.init()
dev = torch.device("cuda", bc.local_rank())
from tensorflow_allreduce_b200.ops import symmetric
bad = []
def fill(dtype, n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
    return torch.randint(-1000, 1000, (n,), generator=g, device="cuda", dtype=dtype)
def ref_sum(xs, dtype):
    if dtype in (torch.bfloat16, torch.float16):
        acc = xs[0].float()
        for x in xs[1:]: acc = acc + x.float()
        return acc.to(dtype)
    acc = xs[0].clone()
    for x in xs[1:]: acc = acc + x
    return acc
def same(got, want, dtype, mag):
    # The in-switch (NVLS) reduction sums in its own order and, for 16-bit floats, may round
    # differently from "sum in fp32, round once": allow one unit in the last place of the largest
    # partial sum that can occur (the sum of magnitudes). Everything else must be bit-exact.
    if dtype.is_floating_point and bc.stats()[-1]["algo"] == "nvls":
        ulp = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 2.0 ** -21}[dtype]
        return bool(((got.float() - want.float()).abs() <= ulp * mag.clamp_min(2.0 ** -10)).all())
    return bool(torch.equal(got, want))
for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64):
    for n in (1, 17, 4913, (1 << 16) + 3, (1 << 21) + 11):
        xs = [fill(dtype, n, 1000 * r + n % 97) for r in range(SIZE)]
        want = ref_sum(xs, dtype)
        mag = sum(x.float().abs() for x in xs)
        got = bc.allreduce(xs[RANK], average=False)
        if not same(got, want, dtype, mag): bad.append(["staged", str(dtype), n, bc.stats()[-1]["algo"], (got.float() - want.float()).abs().max().item()])
        # in place on symmetric memory (zero-copy)
        s = symmetric.empty((n,), dtype)
        s.copy_(xs[RANK])
        bc.allreduce_(s, average=False)
        if not same(s, want, dtype, mag): bad.append(["symmetric", str(dtype), n, bc.stats()[-1]["algo"], (s.float() - want.float()).abs().max().item()])
algos = sorted({e["algo"] for e in bc.stats() if e["device"] == 1})
# variable allgather: (rank+1)*k rows
for k, cols, dtype in ((1, 4, torch.float32), (3, 17, torch.int32), (64, 256, torch.bfloat16), (5, 1, torch.uint8)):
    t = (torch.ones((RANK + 1) * k, cols, device="cuda") * RANK).to(dtype)
    g = bc.allgather(t)
    lo = 0
    for r in range(SIZE):
        rows = (r + 1) * k
        if not bool((g[lo:lo + rows] == r).all()): bad.append(["allgather", k, r])
        lo += rows
    if g.shape[0] != lo: bad.append(["allgather-shape", k])
t = torch.full((0 if RANK == 0 else 3, 2), float(RANK), device="cuda")
g = bc.allgather(t)
if g.shape[0] != 3 * (SIZE - 1): bad.append(["allgather-zero-rows"])
b = bc.broadcast(torch.arange(10., device="cuda") + RANK, root=SIZE - 1)
if not torch.equal(b.cpu(), torch.arange(10.) + SIZE - 1): bad.append(["broadcast"])
torch.cuda.synchronize()
bc.check_device_status()
emit(bad=bad, algos=algos, symm=symmetric.describe())
bc.shutdown()
"""


@pytest.mark.parametrize("world", _worlds())
@pytest.mark.parametrize("env", [{}, {"BC_ALGO": "two_shot"}, {"BC_NVLS": "0"}, {"BC_SYMM": "ipc"}, {"BC_ALGO": "nvls"}])
def test_collectives_across_gpus(world, env):
    res = run(COLLECTIVES, nranks=world, gpus=True, timeout=300, env=env)
    for _, rec in res:
        assert rec["bad"] == [], rec
    if not env:
        assert "one_shot" in res[0][1]["algos"]


@pytest.mark.parametrize("world", _worlds()[:1] + _worlds()[-1:] if len(_worlds()) > 1 else _worlds())
def test_allgather_larger_than_staging_goes_in_rounds(world):
    # Heap and staging area of 1 MiB each: a 6 MiB result can only be gathered piecewise.
    res = run("""
    bc.init()
    bad = []
    for k, cols, dtype in ((20000, 13, torch.float32), (7001, 3, torch.bfloat16), (100000, 1, torch.uint8)):
        rows = (RANK + 1) * k
        t = (torch.arange(rows * cols, device="cuda") % 251 + RANK).reshape(rows, cols).to(dtype)
        g = bc.allgather(t)
        lo = 0
        for r in range(SIZE):
            n = (r + 1) * k
            want = (torch.arange(n * cols, device="cuda") % 251 + r).reshape(n, cols).to(dtype)
            if not torch.equal(g[lo:lo + n], want): bad.append([k, r])
            lo += n
        if g.shape[0] != lo: bad.append(["shape", k])
    torch.cuda.synchronize()
    bc.check_device_status()
    emit(bad=bad)
    bc.shutdown()
    """, nranks=world, gpus=True, timeout=300, env={"BC_STAGING_MB": "1", "BC_HEAP_MB": "1"})
    for _, rec in res:
        assert rec["bad"] == [], rec


def test_error_paths_on_gpu_group():
    res = run("""
    bc.init()
    errs = []
    try:
        bc.allreduce(torch.ones(17 + RANK, device="cuda"))
    except bc.CollectiveError as e:
        errs.append(str(e))
    try:
        bc.allreduce(torch.ones(5, device="cuda") if RANK == 0 else torch.ones(5), name="mixed")
    except bc.CollectiveError as e:
        errs.append(str(e))
    ok = bc.allreduce(torch.ones(4, device="cuda"), average=False)   # still usable afterwards
    emit(errs=errs, ok=ok.tolist())
    bc.shutdown()
    """, nranks=2, gpus=True, timeout=180)
    for _, rec in res:
        assert "Mismatched allreduce tensor shapes" in rec["errs"][0]
        assert "Mismatched devices" in rec["errs"][1]
        assert rec["ok"] == [2.0] * 4


TRAIN = """
import copy
torch.backends.cudnn.allow_tf32 = False
torch.backends.cuda.matmul.allow_tf32 = False
bc.init()
torch.manual_seed(0)
def make():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 64), torch.nn.Tanh(),
                               torch.nn.Linear(64, 8)).cuda()
OPT = os.environ.get("TEST_OPT", "sgd")
def mk(ps):
    if OPT == "sgd": return torch.optim.SGD(ps, lr=0.05, momentum=0.9)
    if OPT == "adamw": return torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.05)
    return torch.optim.RMSprop(ps, lr=1e-3)
mine = make(); ref = make()
o_mine = bc.DistributedOptimizer(mk(mine.parameters()), bucket_mb=0.008)
o_ref = mk(ref.parameters())
g = torch.Generator().manual_seed(5)
X = torch.randn(6, 16 * SIZE, 32, generator=g).cuda(); Y = torch.randn(6, 16 * SIZE, 8, generator=g).cuda()
for it in range(6):
    xs, ys = X[it], Y[it]
    o_ref.zero_grad()
    torch.nn.functional.mse_loss(ref(xs), ys).backward()          # whole batch on one process
    o_ref.step()
    o_mine.zero_grad()
    sl = slice(RANK * 16, (RANK + 1) * 16)                          # this rank's shard
    torch.nn.functional.mse_loss(mine(xs[sl]), ys[sl]).backward()
    o_mine.step()
worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
flat = torch.cat([p.detach().reshape(-1) for p in mine.parameters()])
allp = bc.allgather(flat.unsqueeze(0))
identical = bool((allp == allp[0:1]).all())
bc.check_device_status()
emit(worst=worst, identical=identical, fused=o_mine.fused, buckets=len(o_mine.buckets))
bc.shutdown()
"""


@pytest.mark.parametrize("world", _worlds()[:2])
@pytest.mark.parametrize("opt", ["sgd", "adamw", "rmsprop"])
def test_data_parallel_equals_large_batch(world, opt):
    res = run(TRAIN, nranks=world, gpus=True, timeout=300, env={"TEST_OPT": opt})
    for _, rec in res:
        assert rec["worst"] < 2e-5, rec
        assert rec["identical"], "ranks diverged"
        assert rec["fused"] == (opt != "rmsprop")
        assert rec["buckets"] > 1


@pytest.mark.parametrize("opt", ["sgd", "adamw"])
def test_fused_update_over_nvls(opt):
    # The switch-side reduction forced for every bucket (it is the default only from 4 ranks and
    # 512 KiB on): same equivalence with the single-process large-batch run.
    res = run(TRAIN, nranks=2, gpus=True, timeout=300, env={"TEST_OPT": opt, "BC_ALGO": "nvls"})
    for _, rec in res:
        assert rec["worst"] < 2e-5, rec
        assert rec["identical"], "ranks diverged"
        assert rec["fused"]


def test_synchronize_allows_clipping_before_step():
    from test_cpu_training import CLIP

    res = run(CLIP % ("", "cuda"), nranks=2, gpus=True, timeout=300)
    for _, rec in res:
        assert rec["worst"] < 2e-5 and rec["clipped"] and rec["fused_refuses"]


def test_dependent_allreduce_stress():
    # 13 chained add -> allreduce stages on 1331 x 1331 fp32, closed-form check, many iterations:
    # catches buffer-reuse and epoch bugs.
    res = run("""
    bc.init()
    stages, n = 13, 1331
    bad = 0
    for it in range(60):
        x = torch.ones(n, n, device="cuda") + RANK * 100
        for i in range(stages):
            x = bc.allreduce(x + 2.0 ** (i + 1), average=False)
        want = 1.0
        for i in range(stages):
            want = (want + 2.0 ** (i + 1)) * SIZE + (100 * SIZE * (SIZE - 1) / 2 if i == 0 else 0)
        if not torch.allclose(x, torch.full_like(x, want)): bad += 1
    bc.check_device_status()
    emit(bad=bad)
    bc.shutdown()
    """, nranks=min(_ngpu(), 4) if _ngpu() >= 2 else 2, gpus=True, timeout=300)
    assert all(rec["bad"] == 0 for _, rec in res)


def test_rank_leaves_between_steps():
    # A rank exits cleanly between steps (no kernel in flight); the others learn of it on the
    # host and their next collective fails with an error instead of hanging. NVLS off.
    res = run("""
    bc.init()
    x = bc.allreduce(torch.ones(1000, device="cuda"), average=False)
    torch.cuda.synchronize()
    if RANK == 1:
        emit(left=True)
        os._exit(0)
    import time
    err = None
    t0 = time.time()
    try:
        for i in range(200):
            bc.allreduce(torch.ones(1000, device="cuda"), name=f"after.{i}")
            time.sleep(0.05)
    except bc.CollectiveError as e:
        err = str(e)
    emit(err=err, secs=time.time() - t0, first=float(x[0]))
    """, nranks=2, gpus=True, timeout=120, env={"BC_NVLS": "0", "NCCL_NVLS_ENABLE": "0", "BC_TIMEOUT_S": "5"}, expect_ok=False)
    rec0 = res[0][1]
    assert rec0 is not None and rec0["err"] is not None, res[0][0].stderr[-2000:]
    assert rec0["secs"] < 30 and rec0["first"] == 2.0
