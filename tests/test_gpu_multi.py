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
class Rec(torch.nn.Module):
    # a recurrent stack whose weights share one flat storage after flatten_parameters()
    def __init__(self):
        super().__init__()
        self.inp = torch.nn.Linear(32, 48)
        self.rnn = torch.nn.GRU(48, 40, num_layers=3, bidirectional=True)
        self.out = torch.nn.Linear(80, 8)
    def forward(self, x):                      # [batch, 32] -> a sequence of 4 identical steps
        h = torch.tanh(self.inp(x)).unsqueeze(0).expand(4, -1, -1).contiguous()
        y, _ = self.rnn(h)
        return self.out(y.mean(0))
def make():
    torch.manual_seed(0)
    if os.environ.get("TEST_MODEL", "mlp") == "gru":
        m = Rec().cuda()
        m.rnn.flatten_parameters()
        return m
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
shared = len({p.untyped_storage().data_ptr() for p in mine.parameters()}) < len(list(mine.parameters()))
emit(worst=worst, identical=identical, fused=o_mine.fused, buckets=len(o_mine.buckets), shared_storage=shared)
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


@pytest.mark.parametrize("opt", ["sgd", "adamw", "rmsprop"])
def test_flattened_recurrent_weights_are_cut_into_buckets(opt):
    # nn.GRU after flatten_parameters(): all its weights are views of ONE storage. They keep that
    # layout, but the flat range is cut at parameter boundaries into several buckets that are
    # launched as backward finishes the layers. Same equivalence as above.
    res = run(TRAIN, nranks=2, gpus=True, timeout=300, env={"TEST_OPT": opt, "TEST_MODEL": "gru"})
    for _, rec in res:
        assert rec["worst"] < 1e-4, rec
        assert rec["identical"], "ranks diverged"
        assert rec["fused"] == (opt != "rmsprop")
        assert rec["buckets"] >= 6, rec          # 67 k recurrent weights in 8 KB buckets, plus the linear layers


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
    # 13 chained add -> allreduce stages on 1331 x 1331 fp32 with the closed-form check of the
    # reference (np.allclose there), 1000 iterations on as many GPUs as the box has. On top of it,
    # exactly: every iteration gives the bits of the first one, and all ranks hold the same bits.
    # Catches buffer-reuse and epoch bugs.
    res = run("""
    bc.init()
    stages, n = 13, 1331
    bad, drift = 0, 0
    first = None
    for it in range(1000):
        x = torch.ones(n, n, device="cuda") + RANK * 100
        for i in range(stages):
            x = bc.allreduce(x + 2.0 ** (i + 1), average=False)
        if first is None:
            first = x.clone()
            want = 1.0
            for i in range(stages):
                want = (want + 2.0 ** (i + 1)) * SIZE + (100 * SIZE * (SIZE - 1) / 2 if i == 0 else 0)
            if not torch.allclose(x, torch.full_like(x, want)): bad += 1
            if not bool((x == x[0, 0]).all()): bad += 1
        elif it % 50 == 0 or it == 999:
            if not torch.equal(x, first): drift += 1
    corner = bc.allgather(first[:1, :4].contiguous())
    same = bool((corner == corner[0:1]).all())
    bc.check_device_status()
    emit(bad=bad, drift=drift, same=same)
    bc.shutdown()
    """, nranks=_worlds()[-1], gpus=True, timeout=600)
    assert all(rec["bad"] == 0 and rec["drift"] == 0 and rec["same"] for _, rec in res), [rec for _, rec in res]


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


def test_second_backward_before_step():
    # Unfused: two backward passes before one step() accumulate like torch (the second pass lands
    # in buckets that were already averaged; step() averages those once more, which leaves the
    # part that is already equal on all ranks as it is). Fused: the update has been applied
    # during the first pass, so a second pass is refused with an error that names no_sync().
    res = run("""
    torch.backends.cuda.matmul.allow_tf32 = False
    bc.init()
    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4)).cuda()
    mine, ref = make(), make()
    o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.1, momentum=0.9), fused=False, bucket_mb=0.001)
    o_ref = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(3)
    X = torch.randn(4, 2, 8 * SIZE, 16, generator=g).cuda(); Y = torch.randn(4, 2, 8 * SIZE, 4, generator=g).cuda()
    sl = slice(RANK * 8, (RANK + 1) * 8)
    for it in range(4):
        o_ref.zero_grad(); o_mine.zero_grad()
        for k in range(2):                         # two backward passes, then one step
            torch.nn.functional.mse_loss(ref(X[it, k]), Y[it, k]).backward()
            torch.nn.functional.mse_loss(mine(X[it, k][sl]), Y[it, k][sl]).backward()
        o_ref.step(); o_mine.step()
    worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
    m2 = torch.nn.Sequential(torch.nn.Linear(16, 4)).cuda()
    o2 = bc.DistributedOptimizer(torch.optim.SGD(m2.parameters(), lr=0.1))
    assert o2.fused
    m2(X[0, 0][sl]).sum().backward()
    err = None
    try:
        m2(X[0, 1][sl]).sum().backward()
    except RuntimeError as e:
        err = str(e)
    o2.step()
    with o2.no_sync():                             # the supported way: accumulate locally, reduce with the last pass
        m2(X[1, 0][sl]).sum().backward()
    m2(X[1, 1][sl]).sum().backward()
    o2.step()
    torch.cuda.synchronize()
    bc.check_device_status()
    emit(worst=worst, err=err)
    bc.shutdown()
    """, nranks=2, gpus=True, timeout=300)
    for _, rec in res:
        assert rec["worst"] < 2e-5, rec
        assert rec["err"] and "no_sync" in rec["err"], rec


def test_sparse_gradients_on_a_gpu_group():
    # The reference reduces IndexedSlices by gathering values and indices
    # (tensorflow/contrib/mpi_collectives/__init__.py:148-158). Here: allreduce() of a sparse COO
    # CUDA tensor equals the dense allreduce, and a model with nn.Embedding(sparse=True) trains
    # through DistributedOptimizer(fused=False) like the single-process large batch.
    res = run("""
    bc.init()
    g = torch.Generator().manual_seed(11 + RANK)
    idx = torch.randint(0, 50, (2, 30 + 5 * RANK), generator=g)
    val = torch.randn(30 + 5 * RANK, generator=g)
    sp = torch.sparse_coo_tensor(idx, val, (50, 50)).cuda()
    dense_sum = bc.allreduce(sp.to_dense(), average=False)
    got = bc.allreduce(sp, average=False)
    ok_sum = got.is_sparse and torch.allclose(got.to_dense(), dense_sum, atol=1e-6)
    got = bc.allreduce(sp)                                   # average is the default
    ok_avg = torch.allclose(got.to_dense(), dense_sum / SIZE, atol=1e-6)

    class M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.emb = torch.nn.Embedding(100, 16, sparse=True)
            self.fc = torch.nn.Linear(16, 4)
        def forward(self, ids):
            return self.fc(self.emb(ids).mean(1))
    def make():
        torch.manual_seed(0)
        return M().cuda()
    mine, ref = make(), make()
    o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.5), fused=False)
    o_ref = torch.optim.SGD(ref.parameters(), lr=0.5)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 100, (5, 8 * SIZE, 6), generator=g).cuda(); Y = torch.randn(5, 8 * SIZE, 4, generator=g).cuda()
    sl = slice(RANK * 8, (RANK + 1) * 8)
    for it in range(5):
        o_ref.zero_grad(); o_mine.zero_grad()
        torch.nn.functional.mse_loss(ref(ids[it]), Y[it]).backward()
        torch.nn.functional.mse_loss(mine(ids[it][sl]), Y[it][sl]).backward()
        o_ref.step(); o_mine.step()
    worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
    torch.cuda.synchronize()
    bc.check_device_status()
    emit(ok_sum=bool(ok_sum), ok_avg=bool(ok_avg), worst=worst)
    bc.shutdown()
    """, nranks=2, gpus=True, timeout=300)
    for _, rec in res:
        assert rec["ok_sum"] and rec["ok_avg"], rec
        assert rec["worst"] < 2e-5, rec


def test_parameters_without_gradient_are_updated_with_zeros():
    # Documented difference from torch.optim: every parameter of a bucket is updated in every
    # step; one that received no gradient counts as having a zero gradient, so weight decay and
    # momentum still move it (torch skips parameters whose grad is None). Used parameters are
    # unaffected, and the ranks stay identical.
    res = run("""
    bc.init()
    torch.manual_seed(0)
    used = torch.nn.Linear(8, 4).cuda(); unused = torch.nn.Linear(8, 4).cuda()
    w0 = unused.weight.detach().clone()
    opt = bc.DistributedOptimizer(torch.optim.SGD(list(used.parameters()) + list(unused.parameters()), lr=0.1, momentum=0.9,
                                                  weight_decay=0.5))
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(RANK)).cuda()
    for _ in range(2):
        opt.zero_grad()
        used(x).sum().backward()
        opt.step()
    torch.cuda.synchronize()
    # two steps of p -= lr * buf with g = wd * p: step 1 buf = 0.5 p, p1 = 0.95 p; step 2 buf = 0.45 p + 0.475 p, p2 = p1 - 0.0925 p
    ratio = (unused.weight / w0).mean().item()
    flat = torch.cat([p.detach().reshape(-1) for p in list(used.parameters()) + list(unused.parameters())])
    allp = bc.allgather(flat.unsqueeze(0))
    emit(ratio=ratio, identical=bool((allp == allp[0:1]).all()), fused=opt.fused)
    bc.shutdown()
    """, nranks=2, gpus=True, timeout=300)
    for _, rec in res:
        assert rec["fused"] and rec["identical"]
        assert abs(rec["ratio"] - 0.8575) < 1e-4, rec


def test_staged_collectives_on_two_channels_do_not_share_staging():
    # A negotiated allreduce of a private tensor (channel 0) runs beside an ordered allreduce of
    # another private tensor (channel 2, its own stream): each channel stages in its own slice.
    res = run("""
    from tensorflow_allreduce_b200.ops.direct import allreduce_direct_
    bc.init()
    n = (6 << 20) + 5
    bad = 0
    for it in range(10):
        a = torch.full((n,), float(RANK + 1 + it), device="cuda")
        b = torch.full((n,), float(10 * (RANK + 1) + it), device="cuda")
        h = bc.allreduce_async(a, average=False, name=f"a.{it}")
        allreduce_direct_(b)
        ra = h.wait()
        want_a = sum(r + 1 + it for r in range(SIZE)); want_b = sum(10 * (r + 1) + it for r in range(SIZE))
        if not (bool((ra == want_a).all()) and bool((b == want_b).all())): bad += 1
    torch.cuda.synchronize()
    bc.check_device_status()
    emit(bad=bad)
    bc.shutdown()
    """, nranks=2, gpus=True, timeout=300)
    assert all(rec["bad"] == 0 for _, rec in res)


@pytest.mark.parametrize("world", _worlds()[:1] + _worlds()[-1:] if len(_worlds()) > 1 else _worlds())
def test_large_private_tensors_go_through_both_lanes(world):
    # Staging area of 8 MiB: 1 MiB per lane and channel, so a 9 MiB tensor travels in nine chunks
    # that alternate between the two lanes (streams, signal pads and halves of the slice).
    res = run("""
    bc.init()
    bad = []
    for dtype, n in ((torch.float32, (9 << 18) + 13), (torch.bfloat16, (9 << 19) + 5), (torch.int32, (3 << 18) + 1)):
        for it in range(3):
            g = torch.Generator(device="cuda").manual_seed(100 * it + 7)
            base = torch.randint(-50, 50, (n,), generator=g, device="cuda")
            x = (base + RANK).to(dtype)
            got = bc.allreduce(x, average=False)
            want = (base * SIZE + SIZE * (SIZE - 1) // 2).to(dtype)
            if not torch.equal(got, want): bad.append([str(dtype), it, (got.float() - want.float()).abs().max().item()])
            y = x.clone()
            bc.allreduce_(y, average=True)
            if dtype.is_floating_point and not torch.allclose(y.float(), want.float() / SIZE, rtol=1e-2): bad.append(["avg", str(dtype), it])
    torch.cuda.synchronize()
    bc.check_device_status()
    emit(bad=bad)
    bc.shutdown()
    """, nranks=world, gpus=True, timeout=300, env={"BC_STAGING_MB": "8"})
    for _, rec in res:
        assert rec["bad"] == [], rec


@pytest.mark.skipif(_ngpu() < 4, reason="the switch reduces only in groups of four or more GPUs")
def test_large_private_tensors_go_through_the_staged_pipeline_kernel():
    # A large ordinary tensor (by default from 96 MiB; here from 32 MiB) is reduced by ONE launch
    # whose copier blocks and reducer blocks work on different chunks of a ring in the staging slice. Integer-valued floats make
    # the sums exact: odd element counts (a tail below 16 bytes), fp32 and bf16, sum and average,
    # several calls in a row (the progress words run on), and the same tensors with that kernel
    # switched off must give bit-identical results. Four ranks: the group size at which the kernel
    # has been measured and its defaults chosen.
    world = 4
    res = run("""
    from tensorflow_allreduce_b200 import _lib
    bc.init()
    _lib.lib().bc_set_option(b"pipeline_min_bytes", 32 << 20)
    bad = []
    launches = []
    for dtype, n in ((torch.float32, (13 << 20) + 3), (torch.bfloat16, (40 << 20) + 5), (torch.float32, (96 << 20) + 1)):
        g = torch.Generator(device="cuda").manual_seed(11)
        base = torch.randint(-20, 20, (n,), generator=g, device="cuda", dtype=torch.int32)
        x = (base + RANK).to(dtype)
        want = (base * SIZE + SIZE * (SIZE - 1) // 2).to(dtype)
        outs = []
        for mode in (1, 0, 1):
            _lib.lib().bc_set_option(b"staged_pipeline", mode)
            got = bc.allreduce(x, average=False)
            if not torch.equal(got, want): bad.append([str(dtype), n, mode, (got.float() - want.float()).abs().max().item()])
            rec = [e for e in bc.stats() if e["device"] == 1][-1]
            launches.append([mode, rec["algo"], rec.get("launches", -1)])
            outs.append(got)
        if not (torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])): bad.append(["differs", str(dtype), n])
        y = x.clone()
        bc.allreduce_(y, average=True)
        if not torch.allclose(y.float(), want.float() / SIZE, rtol=1e-2, atol=1e-2): bad.append(["avg", str(dtype), n])
        del x, y, outs, got, want, base
    torch.cuda.synchronize()
    bc.check_device_status()
    emit(bad=bad, launches=launches)
    bc.shutdown()
    """, nranks=world, gpus=True, timeout=300)
    for _, rec in res:
        assert rec["bad"] == [], rec
        assert all(algo == "nvls" for _, algo, _ in rec["launches"]), rec
