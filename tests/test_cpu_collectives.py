"""CPU group, world size 2 and 3 over local sockets: the plumbing configuration (fp32 tensors of
shapes [17], [1000,10], [3,5,7] filled with N(0,1)+rank, sum and average; allgather of
[rank+2, 4]) and the cases of the reference's unit tests
(tensorflow/contrib/mpi_collectives/mpi_ops_test.py:70-263)."""
import pytest

from _util import run

# CPU tensors of ranks on one host travel through shared memory by default and over the socket
# ring with BC_SHM=0 (the ring is also what ranks on different hosts use).
TRANSPORTS = pytest.mark.parametrize("transport", ["shm", "ring"])


def _tenv(transport):
    return {"BC_SHM": "0"} if transport == "ring" else {"BC_SHM_SLOT_KB": "4"}      # 4 KiB slots: many chunks per tensor


def test_rank_size_single_process():
    # Without a launcher the library falls back to rank 0 / size 1 (mpi_ops_test.py:61-62).
    res = run("""
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"): os.environ.pop(k, None)
    bc.init(device="cpu")
    emit(rank=bc.rank(), size=bc.size(), local_rank=bc.local_rank())
    bc.shutdown()
    """, nranks=1)
    assert res[0][1] == {"rank": 0, "size": 1, "local_rank": 0}


@pytest.mark.parametrize("n", [2, 3])
def test_rank_size_env(n):
    res = run("""
    with bc.Session(device="cpu"):
        emit(rank=bc.rank(), size=bc.size(), local_rank=bc.local_rank(), local_size=bc.local_size())
    """, nranks=n)
    for i, (_, rec) in enumerate(res):
        assert rec == {"rank": i, "size": n, "local_rank": i, "local_size": n}


def test_ranks_of_several_hosts_get_per_host_local_ranks():
    # Two "hosts" on one machine (the reported host name is overridden per rank): local_rank counts
    # the lower ranks of the same host, as MPI_Comm_split_type(SHARED) does in the reference
    # (mpi_ops.cc:609-613); collectives span both hosts.
    res = run("""
    bc.init(device="cpu")
    s = bc.allreduce(torch.tensor([float(RANK)]), average=False)
    g = bc.allgather(torch.full((1, 1), float(bc.local_rank())))
    emit(local_rank=bc.local_rank(), local_size=bc.local_size(), s=s.item(), g=g.flatten().tolist())
    bc.shutdown()
    """, nranks=4, per_rank_env={r: {"BC_HOSTNAME": "hostA" if r % 2 == 0 else "hostB", "LOCAL_RANK": "-1"} for r in range(4)})   # -1: no launcher-given local rank
    assert [rec["local_rank"] for _, rec in res] == [0, 0, 1, 1]
    for _, rec in res:
        assert rec["local_size"] == 2 and rec["s"] == 6.0 and rec["g"] == [0.0, 0.0, 1.0, 1.0]


def test_ompi_env_names():
    res = run("""
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        v = os.environ.pop(k)
        os.environ["OMPI_COMM_WORLD_" + {"RANK": "RANK", "WORLD_SIZE": "SIZE", "LOCAL_RANK": "LOCAL_RANK"}[k]] = v
    bc.init(device="cpu")
    emit(rank=bc.rank(), size=bc.size())
    bc.shutdown()
    """, nranks=2)
    assert [r[1]["rank"] for r in res] == [0, 1]
    assert all(r[1]["size"] == 2 for r in res)


@TRANSPORTS
def test_plumbing_config_world2(transport):
    res = run("""
    bc.init(device="cpu")
    ok = True; worst = 0.0
    for shape in ([17], [1000, 10], [3, 5, 7]):
        per_rank = []
        for r in range(SIZE):
            g = torch.Generator().manual_seed(0)
            per_rank.append(torch.randn(shape, generator=g) + r)
        mine = per_rank[RANK]
        want = sum(per_rank)
        s = bc.allreduce(mine, average=False)
        a = bc.allreduce(mine, average=True)
        worst = max(worst, (s - want).abs().max().item(), (a - want / SIZE).abs().max().item())
        ok = ok and s.shape == mine.shape and s.dtype == mine.dtype
    t = (RANK * 100 + torch.arange((RANK + 2) * 4, dtype=torch.float32)).reshape(RANK + 2, 4)
    g = bc.allgather(t)
    want = torch.cat([(r * 100 + torch.arange((r + 2) * 4, dtype=torch.float32)).reshape(r + 2, 4) for r in range(SIZE)])
    emit(ok=bool(ok), worst=worst, gshape=list(g.shape), gather_ok=bool(torch.equal(g, want)))
    bc.shutdown()
    """, nranks=2, env=_tenv(transport))
    for _, rec in res:
        assert rec["ok"] and rec["worst"] <= 1e-6
        assert rec["gshape"] == [5, 4] and rec["gather_ok"]


@TRANSPORTS
@pytest.mark.parametrize("n", [2, 3])
def test_allreduce_cpu_like_reference(n, transport):
    # int32 + float32, 1/2/3-D [17]*dim, same tensor on every rank => expected = tensor * size,
    # exact for size <= 3 (mpi_ops_test.py:84-112).
    res = run("""
    bc.init(device="cpu")
    bad = []
    for dtype in (torch.int32, torch.float32, torch.int64, torch.float64, torch.bfloat16, torch.float16, torch.uint8):
        for dim in (1, 2, 3):
            g = torch.Generator().manual_seed(1234)
            if dtype.is_floating_point:
                t = (torch.rand([17] * dim, generator=g) * 200 - 100).to(dtype)
            elif dtype == torch.uint8:
                t = torch.randint(0, 40, [17] * dim, generator=g, dtype=dtype)
            else:
                t = torch.randint(-100, 100, [17] * dim, generator=g, dtype=dtype)
            s = bc.allreduce(t, average=False)
            want = (t.float() * SIZE).to(dtype) if dtype in (torch.bfloat16, torch.float16) else t * SIZE
            if not torch.equal(s, want):
                bad.append([str(dtype), dim, "sum"])
            a = bc.allreduce(t, average=True)
            if dtype.is_floating_point:
                tol = 1e-2 if dtype in (torch.bfloat16, torch.float16) else 1e-6
                if not torch.allclose(a.float(), t.float(), rtol=tol, atol=tol):
                    bad.append([str(dtype), dim, "avg"])
            elif not torch.equal(a, t):
                bad.append([str(dtype), dim, "avg"])
    emit(bad=bad)
    bc.shutdown()
    """, nranks=n, env=_tenv(transport))
    for _, rec in res:
        assert rec["bad"] == []


@TRANSPORTS
def test_prod_min_max_reductions(transport):
    # The reductions of the reference's NCCL ops (contrib/nccl/python/ops/nccl_ops.py:34-137) on a
    # CPU group of three ranks; a mismatch in the reduction fails on every rank.
    res = run("""
    bc.init(device="cpu")
    bad = []
    for dtype in (torch.float32, torch.int32, torch.int64, torch.float64, torch.bfloat16):
        xs = [((torch.arange(23) % 5) - 2 + r).to(dtype) for r in range(SIZE)]
        for op, fn in (("prod", lambda a, b: a * b), ("min", torch.minimum), ("max", torch.maximum), ("sum", lambda a, b: a + b)):
            want = xs[0]
            for x in xs[1:]:
                want = fn(want.float(), x.float()).to(dtype) if dtype == torch.bfloat16 else fn(want, x)
            got = bc.allreduce(xs[RANK], op=op, average=False)
            if not torch.equal(got, want):
                bad.append([str(dtype), op])
    helpers = [bc.all_sum(torch.tensor([1.0 + RANK])).item(), bc.all_prod(torch.tensor([2.0 + RANK])).item(),
               bc.all_min(torch.tensor([5 - RANK])).item(), bc.all_max(torch.tensor([5 - RANK])).item()]
    err = None
    try:
        bc.allreduce(torch.ones(4), op="max" if RANK == 0 else "min", name="mixed")
    except bc.CollectiveError as e:
        err = str(e)
    try:
        bc.allreduce(torch.ones(4), op="max", average=True)
        refused = False
    except ValueError:
        refused = True
    emit(bad=bad, helpers=helpers, err=err, refused=refused)
    bc.shutdown()
    """, nranks=3, env=_tenv(transport))
    for _, rec in res:
        assert rec["bad"] == []
        assert rec["helpers"] == [6.0, 24.0, 3, 5]
        assert "Mismatched reductions" in rec["err"]
        assert rec["refused"]


@TRANSPORTS
def test_integer_average_truncates(transport):
    res = run("""
    bc.init(device="cpu")
    t = torch.tensor([RANK * 3 + 1, -(RANK * 3 + 1), 7], dtype=torch.int32)
    emit(avg=bc.allreduce(t, average=True).tolist())
    bc.shutdown()
    """, nranks=2, env=_tenv(transport))
    # sums: [5, -5, 14] -> truncating division by 2
    for _, rec in res:
        assert rec["avg"] == [2, -2, 7]


@TRANSPORTS
@pytest.mark.parametrize("n", [2, 3])
def test_allgather_fixed_and_variable(n, transport):
    res = run("""
    bc.init(device="cpu")
    bad = []
    sizes = ([17, 32, 81, 12, 15, 23, 22] * 5)[:SIZE]
    for dtype in (torch.int32, torch.float32):
        for dim in (1, 2, 3):
            t = torch.ones([17] * dim, dtype=dtype) * RANK
            g = bc.allgather(t)
            if list(g.shape) != [17 * SIZE] + [17] * (dim - 1): bad.append(["fixed-shape", dim])
            for i in range(SIZE):
                if not bool((g[i * 17:(i + 1) * 17] == i).all()): bad.append(["fixed", dim, i])
            t = torch.ones([sizes[RANK]] + [17] * (dim - 1), dtype=dtype) * RANK
            g = bc.allgather(t)
            if list(g.shape) != [sum(sizes)] + [17] * (dim - 1): bad.append(["var-shape", dim])
            for i in range(SIZE):
                lo = sum(sizes[:i])
                if not bool((g[lo:lo + sizes[i]] == i).all()): bad.append(["var", dim, i])
    # zero rows on one rank, and everywhere
    t = torch.full((0 if RANK == 0 else 3, 2), float(RANK))
    g = bc.allgather(t)
    if g.shape[0] != 3 * (SIZE - 1): bad.append(["zero-rows", list(g.shape)])
    g = bc.allgather(torch.zeros(0, 5))
    if list(g.shape) != [0, 5]: bad.append(["all-empty", list(g.shape)])
    # zero-sized allreduce
    z = bc.allreduce(torch.zeros(0, 3))
    if list(z.shape) != [0, 3]: bad.append(["empty-allreduce"])
    emit(bad=bad)
    bc.shutdown()
    """, nranks=n, env=_tenv(transport))
    for _, rec in res:
        assert rec["bad"] == []


def test_sparse_allreduce_matches_dense():
    res = run("""
    bc.init(device="cpu")
    idx = torch.tensor([[RANK, 2, 2], [0, 1, RANK]])
    val = torch.tensor([1.0 + RANK, 2.0, 3.0])
    sp = torch.sparse_coo_tensor(idx, val, (4, 3))
    dense_avg = bc.allreduce(sp.to_dense(), average=True)
    sp_avg = bc.allreduce(sp, average=True)
    sp_sum = bc.allreduce(sp, average=False)
    emit(is_sparse=bool(sp_avg.is_sparse), avg_ok=bool(torch.allclose(sp_avg.to_dense(), dense_avg)),
         sum_ok=bool(torch.allclose(sp_sum.to_dense(), dense_avg * SIZE)), nnz=int(sp_sum._nnz()))
    bc.shutdown()
    """, nranks=2)
    for _, rec in res:
        assert rec == {"is_sparse": True, "avg_ok": True, "sum_ok": True, "nnz": 6}


def test_broadcast_and_named_out_of_order():
    res = run("""
    bc.init(device="cpu")
    t = torch.arange(6.).reshape(2, 3) + 10 * RANK
    b = bc.broadcast(t, root=1)
    # names decide what is matched with what, not the call order (mpi_ops.cc:255-269)
    x = torch.full((4,), 1.0 + RANK); y = torch.full((5,), 10.0 + RANK)
    if RANK == 0:
        hx = bc.allreduce_async(x, average=False, name="x"); hy = bc.allreduce_async(y, average=False, name="y")
    else:
        hy = bc.allreduce_async(y, average=False, name="y"); hx = bc.allreduce_async(x, average=False, name="x")
    emit(b=b.tolist(), x=hx.wait().tolist(), y=hy.wait().tolist(), objs=bc.host_allgather({"r": RANK}))
    bc.shutdown()
    """, nranks=2)
    for _, rec in res:
        assert rec["b"] == [[10.0, 11.0, 12.0], [13.0, 14.0, 15.0]]
        assert rec["x"] == [3.0] * 4 and rec["y"] == [21.0] * 5
        assert rec["objs"] == [{"r": 0}, {"r": 1}]


@TRANSPORTS
def test_dependent_allreduce_chain(transport):
    # Chained add -> allreduce stages with a closed-form result, as the reference's stress test
    # (mpi_allreduce_test.py:35-128), shortened for the CPU path.
    res = run("""
    bc.init(device="cpu")
    stages, n = 6, 121
    ok = True
    for it in range(20):
        x = torch.ones(n, n) + RANK * 100
        for i in range(stages):
            x = bc.allreduce(x + 2.0 ** (i + 1), average=False)
        want = 1.0
        for i in range(stages):
            want = (want + 2.0 ** (i + 1)) * SIZE + (100 * SIZE * (SIZE - 1) / 2 if i == 0 else 0)
        ok = ok and bool(torch.allclose(x, torch.full_like(x, want)))
    emit(ok=ok)
    bc.shutdown()
    """, nranks=2, env=_tenv(transport))
    assert all(rec["ok"] for _, rec in res)


def test_concurrent_callers_from_several_threads():
    # Four threads per rank issue named collectives at the same time (the reference's NcclManager test drives its manager from a thread pool,
    # tensorflow/contrib/nccl/kernels/nccl_manager_test.cc:184-282). Names pair the requests up.
    res = run("""
    import threading
    bc.init(device="cpu")
    bad = []
    def work(tid):
        # a thread blocks in every call, so thread `tid` must walk its names in the same order on
        # every rank; the threads of one rank run against each other freely
        order = list(range(12))
        if tid % 2: order.reverse()
        try:
            for k in order:
                x = torch.full((257,), float(RANK + tid + k))
                s = bc.allreduce(x, average=False, name=f"t{tid}.k{k}")
                want = sum(r + tid + k for r in range(SIZE))
                if not bool((s == want).all()): bad.append([tid, k])
                g = bc.allgather(torch.full((RANK + 1, 2), float(tid)), name=f"g{tid}.k{k}")
                if g.shape[0] != SIZE * (SIZE + 1) // 2 or not bool((g == tid).all()): bad.append(["g", tid, k])
        except Exception as e:
            bad.append([tid, "exception", str(e)])
    ts = [threading.Thread(target=work, args=(t,)) for t in range(4)]
    for t in ts: t.start()
    for t in ts: t.join()
    emit(bad=bad)
    bc.shutdown()
    """, nranks=3, timeout=120)
    for _, rec in res:
        assert rec["bad"] == []


def test_shared_memory_that_cannot_be_set_up_falls_back_to_sockets():
    # Slots of 1 TiB cannot be reserved anywhere: every rank learns of it in the same exchange
    # and the group runs over the socket ring.
    res = run("""
    bc.init(device="cpu")
    s = bc.allreduce(torch.arange(1000.0) + RANK, average=False)
    ok = bool(torch.equal(s, torch.arange(1000.0) * SIZE + sum(range(SIZE))))
    emit(ok=ok, algo=[e["algo"] for e in bc.stats() if e["op"] == "allreduce"][-1])
    bc.shutdown()
    """, nranks=3, env={"BC_SHM_SLOT_KB": str(1 << 30)})
    for _, rec in res:
        assert rec["ok"] and rec["algo"] == "cpu_ring"


def test_collectives_carry_no_gradient():
    # The reference registers its ops as NotDifferentiable (mpi_ops.py:135,163): results are
    # plain tensors, and the input's autograd graph is left alone.
    res = run("""
    bc.init(device="cpu")
    x = torch.ones(3, requires_grad=True)
    y = bc.allreduce(x * 2, average=False)
    g = bc.allgather((x * 3).reshape(1, 3))
    b = bc.broadcast(x * 4, root=0)
    (x * 5).sum().backward()
    emit(flags=[y.requires_grad, g.requires_grad, b.requires_grad], fns=[y.grad_fn is None, g.grad_fn is None],
         grad=x.grad.tolist(), y=y.tolist())
    bc.shutdown()
    """, nranks=2)
    for _, rec in res:
        assert rec["flags"] == [False, False, False] and rec["fns"] == [True, True]
        assert rec["grad"] == [5.0, 5.0, 5.0] and rec["y"] == [4.0, 4.0, 4.0]


def test_grouped_allreduce_packs_by_dtype():
    res = run("""
    bc.init(device="cpu")
    ts = [torch.full((3, 2), 1.0 + RANK), torch.arange(5, dtype=torch.int64) * (RANK + 1), torch.full((), 2.0 * RANK), torch.zeros(0)]
    bc.clear_stats()
    avg = bc.grouped_allreduce(ts, name="grp")
    tot = bc.grouped_allreduce(ts, average=False, name="grp2")
    names = sorted(e["name"] for e in bc.stats() if e["op"] == "allreduce")
    tri = SIZE * (SIZE + 1) // 2
    ok = (torch.equal(tot[0], torch.full((3, 2), float(tri))) and torch.equal(tot[1], torch.arange(5) * tri)
          and tot[2].item() == SIZE * (SIZE - 1) and tot[3].shape == (0,)
          and torch.allclose(avg[0], torch.full((3, 2), tri / SIZE)) and avg[2].shape == () and [t.dtype for t in tot] == [t.dtype for t in ts])
    emit(ok=bool(ok), names=names)
    bc.shutdown()
    """, nranks=3)
    for _, rec in res:
        assert rec["ok"] and rec["names"] == ["grp.0", "grp.1", "grp2.0", "grp2.1"]      # one collective per dtype


def test_repeated_init_and_shutdown_leak_nothing():
    # Twenty groups in a row in the same processes: descriptors are all closed again and no
    # shared-memory object is left behind.
    res = run("""
    import glob
    def nfds(): return len(os.listdir("/proc/self/fd"))
    base = None
    for it in range(20):
        bc.init(device="cpu")                     # the same rendezvous port every time
        s = bc.allreduce(torch.ones(1000) * (RANK + it), average=False)
        assert s[0].item() == sum(r + it for r in range(SIZE))
        bc.allgather(torch.ones(RANK + 1, 2))
        bc.shutdown()
        if it == 2: base = nfds()
    emit(grew=nfds() - base, shm=sorted(glob.glob("/dev/shm/bcoll-*")))
    """, nranks=3, timeout=180)
    for _, rec in res:
        assert rec["grew"] == 0 and rec["shm"] == []
