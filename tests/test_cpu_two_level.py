"""Groups whose ranks sit on several hosts: node groups, rails and the two-level allreduce, with
one machine standing in for the hosts (every rank reports a host name of the test's choosing) and
host memory standing in for the GPUs. The reference reaches other hosts through MPI
(tensorflow/contrib/mpi_collectives/ring.h:183-225, mpi_ops.cc:609-613)."""
import pytest

from _util import run


def _hosts(nranks, per_host, interleaved=False):
    n_hosts = nranks // per_host
    env = {}
    for r in range(nranks):
        h = r % n_hosts if interleaved else r // per_host
        env[r] = {"BC_HOSTNAME": f"host{h}", "LOCAL_RANK": "-1", "BC_NODE_GROUPS": "1"}
    return env


BODY = """
import ctypes as C
from tensorflow_allreduce_b200 import _lib
bc.init(device="cpu")
lib = _lib.lib()
bad = []
from tensorflow_allreduce_b200.core import _DTYPES
for dtype in (torch.float32, torch.float64, torch.int32, torch.int64):
    for count in (0, 1, 3, 17, 1000, 4099):
        for op, average in ((0, 0), (0, 1), (2, 0), (3, 0)):
            g = torch.Generator().manual_seed(count * 7 + op)
            per_rank = [(torch.randint(-50, 50, (count,), generator=g) + r).to(dtype) for r in range(SIZE)]
            t = per_rank[RANK].clone()
            rc = lib.bc_two_level_allreduce_host(C.c_void_p(t.data_ptr()), count, _DTYPES[dtype], average, op)
            if rc != 0:
                bad.append(["rc", str(dtype), count, op, _lib.last_error()]); continue
            stack = torch.stack(per_rank) if count else torch.zeros(SIZE, 0, dtype=dtype)
            if op == 0:
                want = stack.sum(0)
                if average:
                    want = want / SIZE if dtype.is_floating_point else torch.div(want, SIZE, rounding_mode="trunc")
            elif op == 2:
                want = stack.min(0).values if count else stack[0]
            else:
                want = stack.max(0).values if count else stack[0]
            ok = torch.allclose(t.double(), want.double(), rtol=1e-6, atol=1e-6)
            if not ok:
                bad.append([str(dtype), count, op, average])
# the job-wide collectives still work next to the node groups
s = bc.allreduce(torch.tensor([float(RANK)]), average=False)
emit(bad=bad, nodes=bc.n_nodes(), node=bc.node_index(), local_rank=bc.local_rank(), local_size=bc.local_size(), s=s.item())
bc.shutdown()
"""


@pytest.mark.parametrize("nranks,per_host,interleaved", [(4, 2, False), (6, 2, True), (6, 3, False), (3, 1, False)])
def test_two_level_allreduce_over_fake_hosts(nranks, per_host, interleaved):
    res = run(BODY, nranks=nranks, per_rank_env=_hosts(nranks, per_host, interleaved), timeout=180)
    n_hosts = nranks // per_host
    for r, (_, rec) in enumerate(res):
        assert rec["bad"] == []
        assert rec["nodes"] == n_hosts and rec["local_size"] == per_host
        assert rec["node"] == (r % n_hosts if interleaved else r // per_host)
        assert rec["local_rank"] == (r // n_hosts if interleaved else r % per_host)
        assert rec["s"] == sum(range(nranks))


def test_one_host_has_no_node_groups():
    res = run("""
    import ctypes as C
    from tensorflow_allreduce_b200 import _lib
    bc.init(device="cpu")
    t = torch.ones(4)
    rc = _lib.lib().bc_two_level_allreduce_host(C.c_void_p(t.data_ptr()), 4, 0, 0, 0)
    emit(nodes=bc.n_nodes(), rc=rc, err=_lib.last_error())
    bc.shutdown()
    """, nranks=2, env={"BC_NODE_GROUPS": "1"})
    for _, rec in res:
        assert rec["nodes"] == 1 and rec["rc"] != 0 and "one host" in rec["err"]


def test_hosts_with_different_rank_counts_are_refused():
    env = {0: {"BC_HOSTNAME": "hostA"}, 1: {"BC_HOSTNAME": "hostA"}, 2: {"BC_HOSTNAME": "hostB"}}
    for e in env.values():
        e.update({"LOCAL_RANK": "-1", "BC_NODE_GROUPS": "1"})
    res = run("""
    try:
        bc.init(device="cpu")
        emit(ok=True)
        bc.shutdown()
    except Exception as e:
        emit(ok=False, err=str(e))
    """, nranks=3, per_rank_env=env)
    for _, rec in res:
        assert not rec["ok"] and "same number of ranks" in rec["err"] and "hostB" in rec["err"]


def test_distributed_optimizer_uses_flat_buffers_in_a_two_level_group():
    # 2 hosts x 2 ranks: gradients are averaged in flat buffers (two with this small bucket
    # size), and the
    # result equals the single-process large-batch run.
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
    worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
    names = sorted({s["name"] for s in bc.stats() if ".flat." in s["name"]})
    emit(worst=worst, names=names, nodes=bc.n_nodes())
    bc.shutdown()
    """, nranks=4, per_rank_env=_hosts(4, 2), env={"BC_BUCKET_MB": "0.001"})
    for _, rec in res:
        assert rec["worst"] < 1e-6 and rec["nodes"] == 2
        # 1048-byte buckets: the first weight (2048 bytes) alone, the other three tensors together
        assert rec["names"] == ["DistributedSGD.flat.0", "DistributedSGD.flat.1"]


PUBLIC = """
bc.init(device="cpu")
bad = []
for dtype in (torch.float32, torch.float64, torch.int32, torch.int64, torch.bfloat16, torch.uint8):
    for count in (0, 1, 5, 1000, 40001):
        g = torch.Generator().manual_seed(count)
        per_rank = [(torch.randint(0, 9, (count,), generator=g) + r).to(dtype) for r in range(SIZE)]
        x = per_rank[RANK]
        want = torch.stack([p.double() for p in per_rank]).sum(0) if count else torch.zeros(0, dtype=torch.float64)
        got = bc.allreduce(x, average=False)
        if got.dtype != dtype or not torch.equal(got.double(), want): bad.append(["sum", str(dtype), count])
        if dtype.is_floating_point:
            got = bc.allreduce(x, average=True)
            if not torch.allclose(got.double(), want / SIZE, rtol=1e-2 if dtype == torch.bfloat16 else 1e-6): bad.append(["avg", str(dtype), count])
        if count:
            got = bc.all_min(x)
            if not torch.equal(got.double(), torch.stack([p.double() for p in per_rank]).min(0).values): bad.append(["min", str(dtype), count])
t = torch.full((RANK + 1, 3), float(RANK))
g = bc.allgather(t)
if g.shape[0] != SIZE * (SIZE + 1) // 2 or g[-1, 0] != SIZE - 1: bad.append(["allgather"])
algos = sorted({s["algo"] for s in bc.stats() if s["op"] == "allreduce"})
phases = [s.get("two_level_s") for s in bc.stats() if s["op"] == "allreduce" and s["bytes"] > 100000][-1]
emit(bad=bad, nodes=bc.n_nodes(), algos=algos, phases=phases)
bc.shutdown()
"""


@pytest.mark.parametrize("groups", ["default", "pipelined", "pipelined_3x2", "off"])
def test_public_cpu_collectives_over_fake_hosts(groups):
    # 2 hosts x 2 ranks. By default the allreduce runs in two levels (shared memory inside a host,
    # rails between hosts; small slots so that tensors span many chunks); with BC_NODE_GROUPS=0 it
    # is the single ring over all ranks. "pipelined": chunks of 1 KiB, so that tensors from 4 KiB
    # on go chunk by chunk with the step between the hosts on a helper thread (the library's
    # chunks are 2 MiB); also with three hosts of two ranks.
    nranks = 6 if groups == "pipelined_3x2" else 4
    env = {r: {"BC_HOSTNAME": f"host{r // 2}", "LOCAL_RANK": "-1", "BC_SHM_SLOT_KB": "4"} for r in range(nranks)}
    for e in env.values():
        if groups == "off":
            e["BC_NODE_GROUPS"] = "0"
        e["BC_TWO_LEVEL_CHUNK_KB"] = "1" if groups.startswith("pipelined") else "0"
    res = run(PUBLIC, nranks=nranks, per_rank_env=env, timeout=180)
    for _, rec in res:
        assert rec["bad"] == []
        assert rec["nodes"] == (1 if groups == "off" else nranks // 2)
        assert rec["algos"] == (["cpu_ring"] if groups == "off" else ["cpu_shm"])
        # the records of a two-level allreduce carry the time of its three steps
        if groups != "off":
            assert len(rec["phases"]) == 3 and all(p > 0 for p in rec["phases"])
        else:
            assert rec["phases"] is None


def test_flat_buckets_with_accumulation_and_unused_parameters():
    # Two backward passes before one step (with and without no_sync()), a parameter that never
    # receives a gradient, and a check that the buckets really go out while backward still runs.
    res = run("""
    bc.init(device="cpu")
    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(0)
            self.a = torch.nn.Linear(8, 16); self.b = torch.nn.Linear(16, 2); self.unused = torch.nn.Linear(3, 3)
        def forward(self, x):
            return self.b(torch.tanh(self.a(x)))
    mine, ref = Net(), Net()
    o_mine = bc.DistributedOptimizer(torch.optim.SGD(mine.parameters(), lr=0.1))
    o_ref = torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(11)
    X = torch.randn(6, 4 * SIZE, 8, generator=g); Y = torch.randn(6, 4 * SIZE, 2, generator=g)
    sl = slice(RANK * 4, (RANK + 1) * 4)
    loss = torch.nn.functional.mse_loss
    launched_in_backward = []
    for it in range(0, 6, 2):
        o_ref.zero_grad()
        loss(ref(X[it]), Y[it]).backward(); loss(ref(X[it + 1]), Y[it + 1]).backward()
        o_ref.step()
        o_mine.zero_grad()
        if it == 2:
            with o_mine.no_sync():
                loss(mine(X[it][sl]), Y[it][sl]).backward()
        else:
            loss(mine(X[it][sl]), Y[it][sl]).backward()          # the buckets go out here already ...
        launched_in_backward.append(sum(b.handle is not None for b in o_mine._flat))
        loss(mine(X[it + 1][sl]), Y[it + 1][sl]).backward()      # ... and are reduced again after this one
        o_mine.step()
    worst = max((a - b).abs().max().item() for a, b in zip(ref.parameters(), mine.parameters()))
    emit(worst=worst, launched=launched_in_backward, unused_grad=mine.unused.weight.grad is None, buckets=len(o_mine._flat))
    bc.shutdown()
    """, nranks=4, per_rank_env=_hosts(4, 2), env={"BC_BUCKET_MB": "0.0002"})     # 209-byte buckets: [unused.*, b.*], [a.bias], [a.weight]
    for _, rec in res:
        assert rec["worst"] < 1e-6, rec
        assert rec["unused_grad"] and rec["buckets"] >= 3
        # iterations 0 and 4: every bucket whose parameters all got gradients was launched during
        # backward; iteration 2 ran under no_sync()
        assert rec["launched"][1] == 0 and rec["launched"][0] >= 2 and rec["launched"][2] >= 2
