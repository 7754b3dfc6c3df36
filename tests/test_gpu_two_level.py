"""A GPU group whose ranks report several hosts (one box stands in for them): the NVLink kernels
reduce inside each host, the rails carry the slices between hosts, and the optimizer wrapper
falls back to flat negotiated allreduces. 2 GPUs = 2 hosts x 1 rank, 4 GPUs = 2 hosts x 2 ranks.
8 GPUs = 2 hosts x 4 ranks.
The reference crosses hosts through a GPU-aware MPI (tensorflow/contrib/mpi_collectives/ring.h:183-225)."""
import pytest
import torch

from _util import run

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _layouts():
    out = [(2, 1)]
    if _ngpu() >= 4:
        out.append((4, 2))
    if _ngpu() >= 8:
        out.append((8, 4))
    return out


def _hosts(nranks, per_host):
    return {r: {"BC_HOSTNAME": f"host{r // per_host}", "LOCAL_RANK": "-1", "BC_NVLS": "0", "NCCL_NVLS_ENABLE": "0"}
            for r in range(nranks)}


COLLECTIVES = """
bc.init()
torch.cuda.set_device(RANK % torch.cuda.device_count())
bad = []
for dtype in (torch.float32, torch.bfloat16, torch.int32):
    for n in (1, 3, 1000, 70001, 3 << 20):
        g = torch.Generator().manual_seed(n)
        per_rank = [(torch.randint(-40, 40, (n,), generator=g) + r).to(dtype) for r in range(SIZE)]
        x = per_rank[RANK].cuda()
        want = torch.stack([p.double() for p in per_rank]).sum(0)
        got = bc.allreduce(x, average=False)
        if not torch.allclose(got.double().cpu(), want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-6):
            bad.append(["sum", str(dtype), n])
        if dtype.is_floating_point:
            got = bc.allreduce(x, average=True)
            if not torch.allclose(got.double().cpu(), want / SIZE, rtol=2e-2 if dtype == torch.bfloat16 else 1e-6, atol=1e-3):
                bad.append(["avg", str(dtype), n])
        got = bc.all_max(x)
        if not torch.equal(got.double().cpu(), torch.stack([p.double() for p in per_rank]).max(0).values):
            bad.append(["max", str(dtype), n])
t = (RANK * 100 + torch.arange((RANK + 2) * 4, dtype=torch.float32)).reshape(RANK + 2, 4).cuda()
g = bc.allgather(t)
want = torch.cat([(r * 100 + torch.arange((r + 2) * 4, dtype=torch.float32)).reshape(r + 2, 4) for r in range(SIZE)])
if not torch.equal(g.cpu(), want): bad.append(["allgather"])
torch.cuda.synchronize()
bc.check_device_status()
emit(bad=bad, nodes=bc.n_nodes(), local_size=bc.local_size())
bc.shutdown()
"""


@pytest.mark.parametrize("nranks,per_host", _layouts())
def test_collectives_over_fake_hosts(nranks, per_host):
    res = run(COLLECTIVES, nranks=nranks, gpus=True, timeout=300, per_rank_env=_hosts(nranks, per_host))
    for _, rec in res:
        assert rec["bad"] == [] and rec["nodes"] == nranks // per_host and rec["local_size"] == per_host


@pytest.mark.parametrize("nranks,per_host", _layouts())
def test_data_parallel_equals_large_batch_over_fake_hosts(nranks, per_host):
    from test_gpu_multi import TRAIN

    res = run(TRAIN, nranks=nranks, gpus=True, timeout=300, env={"TEST_OPT": "sgd"}, per_rank_env=_hosts(nranks, per_host))
    for _, rec in res:
        assert rec["worst"] < 2e-5, rec
        assert rec["identical"], "ranks diverged"
        assert not rec["fused"] and rec["buckets"] == 0
