"""`bc_group_allreduce_static`: the group allreduce for callers that cannot allocate device memory
(a process whose GPU memory is owned by one pool, or a loop that cannot afford the device-wide
synchronisation inside cudaMalloc). It is called here through its exported C symbol, several times
in a row, and each result is compared with the allocating entry point (`bc_emu_allreduce`) on the
same data and with a plain PyTorch sum in fp32 (rank order, rounded once). The scratch of the new entry point is one static array shared by all calls, so the
second call also proves that leftovers of the first one do no harm.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.float32: 0, torch.int32: 1, torch.bfloat16: 3}


def _static_fn():
    from tensorflow_allreduce_b200 import _lib

    lib = _lib.lib()
    fn = lib.bc_group_allreduce_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_longlong, C.c_int, C.c_float, C.c_int,
                   C.c_void_p, C.c_void_p, C.c_char_p, C.c_int]
    return fn


def _call_static(fn, ins, outs, count, dtype, scale, blocks, status):
    n = len(ins)
    ip = (C.c_void_p * n)(*[t if isinstance(t, int) else t.data_ptr() for t in ins])
    op = (C.c_void_p * n)(*[t if isinstance(t, int) else t.data_ptr() for t in outs])
    err = C.create_string_buffer(512)
    rc = fn(n, ip, op, count, DT[dtype], scale, blocks, C.c_void_p(status.data_ptr()) if status is not None else None,
            C.c_void_p(torch.cuda.current_stream().cuda_stream), err, len(err))
    return rc, err.value.decode()


def _torch_sum(xs, scale):
    """The same sum in plain PyTorch: rank order, fp32 accumulation for the 16-bit types, one rounding."""
    dtype = xs[0].dtype
    if not dtype.is_floating_point:
        acc = xs[0].clone()
        for x in xs[1:]:
            acc += x
        return acc
    acc = xs[0].float()
    for x in xs[1:]:
        acc = acc + x.float()
    return (acc * scale).to(dtype)


def _fill(dtype, n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
    return torch.randint(-1000, 1000, (n,), generator=g, device="cuda", dtype=dtype)


def test_static_entry_point_matches_allocating_one_twice():
    from tensorflow_allreduce_b200.ops.emulated import EmulatedGroup

    fn = _static_fn()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # two calls in a row with different group sizes, dtypes, lengths and grids
    for call, (nranks, dtype, n, scale, blocks) in enumerate([(4, torch.float32, 70001, 0.25, 3),
                                                              (8, torch.bfloat16, 12345, 1.0, 2),
                                                              (2, torch.int32, 999, 1.0, 1)]):
        xs = [_fill(dtype, n, 17 * call + r) for r in range(nranks)]
        keep = [x.clone() for x in xs]
        # existing, allocating entry point
        g = EmulatedGroup(nranks, 1 << 20)
        for r in range(nranks):
            g.buffer(r, dtype, n).copy_(xs[r])
        want = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(nranks)]
        g.allreduce(n, dtype, "two_shot", outs=want, scale=scale, blocks=blocks)
        # new entry point: nothing allocated on its behalf, inputs and outputs are ours
        got = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(nranks)]
        rc, err = _call_static(fn, xs, got, n, dtype, scale, blocks, status)
        assert rc == 0, err
        torch.cuda.synchronize()
        assert g.status == 0 and int(status.item()) == 0
        ref = _torch_sum(keep, scale)
        for r in range(nranks):
            assert torch.equal(got[r], want[r]), f"call {call} rank {r}"
            assert torch.equal(got[r], ref), f"call {call} rank {r}: differs from the PyTorch sum"
            assert torch.equal(xs[r], keep[r]), "inputs must stay untouched"
        g.close()


def test_static_entry_point_refuses_oversize_requests():
    fn = _static_fn()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    n = (1 << 20) // 4 + 4                       # just over 1 MiB of float32 per rank
    xs = [torch.zeros(n, device="cuda") for _ in range(2)]
    outs = [torch.full((n,), 7.0, device="cuda") for _ in range(2)]
    rc, err = _call_static(fn, xs, outs, n, torch.float32, 1.0, 1, status)
    assert rc == -1 and "exceeds the static scratch limit" in err
    rc, err = _call_static(fn, xs * 5, outs * 5, 16, torch.float32, 1.0, 1, status)   # 10 ranks
    assert rc == -1 and "nranks" in err
    rc, err = _call_static(fn, xs, xs, 16, torch.float32, 1.0, 1, status)
    assert rc == -1 and "aliases" in err
    # byte ranges that overlap without starting at the same address
    rc, err = _call_static(fn, xs, [xs[0].data_ptr() + 32, outs[1]], 16, torch.float32, 1.0, 1, status)
    assert rc == -1 and "aliases an input" in err
    rc, err = _call_static(fn, xs, [outs[0], outs[0].data_ptr() + 16], 16, torch.float32, 1.0, 1, status)
    assert rc == -1 and "two outputs alias" in err
    # a count whose size in bytes wraps around to zero must be refused as well
    for huge in (1 << 61, 1 << 62, (1 << 63) - 1):
        rc, err = _call_static(fn, xs, outs, huge, torch.float32, 1.0, 1, status)
        assert rc == -1 and "exceeds the static scratch limit" in err, (huge, err)
    # without a status word a timed-out wait could not be reported
    rc, err = _call_static(fn, xs, outs, 16, torch.float32, 1.0, 1, None)
    assert rc == -1 and "status_out" in err
    torch.cuda.synchronize()
    assert float(outs[0][0]) == 7.0              # nothing was launched
    # the limit itself is accepted
    n = (1 << 20) // 4
    xs = [torch.ones(n, device="cuda") * (r + 1) for r in range(2)]
    outs = [torch.empty(n, device="cuda") for _ in range(2)]
    rc, err = _call_static(fn, xs, outs, n, torch.float32, 1.0, 4, status)
    assert rc == 0, err
    torch.cuda.synchronize()
    assert float(outs[1][n - 1]) == 3.0 and int(status.item()) == 0
