"""Negotiation: mismatched requests fail on EVERY rank with the reference's wording and leave the
group usable (tensorflow/contrib/mpi_collectives/mpi_ops_test.py:158-202, 265-297; rules in
mpi_ops.cc:277-432), plus the validation function on synthetic requests."""
import ctypes as C

import pytest

from _util import run


def _validate(lib, ops, dtypes, shapes, devices=None):
    n = len(ops)
    devices = devices or [0] * n
    arr = lambda xs: (C.c_int * n)(*xs)  # noqa: E731
    flat = (C.c_longlong * (8 * n))()
    for r, s in enumerate(shapes):
        for i, d in enumerate(s):
            flat[8 * r + i] = d
    err = C.create_string_buffer(1024)
    dim0 = (C.c_longlong * n)()
    rt = lib.bc_test_validate(n, arr(ops), arr(dtypes), arr(devices), arr([len(s) for s in shapes]), flat, err, 1024, dim0)
    return rt, err.value.decode(), list(dim0)


def test_validation_rules(native_lib):
    AR, AG, ERR = 0, 1, 3
    F32, I32 = 0, 1
    rt, err, _ = _validate(native_lib, [AR, AR], [F32, F32], [[17, 3], [17, 3]])
    assert rt == 0 and err == ""
    rt, err, _ = _validate(native_lib, [AR, AR], [F32, I32], [[17], [17]])
    assert rt == ERR and err == "Mismatched data types: One rank had type float32, but another rank had type int32."
    rt, err, _ = _validate(native_lib, [AR, AG], [F32, F32], [[17], [17]])
    assert rt == ERR and err.startswith("Mismatched MPI operations: One rank did an ALLREDUCE, but another rank did an ALLGATHER")
    rt, err, _ = _validate(native_lib, [AR, AR, AR], [F32] * 3, [[17, 23 * 57], [17, 23, 57], [17, 23, 57]])
    assert rt == ERR and "Mismatched allreduce tensor shapes" in err and "[17,1311]" in err and "[17,23,57]" in err
    rt, err, dim0 = _validate(native_lib, [AG, AG, AG], [F32] * 3, [[2, 4], [0, 4], [5, 4]])
    assert rt == 1 and dim0 == [2, 0, 5]      # a zero-sized dimension survives the wire format
    rt, err, _ = _validate(native_lib, [AG, AG], [F32, F32], [[3, 10, 17], [3, 20, 17]])
    assert rt == ERR and err == ("Mismatched allgather tensor shapes: One rank gathered a tensor with dimension 1 equal to 10, "
                                 "but another rank sent a tensor with dimension 1 equal to 20.")
    rt, err, _ = _validate(native_lib, [AG, AG], [F32, F32], [[3, 10], [3, 10, 1]])
    assert rt == ERR and "One rank gathered a tensor of rank 2, but another rank sent a tensor of rank 3" in err
    rt, err, _ = _validate(native_lib, [AG, AG], [F32, F32], [[], []])
    assert rt == ERR and err == "Rank zero tried to gather a rank-zero tensor."
    rt, err, _ = _validate(native_lib, [AR, AR], [F32, F32], [[4], [4]], devices=[0, 1])
    assert rt == ERR and "Mismatched devices" in err


def test_use_before_init_fails():
    res = run("""
    try:
        bc.allreduce(torch.ones(3))
        emit(err=None)
    except bc.CollectiveError as e:
        emit(err=str(e))
    """, nranks=1)
    assert "MPI has not been initialized" in res[0][1]["err"]


@pytest.mark.parametrize("n", [2, 3])
def test_mismatch_errors_reach_every_rank(n):
    res = run("""
    bc.init(device="cpu")
    errs = {}
    def attempt(key, fn):
        try:
            fn(); errs[key] = None
        except bc.CollectiveError as e:
            errs[key] = str(e)
    attempt("shape", lambda: bc.allreduce(torch.ones([17 + RANK] * 3)))
    attempt("rank", lambda: bc.allreduce(torch.ones(17, 23 * 57) if RANK == 0 else torch.ones(17, 23, 57)))
    attempt("dtype", lambda: bc.allreduce(torch.ones([17] * 3, dtype=torch.int32 if RANK % 2 == 0 else torch.float32)))
    def ag_shape():
        s = [17] * 3; s[1] = 10 * (RANK + 1)
        bc.allgather(torch.ones(s) * RANK)
    attempt("ag_shape", ag_shape)
    attempt("ag_dtype", lambda: bc.allgather(torch.ones([17] * 3, dtype=torch.int32 if RANK % 2 == 0 else torch.float32)))
    attempt("ag_scalar", lambda: bc.allgather(torch.tensor(1.0)))
    attempt("op", lambda: (bc.allreduce(torch.ones(4), name="same") if RANK == 0 else bc.allgather(torch.ones(4), name="same")))
    # the group still works afterwards
    ok = bc.allreduce(torch.ones(5), average=False).tolist()
    emit(errs=errs, ok=ok)
    bc.shutdown()
    """, nranks=n)
    for _, rec in res:
        e = rec["errs"]
        assert "Mismatched allreduce tensor shapes" in e["shape"]
        assert "Mismatched allreduce tensor shapes" in e["rank"]
        assert "Mismatched data types" in e["dtype"]
        assert "Mismatched allgather tensor shapes" in e["ag_shape"]
        assert "Mismatched data types" in e["ag_dtype"]
        assert "rank-zero tensor" in e["ag_scalar"]
        assert "Mismatched MPI operations" in e["op"]
        assert rec["ok"] == [float(n)] * 5


def test_duplicate_name_in_flight_is_rejected():
    res = run("""
    bc.init(device="cpu")
    import time
    err = None
    if RANK == 0:
        h = bc.allreduce_async(torch.ones(3), name="dup")
        try:
            bc.allreduce_async(torch.ones(3), name="dup")
        except bc.CollectiveError as e:
            err = str(e)
        bc.barrier(name="go")
        out = h.wait()
    else:
        bc.barrier(name="go")
        out = bc.allreduce(torch.ones(3), name="dup")
    emit(err=err, out=out.tolist())
    bc.shutdown()
    """, nranks=2)
    assert "already in flight" in res[0][1]["err"]
    assert res[0][1]["out"] == [1.0] * 3 and res[1][1]["out"] == [1.0] * 3
