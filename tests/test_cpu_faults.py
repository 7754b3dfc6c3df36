"""Failure detection, exercised on the host only (CPU ranks, no GPU involved): a request that is
never sent, a late rank, a rank that exits (before or inside a collective), a control connection that closes. The reference has
none of this: a missing rank blocks everyone in MPI_Probe for ever
(tensorflow/contrib/mpi_collectives/mpi_ops.cc:684,763)."""
import time

import pytest

from _util import run


def test_dropped_request_times_out_on_every_rank():
    res = run("""
    bc.init(device="cpu")
    import time
    t0 = time.time()
    try:
        bc.allreduce(torch.ones(4), name="lost")
        err = None
    except bc.CollectiveError as e:
        err = str(e)
    dt = time.time() - t0
    ok = bc.allreduce(torch.ones(2), average=False, name="after").tolist()   # group survives a timeout
    emit(err=err, dt=dt, ok=ok)
    bc.shutdown()
    """, nranks=2, env={"BC_TIMEOUT_S": "2", "BC_FAULT": "drop_request:rank=1:name=lost"}, timeout=60)
    for _, rec in res:
        assert rec["err"] is not None and "Timed out" in rec["err"] and "rank(s) 1" in rec["err"]
        assert rec["dt"] < 15
        assert rec["ok"] == [2.0, 2.0]


def test_late_rank_within_deadline_is_fine():
    res = run("""
    bc.init(device="cpu")
    out = bc.allreduce(torch.ones(4) * (RANK + 1), average=False, name="slow")
    emit(out=out.tolist())
    bc.shutdown()
    """, nranks=2, env={"BC_TIMEOUT_S": "20", "BC_FAULT": "delay_ms=700:rank=1:name=slow"}, timeout=60)
    for _, rec in res:
        assert rec["out"] == [3.0] * 4


def test_rank_exit_fails_the_others_quickly():
    t0 = time.time()
    res = run("""
    bc.init(device="cpu")
    bc.allreduce(torch.ones(4), name="warm")
    try:
        bc.allreduce(torch.ones(4), name="doomed")
        err = None
    except bc.CollectiveError as e:
        err = str(e)
    later = None
    try:
        bc.allreduce(torch.ones(4), name="later")
    except bc.CollectiveError as e:
        later = str(e)
    emit(err=err, later=later)
    """, nranks=3, env={"BC_TIMEOUT_S": "30", "BC_FAULT": "exit_before:rank=2:name=doomed"}, timeout=90, expect_ok=False)
    assert time.time() - t0 < 60
    assert res[2][0].returncode == 41            # the injected exit
    for r in (0, 1):
        rec = res[r][1]
        assert rec is not None, res[r][0].stderr[-2000:]
        assert rec["err"] is not None and ("lost" in rec["err"] or "closed" in rec["err"] or "failed" in rec["err"])
        assert rec["later"] is not None and "broken" in rec["later"]


def test_closed_control_connection_is_detected():
    res = run("""
    bc.init(device="cpu")
    try:
        bc.allreduce(torch.ones(4), name="x")
        err = None
    except bc.CollectiveError as e:
        err = str(e)
    emit(err=err)
    """, nranks=2, env={"BC_TIMEOUT_S": "10", "BC_FAULT": "close_ctrl:rank=1:name=x"}, timeout=60, expect_ok=False)
    for r, rec in res:
        assert rec is not None and rec["err"] is not None


@pytest.mark.parametrize("transport", ["shm", "ring"])
def test_rank_exit_inside_the_data_phase_is_detected(transport):
    # Rank 2 leaves after the go-ahead, when the others are already exchanging data: over sockets
    # they see the closed connection, in shared memory the waiting ranks notice that the process
    # is gone. Either way well before the 60 s deadline.
    env = {"BC_TIMEOUT_S": "60", "BC_FAULT": "exit_in_collective:rank=2:name=doomed"}
    if transport == "ring":
        env["BC_SHM"] = "0"
    t0 = time.time()
    res = run("""
    import time
    bc.init(device="cpu")
    bc.allreduce(torch.ones(4), name="warm")
    t0 = time.time()
    try:
        bc.allreduce(torch.ones(100000), name="doomed")
        err = None
    except bc.CollectiveError as e:
        err = str(e)
    emit(err=err, seconds=time.time() - t0)
    """, nranks=3, env=env, timeout=100, expect_ok=False)
    assert res[2][0].returncode == 42            # the injected exit
    for r in (0, 1):
        rec = res[r][1]
        assert rec is not None, res[r][0].stderr[-2000:]
        assert rec["err"] is not None and rec["seconds"] < 20, rec


def test_survivors_form_a_new_group_after_a_rank_is_lost():
    # Rank 2 ends inside a collective. The others get an error, shut the broken group down and
    # start a group of two in the same processes (same rendezvous port), which works.
    res = run("""
    bc.init(device="cpu")
    bc.allreduce(torch.ones(4), name="warm")
    try:
        bc.allreduce(torch.ones(1000), name="doomed")
        err = None
    except bc.CollectiveError as e:
        err = str(e)
    broken = bc.is_broken()
    bc.shutdown()
    bc.init(device="cpu", rank=RANK, size=2)
    broken = broken and not bc.is_broken()
    s = bc.allreduce(torch.arange(3.0) + RANK, average=False, name="again")
    g = bc.allgather(torch.full((1, 1), float(RANK)))
    emit(err=err, size=bc.size(), s=s.tolist(), g=g.flatten().tolist(), broken=broken)
    bc.shutdown()
    """, nranks=3, env={"BC_TIMEOUT_S": "30", "BC_FAULT": "exit_in_collective:rank=2:name=doomed"}, timeout=100, expect_ok=False)
    assert res[2][0].returncode == 42
    for r in (0, 1):
        rec = res[r][1]
        assert rec is not None, res[r][0].stderr[-2000:]
        assert rec["err"] is not None and rec["broken"] and rec["size"] == 2 and rec["s"] == [1.0, 3.0, 5.0] and rec["g"] == [0.0, 1.0]


def test_fault_specs_are_parsed_or_refused():
    # Any text is either a fault specification or an error; a specification that names another
    # rank or another collective leaves this one alone.
    res = run("""
    from hypothesis import given, settings, strategies as st
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"): os.environ.pop(k, None)
    bc.init(device="cpu")
    outcomes = {"ok": 0, "refused": 0}
    @settings(max_examples=300, deadline=None)
    @given(st.text(alphabet="abcdefghijklmnopqrstuvwxyz_=:0123456789-", max_size=40))
    def check(text):
        try:
            bc.set_fault(text)
            outcomes["ok"] += 1
        except bc.CollectiveError as e:
            assert "unknown fault kind" in str(e)
            outcomes["refused"] += 1
    check()
    bc.set_fault("exit_before:rank=5:name=elsewhere")
    bc.set_fault("drop_request:name=other")
    s = bc.allreduce(torch.ones(3), name="mine")
    bc.set_fault("")
    emit(outcomes=outcomes, s=s.tolist())
    bc.shutdown()
    """, nranks=1)
    rec = res[0][1]
    assert rec["s"] == [1.0, 1.0, 1.0] and rec["outcomes"]["ok"] >= 1 and rec["outcomes"]["refused"] >= 1


@pytest.mark.parametrize("chunk_kb", ["0", "16"])
def test_rank_exit_inside_a_two_level_allreduce_is_detected(chunk_kb):
    # Two hosts of two ranks (one machine, made-up host names). Rank 3 leaves after the go-ahead of
    # a large allreduce: its neighbour in shared memory notices that the process is gone, its
    # partner on the rail sees the closed connection, and the failure reaches the remaining rank
    # through them. With chunks ("16": tensors from 64 KiB on go chunk by chunk, the step between
    # the hosts on a helper thread) the helper's error must surface on the thread that waits for it,
    # and a thread that gives up must not leave the helper behind. Well before the 60 s deadline.
    env = {r: {"BC_HOSTNAME": f"host{r // 2}", "LOCAL_RANK": "-1", "BC_TIMEOUT_S": "60", "BC_TWO_LEVEL_CHUNK_KB": chunk_kb,
               "BC_FAULT": "exit_in_collective:rank=3:name=doomed"} for r in range(4)}
    res = run("""
    import time
    bc.init(device="cpu")
    bc.allreduce(torch.ones(50000), name="warm")
    t0 = time.time()
    try:
        bc.allreduce(torch.ones(100000), name="doomed")
        err = None
    except bc.CollectiveError as e:
        err = str(e)
    emit(err=err, seconds=time.time() - t0, nodes=bc.n_nodes())
    """, nranks=4, per_rank_env=env, timeout=150, expect_ok=False)
    assert res[3][0].returncode == 42            # the injected exit
    for r in (0, 1, 2):
        rec = res[r][1]
        assert rec is not None, res[r][0].stderr[-2000:]
        assert rec["nodes"] == 2 and rec["err"] is not None and rec["seconds"] < 30, rec
