"""Utilities that need no GPU: the clock sampler against a fake NVML, the timeline export."""
import sys
import time
import types


def test_clock_sampler_reads_nvml(monkeypatch):
    fake = types.ModuleType("pynvml")
    fake.NVML_CLOCK_SM = 1
    calls = {"n": 0}
    fake.nvmlInit = lambda: None
    fake.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    fake.nvmlDeviceGetMaxClockInfo = lambda h, k: 1965

    def clock(h, k):
        calls["n"] += 1
        return 1200 + 10 * (calls["n"] % 3)

    fake.nvmlDeviceGetClockInfo = clock
    fake.nvmlDeviceGetPowerUsage = lambda h: 950000
    fake.nvmlDeviceGetCurrentClocksEventReasons = lambda h: 0x4        # sw_power_cap only
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,5")
    from tensorflow_allreduce_b200.utils.clocks import ClockSampler

    with ClockSampler(1, nvml_period_ms=5) as c:
        time.sleep(0.1)
    s = c.summary()
    assert c.source == "nvml" and s["source"] == "nvml"
    assert s["samples"] >= 5 and s["sm_max_mhz"] == 1965 and 1200 <= s["sm_mhz"] <= 1220
    assert s["reasons"] == ["sw_power_cap"] and abs(s["power_w_max"] - 950.0) < 1e-6
    assert c.samples[0][0] == "5"                                       # CUDA ordinal 1 -> NVML index 5


def test_bus_bandwidth_arithmetic():
    # allreduce: bytes / time * 2 (P - 1) / P; allgather: total bytes / time * (P - 1) / P
    from tensorflow_allreduce_b200.core import bus_gbs

    assert abs(bus_gbs("allreduce", 1 << 30, 8, 2.4e-3) - (1 << 30) / 2.4e-3 * 1.75 / 1e9) < 1e-9
    assert abs(bus_gbs("allreduce", 64 << 20, 2, 1e-3) - (64 << 20) / 1e-3 / 1e9) < 1e-9
    assert abs(bus_gbs("allgather", 1 << 20, 4, 1e-4) - (1 << 20) / 1e-4 * 0.75 / 1e9) < 1e-9
    assert bus_gbs("allreduce", 1 << 20, 1, 1e-3) == 0.0 and bus_gbs("allreduce", 1 << 20, 8, 0.0) == 0.0


def test_timeline_export():
    from tensorflow_allreduce_b200.utils import timeline

    recs = [{"name": "a", "op": "allreduce", "algo": "nvls", "blocks": 64, "bytes": 1 << 20, "device": 1,
             "t_enqueue": 1.0, "t_negotiated": 1.0002, "t_done": 1.0003},
            {"name": "b", "op": "allgather", "algo": "cpu_ring", "blocks": 0, "bytes": 100, "device": 0,
             "t_enqueue": 1.001, "t_negotiated": 1.0012, "t_done": 1.002}]
    ev = timeline.chrome_trace(recs, pid=0)
    assert len(ev) == 4 and ev[0]["cat"] == "allreduce.negotiate" and ev[1]["cat"] == "allreduce.launch" and ev[3]["cat"] == "allgather.run"
    assert abs(ev[0]["dur"] - 200.0) < 1e-3
    s = timeline.summary(recs)
    assert s["allreduce/nvls"]["calls"] == 1 and s["allgather/cpu_ring"]["bytes"] == 100
    # an allreduce in two levels shows its three steps back to back
    two = dict(recs[0], name="c", two_level_s=[1e-4, 3e-4, 2e-4])
    steps = [e for e in timeline.chrome_trace([two], pid=0) if e["cat"] == "allreduce.two_level"]
    assert [e["name"] for e in steps] == ["inside the host", "rail between hosts", "gather inside the host"]
    assert abs(steps[1]["ts"] - steps[0]["ts"] - 100.0) < 1e-3 and abs(steps[2]["dur"] - 200.0) < 1e-3
    # a record that was timed on the device adds a span of that length on the lane of its channel
    timed = dict(recs[0], name="fused_step", device_us=250.0, channel=1, bus_gbs=512.0, link_frac=0.67)
    dev = [e for e in timeline.chrome_trace([timed], pid=0) if e["cat"] == "allreduce.device"]
    assert len(dev) == 1 and dev[0]["tid"] == 11 and dev[0]["dur"] == 250.0 and dev[0]["args"]["bus_gbs"] == 512.0
    s = timeline.summary(recs + [timed])
    assert s["allreduce/nvls"]["calls"] == 2 and s["allreduce/nvls"]["device_timed"] == 1 and s["allreduce/nvls"]["device_us"] == 250.0


def test_launcher_starts_ranks_and_propagates_failure(tmp_path):
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "job.py"
    script.write_text(
        "import os, sys\n"
        f"sys.path.insert(0, {root!r})\n"
        "import torch, tensorflow_allreduce_b200 as bc\n"
        "with bc.Session(device='cpu'):\n"
        "    s = bc.allreduce(torch.tensor([float(bc.rank() + 1)]), average=False)\n"
        "    me = bc.rank()\n"
        "    sys.stdout.write(f'SUM {me} {bc.size()} {bc.local_rank()} {s.item()}\\n'); sys.stdout.flush()\n"
        "sys.exit(int(sys.argv[1]) if me == 1 else 0)\n")
    cmd = [sys.executable, "-m", "tensorflow_allreduce_b200.launch", "--nproc", "3", "--cpu", str(script)]
    ok = subprocess.run(cmd + ["0"], cwd=root, capture_output=True, text=True, timeout=120)
    assert ok.returncode == 0, ok.stderr[-2000:]
    lines = sorted(l for l in ok.stdout.splitlines() if l.startswith("SUM"))
    assert lines == [f"SUM {r} 3 {r} 6.0" for r in range(3)]
    bad = subprocess.run(cmd + ["7"], cwd=root, capture_output=True, text=True, timeout=120)
    assert bad.returncode == 7


def test_stats_jsonl_is_written_at_shutdown(tmp_path):
    import json

    from _util import run

    path = str(tmp_path / "stats.{rank}.jsonl")
    run("""
    bc.init(device="cpu")
    bc.allreduce(torch.ones(100), name="x")
    bc.allgather(torch.ones(RANK + 1, 2), name="y")
    bc.shutdown()
    emit(ok=True)
    """, nranks=2, env={"BC_STATS_JSONL": path})
    for r in range(2):
        recs = [json.loads(l) for l in open(path.replace("{rank}", str(r)))]
        names = {e["name"]: e for e in recs}
        assert names["x"]["op"] == "allreduce" and names["x"]["bytes"] == 400 and names["x"]["rank"] == r
        assert names["y"]["op"] == "allgather" and names["y"]["algo"] == "cpu_shm" and names["y"]["device"] == "cpu"


def test_gru_workspace_size_and_dimension_checks(native_lib):
    # Pure host arithmetic of the persistent GRU entry points (no GPU needed): the exchange
    # workspace of the benchmark shape, and dimensions that the kernels do not take.
    assert native_lib.bc_gru_workspace_bytes(350, 32, 1024, 2) == 2 * 64 * 16 * 32 * 16 * 4     # backward groups of 16
    assert native_lib.bc_gru_workspace_bytes(10, 4, 128, 1) == 8 * 4 * 32 * 48 * 4             # forward groups of 4
    for T, B, H, nd in ((10, 33, 128, 2), (10, 8, 100, 1), (10, 8, 2048, 2), (5000, 8, 128, 1), (10, 8, 128, 3)):
        assert native_lib.bc_gru_workspace_bytes(T, B, H, nd) == 0
        assert native_lib.bc_gru_supported(0, T, B, H, nd) == 0


def test_runner_kills_an_overstaying_rank_and_keeps_its_stacks():
    # Rank 1 never finishes: the runner reports it with returncode None and its Python stacks
    # (the scripts register faulthandler on SIGUSR1), rank 0 is unaffected.
    from _util import run

    t0 = time.time()
    res = run("""
    import time
    def stuck_here():
        time.sleep(600)
    if RANK == 1:
        stuck_here()
    emit(done=True)
    """, nranks=2, timeout=8, expect_ok=False)
    assert time.time() - t0 < 60
    (r0, rec0), (r1, rec1) = res
    assert r0.returncode == 0 and rec0 == {"done": True}
    assert r1.returncode is None and rec1 is None
    assert "stuck_here" in r1.stderr


def test_free_port_avoids_the_ephemeral_range():
    from tensorflow_allreduce_b200.utils.spawn import free_port

    low = int(open("/proc/sys/net/ipv4/ip_local_port_range").read().split()[0])
    ports = {free_port() for _ in range(8)}
    if low > 21000:
        assert all(20000 <= p < low for p in ports)
    assert len(ports) > 1


def test_one_launcher_per_host_forms_one_job(tmp_path):
    # Two launchers (node-rank 0 and 1) on this machine, each reporting a host name of its own:
    # 2 hosts x 2 ranks, global ranks 0..3, and the collectives run in two levels.
    import os
    import subprocess

    from tensorflow_allreduce_b200.utils.spawn import free_port

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "job.py"
    script.write_text(
        "import os, sys\n"
        f"sys.path.insert(0, {root!r})\n"
        "import torch, tensorflow_allreduce_b200 as bc\n"
        "with bc.Session(device='cpu'):\n"
        "    s = bc.allreduce(torch.arange(5.0) + bc.rank(), average=False)\n"
        "    sys.stdout.write(f'JOB {bc.rank()} {bc.size()} {bc.local_rank()} {bc.local_size()} {bc.n_nodes()} {bc.node_index()} {s.tolist()}\\n')\n"
        "    sys.stdout.flush()\n")
    port = str(free_port())
    procs = []
    for node in range(2):
        env = dict(os.environ, BC_HOSTNAME=f"host{node}", BC_TIMEOUT_S="60")
        cmd = [sys.executable, "-m", "tensorflow_allreduce_b200.launch", "--nnodes", "2", "--node-rank", str(node),
               "--port", port, "--nproc", "2", "--cpu", str(script)]
        procs.append(subprocess.Popen(cmd, cwd=root, env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    lines = []
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err[-2000:]
        lines += [l for l in out.splitlines() if l.startswith("JOB")]
    want_sum = [float(4 * i + 6) for i in range(5)]
    assert sorted(lines) == [f"JOB {r} 4 {r % 2} 2 2 {r // 2} {want_sum}" for r in range(4)]


def test_ranks_started_by_torchrun_find_each_other(tmp_path):
    # Under torchrun MASTER_PORT belongs to the launcher's store: rank 0 publishes a port of its
    # own for the control plane through that store (core._resolve_port).
    import os
    import subprocess

    from tensorflow_allreduce_b200.utils.spawn import free_port

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "job.py"
    script.write_text(
        "import sys\n"
        f"sys.path.insert(0, {root!r})\n"
        "import torch, tensorflow_allreduce_b200 as bc\n"
        "bc.init(device='cpu')\n"
        "s = bc.allreduce(torch.ones(3) * (bc.rank() + 1), average=False)\n"
        "sys.stdout.write(f'TR {bc.rank()} {bc.size()} {bc.local_rank()} {s.tolist()}\\n'); sys.stdout.flush()\n"
        "bc.shutdown()\n")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", BC_TIMEOUT_S="60")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "3", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), str(script)]
    r = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stderr[-3000:]
    lines = sorted(l for l in r.stdout.splitlines() if l.startswith("TR"))
    assert lines == [f"TR {k} 3 {k} [6.0, 6.0, 6.0]" for k in range(3)]


def test_info_command_reports_and_checks():
    import json
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", BC_BUCKET_MB="8")
    r = subprocess.run([sys.executable, "-m", "tensorflow_allreduce_b200", "--check"], cwd=root, env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    info = json.loads(r.stdout)
    assert info["library_built"] and info["library_matches_sources"] and info["check"] == {"cpu": True}
    assert info["config"]["bucket_mb"] == 8.0 and info["environment"]["BC_BUCKET_MB"] == "8"


def test_bench_reference_arm_reports_unavailable():
    # The reference (a TensorFlow 1.3 fork) cannot be installed offline: its arm prints one JSON
    # line saying so and exits 0, also when every rank of a torchrun launch runs it.
    import json
    import os
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for rank in ("0", "1"):
        env = dict(os.environ, RANK=rank, WORLD_SIZE="2")
        r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "2", "--warmup", "3"],
                           cwd=root, env=env, capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr[-2000:]
        lines = [l for l in r.stdout.splitlines() if l.strip()]
        if rank == "0":
            rec = json.loads(lines[-1])
            assert rec["impl"] == "reference" and "unavailable" in rec and len(lines) == 1
        else:
            assert lines == []


def test_entry_point_build_leaves_both_libraries_current():
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    import __graft_entry__ as entry
    from tensorflow_allreduce_b200 import build

    entry.build()
    assert build.LIB.exists() and build.LIB_DEBUG.exists()
    assert not build.needs_build() and not build.needs_build(debug=True)
    assert callable(entry.smoke)


def test_chunks_by_bytes_partitions_in_order():
    import torch
    from hypothesis import given, settings, strategies as st

    from tensorflow_allreduce_b200.parallel.distributed_optimizer import _chunks_by_bytes

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.integers(min_value=0, max_value=50), max_size=30), st.integers(min_value=1, max_value=120))
    def check(sizes, limit):
        tensors = [torch.empty(n, dtype=torch.float32) for n in sizes]
        runs = list(_chunks_by_bytes(tensors, limit))
        flat = [t for run in runs for t in run]
        assert len(flat) == len(tensors) and all(a is b for a, b in zip(flat, tensors))      # same tensors, same order
        for i, run in enumerate(runs):
            size = sum(t.numel() * 4 for t in run)
            assert run and (size <= limit or len(run) == 1)                                    # only a lone tensor may exceed the limit
            if i + 1 < len(runs):                                                              # greedy: the next tensor did not fit
                assert size + runs[i + 1][0].numel() * 4 > limit

    check()


def test_symmetric_heap_allocator_never_overlaps_and_coalesces():
    # The first-fit allocator that sub-divides the symmetric heap, driven without a GPU: random
    # allocations and frees, blocks whose reuse waits for an event, and full recovery at the end.
    import random

    import torch

    from tensorflow_allreduce_b200.ops.symmetric import _ALIGN, _Heap

    class FakeEvent:
        def __init__(self):
            self.done = False
            self.waited = False

        def query(self):
            return self.done

        def synchronize(self):
            self.waited = self.done = True

    rng = random.Random(7)
    size = 64 * _ALIGN
    heap = _Heap(0, size, torch.device("cpu"))
    live = {}                                   # offset -> length (rounded)
    events = []
    for step in range(3000):
        if live and rng.random() < 0.45:
            off = rng.choice(sorted(live))
            length = live.pop(off)
            if rng.random() < 0.5:
                ev = FakeEvent()
                events.append(ev)
                heap.limbo.append((ev, off, length))          # reuse must wait for this event
            else:
                heap.release_later(off, length)               # no CUDA here: free at once
        else:
            nbytes = rng.choice([1, 100, _ALIGN, _ALIGN + 1, 5 * _ALIGN, 17 * _ALIGN])
            need = (nbytes + _ALIGN - 1) // _ALIGN * _ALIGN
            off = heap.alloc(nbytes)
            if off is None:
                # refused only when no hole fits, even after waiting for every pending free
                assert all(e.done for e in events)
                assert all(l < need for _, l in heap.free)
                continue
            assert off % _ALIGN == 0 and 0 <= off and off + need <= size
            for o, l in live.items():
                assert off + need <= o or o + l <= off, "overlapping blocks"
            live[off] = need
        if rng.random() < 0.1:
            for e in events:
                e.done = True
    for off, length in list(live.items()):
        heap.release_later(off, length)
    for e in events:
        e.done = True
    assert heap.alloc(size) == 0                # everything came back and merged into one hole


def test_algorithm_selector_table(native_lib):
    # The selector is a pure function, so the table it implements is checked without a GPU:
    # small separate outputs one-shot; floats from 512 KiB on NVLS when a multicast mapping exists
    # and the group has at least 4 ranks; everything else two-shot; forced choices fall back to
    # two-shot where they cannot apply.
    F32, I32, BF16 = 0, 1, 3
    ONE, TWO, NVLS = 1, 2, 3

    def sel(world, nbytes, dtype=F32, in_place=True, mc=True, force=0, one_max=-1, nvls_min=-1, use_nvls=1):
        return native_lib.bc_select_algo(world, nbytes, dtype, int(in_place), int(mc), force, one_max, nvls_min, use_nvls)

    assert sel(8, 4 << 10, in_place=False) == ONE and sel(8, 256 << 10, in_place=False) == ONE
    assert sel(8, (256 << 10) + 4, in_place=False, mc=False) == TWO
    assert sel(8, 4 << 10, in_place=True) == TWO                      # in place / fused: never one-shot
    assert sel(8, 512 << 10) == NVLS and sel(8, (512 << 10) - 4) == TWO and sel(4, 64 << 20, BF16) == NVLS
    assert sel(2, 256 << 20) == TWO                                   # two ranks: the switch saves nothing
    assert sel(2, 256 << 20, in_place=False) == ONE and sel(4, 256 << 20, in_place=False, mc=False) == TWO   # two ranks, separate output
    assert sel(8, 64 << 20, mc=False) == TWO and sel(8, 64 << 20, use_nvls=0) == TWO
    assert sel(8, 64 << 20, I32) == TWO                               # the switch adds floats only
    assert sel(8, 1 << 20, nvls_min=2 << 20) == TWO and sel(8, 1 << 20, in_place=False, one_max=1 << 20) == ONE
    assert sel(2, 1 << 20, force=NVLS) == NVLS and sel(8, 1 << 20, force=NVLS, mc=False) == TWO
    assert sel(8, 1 << 30, force=ONE, in_place=False) == ONE and sel(8, 1 << 20, force=ONE, in_place=True) == TWO
    assert sel(8, 4 << 10, in_place=False, force=TWO) == TWO
    # grid, per algorithm and group size (bytes, world, algo, fused, SMs, cap override, beside compute):
    blocks = native_lib.bc_choose_blocks
    # peer loads: one block per 32 KiB, at most 128 (two ranks: one per SM)
    assert blocks(1, 8, TWO, 0, 148, 0, 0) == 1 and blocks(32 << 10, 8, TWO, 0, 148, 0, 0) == 1 and blocks((32 << 10) + 1, 8, TWO, 0, 148, 0, 0) == 2
    assert blocks(1 << 30, 8, TWO, 0, 148, 0, 0) == 128 and blocks(1 << 30, 4, TWO, 0, 148, 0, 0) == 128 and blocks(1 << 30, 2, TWO, 0, 148, 0, 0) == 148
    assert blocks(256 << 10, 8, ONE, 0, 148, 0, 0) == 8 and blocks(64 << 20, 2, ONE, 0, 148, 0, 0) == 148
    # NVLS: one block per 64 KiB, at most 16 up to 256 MiB and 32 above (the switch does the work; few blocks issue it
    # best), with more than 4 ranks at most 64
    assert blocks(512 << 10, 4, NVLS, 0, 148, 0, 0) == 8 and blocks(1 << 20, 4, NVLS, 0, 148, 0, 0) == 16
    assert blocks(256 << 20, 4, NVLS, 0, 148, 0, 0) == 16 and blocks(512 << 20, 4, NVLS, 0, 148, 0, 0) == 32
    assert blocks(512 << 10, 8, NVLS, 0, 148, 0, 0) == 8 and blocks(2 << 20, 8, NVLS, 0, 148, 0, 0) == 32
    assert blocks(256 << 20, 8, NVLS, 0, 148, 0, 0) == 64 and blocks(1 << 30, 8, NVLS, 0, 148, 0, 0) == 64
    # a fused update wants every SM twice; beside the backward pass only what a 128-SM kernel leaves free
    assert blocks(1 << 30, 8, NVLS, 1, 148, 0, 0) == 296 and blocks(1 << 30, 8, NVLS, 1, 148, 0, 1) == 20
    assert blocks(1 << 30, 8, NVLS, 1, 132, 0, 1) == 8 and blocks(64 << 10, 8, TWO, 1, 148, 0, 1) == 2
    assert blocks(1 << 30, 8, TWO, 0, 148, 16, 0) == 16 and blocks(1 << 30, 8, NVLS, 1, 148, 24, 1) == 24


def test_gather_rounds_cover_every_slab_and_fit_the_staging_area(native_lib):
    import ctypes as C

    from hypothesis import given, settings, strategies as st

    @settings(max_examples=300, deadline=None)
    @given(st.lists(st.integers(min_value=0, max_value=5_000_000), min_size=1, max_size=8), st.integers(min_value=4096, max_value=1 << 20))
    def check(slabs, staging):
        world = len(slabs)
        arr = (C.c_ulonglong * world)(*slabs)
        pieces = (C.c_ulonglong * world)()
        rounds = native_lib.bc_plan_gather_rounds(world, arr, staging, pieces)
        assert rounds >= 1
        for p in range(world):
            assert pieces[p] % 16 == 0 and rounds * pieces[p] >= slabs[p]          # every byte of every slab gets its round
        for j in range(rounds):                                                     # what round j puts into the staging area
            total = sum(min(pieces[p], max(0, slabs[p] - j * pieces[p])) for p in range(world))
            assert total <= staging
        if rounds > 1:                                                              # no more rounds than the sizes call for
            assert sum(slabs) > (rounds - 1) * (staging - 16 * world)

    check()


def test_pipeline_plan_keeps_the_ring_inside_the_slice_and_the_copy_out_behind_the_copy_in(native_lib):
    # The staged pipeline kernel's cut of a tensor is a pure function of the size and the
    # settings (every rank must arrive at the same one): chunks are multiples of 4 KiB, the ring
    # fits the channel's slice, a tensor has at least eight chunks where its size allows, and a
    # slot is copied out before the chunk that follows in it is copied in.
    import ctypes as C

    from hypothesis import given, settings, strategies as st

    @settings(max_examples=300, deadline=None)
    @given(st.integers(min_value=16, max_value=1 << 34), st.integers(min_value=21, max_value=30),
           st.sampled_from([0, 64 << 10, 1 << 20, 8 << 20]), st.sampled_from([0, 2, 4, 16, 64]), st.integers(min_value=1, max_value=4))
    def check(nbytes, slice_log2, chunk, slots, groups):
        out = (C.c_longlong * 4)()
        assert native_lib.bc_plan_pipeline(nbytes, 1 << slice_log2, chunk, slots, groups, 0, out) == 0
        chunk_bytes, nchunks, nslots, lag = out[0], out[1], out[2], out[3]
        ring = max((slots or 16) // groups * groups, 2 * groups)             # slots asked for, in whole groups
        assert chunk_bytes >= 4096 and chunk_bytes % 4096 == 0 and chunk_bytes <= min(chunk or 8 << 20, 4 << 20)
        assert 1 <= nchunks <= 2048 and 1 <= nslots <= ring and nslots <= nchunks
        assert nslots * chunk_bytes <= 1 << slice_log2
        assert nchunks * chunk_bytes >= nbytes or nchunks == 2048          # one launch covers it, or the caller launches again
        assert lag >= groups and lag % groups == 0
        if nchunks > nslots:                                               # the ring wraps: a slot keeps its group of copiers
            assert nslots % groups == 0 and lag < nslots
        if nbytes >= 8 * (64 << 10) and min(chunk or 8 << 20, 4 << 20) >= 64 << 10 and nbytes // 8 <= (1 << slice_log2) // ring:
            assert nchunks >= 8

    check()
    out = (C.c_longlong * 4)()
    native_lib.bc_plan_pipeline(64 << 20, 256 << 20, 0, 0, 0, 0, out)
    assert list(out) == [4 << 20, 16, 16, 8]
    native_lib.bc_plan_pipeline(1 << 30, 256 << 20, 0, 0, 0, 0, out)
    assert list(out) == [4 << 20, 256, 16, 8]
    native_lib.bc_plan_pipeline(4 << 20, 256 << 20, 0, 0, 0, 0, out)
    assert list(out) == [512 << 10, 8, 8, 8]
    # streaming reducers: chunks are whole steps of all ranks' reducer blocks (4 ranks x 16 blocks x 512 threads x
    # 4 packs = 2 MiB): a 64th of the tensor, at least two steps, at most 8 MiB
    unit = 4 * 16 * 512 * 4 * 16
    native_lib.bc_plan_pipeline(1 << 30, 256 << 20, 0, 0, 0, unit, out)
    assert list(out) == [8 << 20, 128, 16, 8]
    native_lib.bc_plan_pipeline(256 << 20, 256 << 20, 0, 0, 0, unit, out)
    assert list(out) == [4 << 20, 64, 16, 8]
    native_lib.bc_plan_pipeline(64 << 20, 256 << 20, 0, 0, 0, unit, out)
    assert list(out) == [4 << 20, 16, 16, 8]
    native_lib.bc_plan_pipeline(4 << 20, 256 << 20, 0, 0, 0, unit, out)
    assert list(out) == [4 << 20, 1, 1, 8]
    native_lib.bc_plan_pipeline(1 << 30, 256 << 20, 0, 0, 0, 4 * unit, out)      # two steps win over the 8 MiB cap
    assert list(out) == [16 << 20, 64, 16, 8]
    native_lib.bc_plan_pipeline(1 << 30, 8 << 20, 0, 0, 0, unit, out)            # a slice that cannot hold the ring: no plan
    assert out[1] == 0


def test_static_allreduce_refuses_bad_requests_before_touching_a_device(native_lib):
    # Every refusal of bc_group_allreduce_static is decided on the host before the first CUDA
    # call, so the checks run here with made-up addresses: a count whose byte size would wrap
    # around to zero, too many ranks, overlapping byte ranges, a missing status word.
    import ctypes as C

    fn = native_lib.bc_group_allreduce_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_longlong, C.c_int, C.c_float, C.c_int,
                   C.c_void_p, C.c_void_p, C.c_char_p, C.c_int]

    def call(ins, outs, count, dtype=0, status=0x1000):
        n = len(ins)
        err = C.create_string_buffer(512)
        rc = fn(n, (C.c_void_p * n)(*ins), (C.c_void_p * n)(*outs), count, dtype, 1.0, 1,
                C.c_void_p(status) if status else None, None, err, len(err))
        return rc, err.value.decode()

    ins, outs = [0x10000, 0x20000], [0x30000, 0x40000]
    for dtype, count in ((0, 1 << 61), (0, 1 << 62), (2, 1 << 61), (6, (1 << 63) - 1), (0, (1 << 18) + 1)):
        rc, err = call(ins, outs, count, dtype)
        assert rc == -1 and "exceeds the static scratch limit" in err, (dtype, count, err)
    assert call(ins * 5, outs * 5, 16) == (-1, "nranks must be between 1 and 8")
    rc, err = call(ins, [0x10020, 0x40000], 16)
    assert rc == -1 and "aliases an input" in err
    rc, err = call(ins, [0x30000, 0x30010], 16)
    assert rc == -1 and "two outputs alias" in err
    rc, err = call(ins, outs, 16, status=0)
    assert rc == -1 and "status_out" in err
    rc, err = call(ins, outs, 16, dtype=99)
    assert rc == -1 and "dtype" in err
    rc, err = call(ins, [0x30004, 0x40000], 16)
    assert rc == -1 and "aligned" in err


def test_bucket_plan_covers_every_parameter_once_and_cuts_on_pack_boundaries():
    # plan_buckets is pure arithmetic: random units (single parameters and shared storages with
    # gaps), checked for disjoint ranges, full coverage, 16-byte aligned starts and sizes.
    from hypothesis import given, settings, strategies as st

    from tensorflow_allreduce_b200.parallel.distributed_optimizer import plan_buckets

    member = st.tuples(st.integers(min_value=1, max_value=5000), st.integers(min_value=0, max_value=40))   # (numel, gap after it)
    unit = st.lists(member, min_size=1, max_size=12)

    @settings(max_examples=300, deadline=None)
    @given(st.lists(unit, min_size=1, max_size=8), st.sampled_from([2, 4]), st.integers(min_value=64, max_value=20000), st.randoms())
    def check(raw, esize, bucket_bytes, rnd):
        units, reg, sizes = [], 0, {}
        for ui, ms in enumerate(raw):
            members, off = [], 0
            regs = list(range(reg, reg + len(ms)))
            reg += len(ms)
            if len(ms) > 2:
                rnd.shuffle(regs)                       # storage order need not be registration order
            for (n, gap), r in zip(ms, regs):
                key = (ui, len(members))
                members.append((key, off, n, r))
                sizes[key] = n
                off += n + gap
            units.append((off, members))
        total, placements, ranges = plan_buckets(units, esize, bucket_bytes)
        assert len(placements) == len(units) and all(p * esize % 256 == 0 for p in placements)
        where = {}
        for lo, hi, slots in ranges:
            assert 0 <= lo < hi <= total and lo * esize % 16 == 0 and slots
            for key, o in slots:
                assert key not in where
                assert 0 <= o and o + sizes[key] <= hi - lo
                where[key] = (lo + o, lo + o + sizes[key])
        assert set(where) == set(sizes)                                  # every parameter in exactly one range
        spans = sorted((lo, hi) for lo, hi, _ in ranges)
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))      # ranges do not overlap
        for (numel, members), p in zip(units, placements):               # parameters keep their place inside a unit
            for key, o, n, _ in members:
                assert where[key] == (p + o, p + o + n)

    check()


def test_bucket_plan_of_a_recurrent_stack_follows_the_layers():
    # Five bidirectional GRU layers of 1024 in one flat storage (as after flatten_parameters()),
    # in two storage orders: parameters of a layer together, or all matrices first and all bias
    # vectors last. Either way every layer-direction becomes one range of its own, launched in
    # the order in which backward finishes the layers, and no matrix range waits for a vector of
    # an earlier layer.
    from tensorflow_allreduce_b200.parallel.distributed_optimizer import plan_buckets

    names, reg = [], 0
    for layer in range(5):
        inp = 1312 if layer == 0 else 2048
        for d in range(2):
            for kind, n in (("w_ih", 3072 * inp), ("w_hh", 3072 * 1024), ("b_ih", 3072), ("b_hh", 3072)):
                names.append(((layer, d, kind), n, reg))
                reg += 1
    for biases_last in (False, True):
        order = names if not biases_last else [m for m in names if m[0][2][0] == "w"] + [m for m in names if m[0][2][0] == "b"]
        members, off = [], 0
        for key, n, r in order:
            members.append((key, off, n, r))
            off += n
        total, placements, ranges = plan_buckets([(off, members)], 4, 32 << 20)
        assert total == off and placements == [0]
        matrix_ranges = [r for r in ranges if any(k[2][0] == "w" for k, _ in r[2])]
        assert len(matrix_ranges) == 10
        for i, (lo, hi, slots) in enumerate(matrix_ranges):
            layers = {(k[0], k[1]) for k, _ in slots}
            assert layers == {(4 - i // 2, 1 - i % 2)}                   # layer 4 reverse first, layer 0 forward last
            assert (hi - lo) * 4 <= 40 << 20
        assert len(ranges) == (11 if biases_last else 10)


def test_settings_come_from_the_environment_and_overrides(monkeypatch):
    # Every field of Config has a BC_* variable; overrides given in code win over the environment,
    # None leaves a field alone. The staged pipeline's defaults are the conservative ones: on where
    # the switch reduces, from 96 MiB, copiers sized by the library (0 = half of the SMs).
    from tensorflow_allreduce_b200.config import Config

    for name in ("BC_STAGED_PIPELINE", "BC_PIPELINE_MIN_MB", "BC_PIPELINE_COPIERS", "BC_PIPELINE_CGROUPS", "BC_STAGING_MB", "BC_NVLS"):
        monkeypatch.delenv(name, raising=False)
    c = Config.from_env()
    assert (c.staged_pipeline, c.pipeline_min_mb, c.pipeline_copiers, c.pipeline_cgroups, c.pipeline_streaming) == (1, 96, 0, 4, True)
    assert c.staging_mb == 1024 and c.nvls is True
    monkeypatch.setenv("BC_STAGED_PIPELINE", "2")
    monkeypatch.setenv("BC_PIPELINE_COPIERS", "128")
    monkeypatch.setenv("BC_PIPELINE_MIN_MB", "48")
    monkeypatch.setenv("BC_PIPELINE_STREAMING", "0")
    monkeypatch.setenv("BC_STAGING_MB", "64")
    monkeypatch.setenv("BC_NVLS", "0")
    c = Config.from_env(staging_mb=None, heap_mb=512)
    assert (c.staged_pipeline, c.pipeline_copiers, c.pipeline_min_mb, c.pipeline_streaming) == (2, 128, 48, False)
    assert c.staging_mb == 64 and c.heap_mb == 512 and c.nvls is False
    assert Config.from_env(staging_mb=8).staging_mb == 8


def test_sweep_tables_show_every_arm_and_the_best_of_this_library():
    # bench/sweep_collectives.py renders its rows as markdown: one table per operation and dtype,
    # a time and a bandwidth column per arm that has numbers, the best of this library's arms as a
    # fraction of the measured and of the nominal link rate, and the correctness flags.
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench", "sweep_collectives.py")
    spec = importlib.util.spec_from_file_location("sweep_collectives", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    rows = [
        {"op": "allreduce", "dtype": "fp32", "bytes": 64 << 20, "ours_direct_ms": 0.1628, "ours_direct_busbw": 618.3,
         "ours_private_ms": 0.1821, "ours_private_busbw": 552.9, "ours_nopipeline_ms": 0.1929, "ours_nopipeline_busbw": 521.9,
         "nccl_ms": 0.18, "nccl_busbw": 548.1, "direct_correct": True, "private_correct": True, "nopipeline_correct": False},
        {"op": "allreduce", "dtype": "fp32", "bytes": 1 << 10, "ours_direct_ms": 0.0173, "ours_direct_busbw": 0.1, "nccl_busbw": 0.1},
        {"op": "allgather", "dtype": "bf16", "bytes": 255 << 20, "ours_direct_ms": 0.4, "ours_direct_busbw": 501.0, "nccl_padded_busbw": 345.0, "correct": True},
    ]
    text = mod.markdown(rows, 4)
    assert "### allreduce, 4 GPUs, fp32" in text and "### allgather, 4 GPUs, bf16" in text and "### allreduce, 4 GPUs, bf16" not in text
    head = [l for l in text.splitlines() if l.startswith("| bytes")][0]
    for col in ("ours_direct ms", "ours_private ms", "ours_nopipeline ms", "ours_direct GB/s", "nccl GB/s", "ours / 764", "ours / 900", "correct"):
        assert col in head, col
    assert "ours_staged" not in head                     # no numbers, no column
    line = [l for l in text.splitlines() if l.startswith("| 64 MiB")][0]
    assert "618.3" in line and "0.81" in line and "0.69" in line          # best arm / 764 and / 900
    assert "direct=ok" in line and "nopipeline=WRONG" in line
    assert [l for l in text.splitlines() if l.startswith("| 1 KiB")][0].count("-") >= 2      # arms without a number show a dash
    assert mod._size(255 << 20) == "255 MiB" and mod._size(1536) == "1.5 KiB" and mod._size(100) == "100 B"
