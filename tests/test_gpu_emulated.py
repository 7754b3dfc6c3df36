"""The production kernels on ONE GPU with 2/4/8 emulated ranks, against plain PyTorch fp32
references. Counterpart of the reference's GPU allreduce/allgather tests
(tensorflow/contrib/mpi_collectives/mpi_ops_test.py:114-156, 204-263), which need one GPU per rank."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.float64, torch.uint8]
PACK = {torch.float32: 4, torch.bfloat16: 8, torch.float16: 8, torch.int32: 4, torch.int64: 2, torch.float64: 2, torch.uint8: 16}


def _fill(dtype, n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, generator=g, device="cuda") * 2 - 1).to(dtype)
    if dtype == torch.uint8:
        return torch.randint(0, 16, (n,), generator=g, device="cuda", dtype=torch.int32).to(dtype)
    return torch.randint(-1000, 1000, (n,), generator=g, device="cuda", dtype=dtype)


def _reference_sum(xs, dtype, scale=1.0, idiv=1):
    """Sum in rank order; 16-bit floats accumulate in fp32 and round once (as the kernels do)."""
    if dtype in (torch.bfloat16, torch.float16):
        acc = xs[0].float()
        for x in xs[1:]:
            acc = acc + x.float()
        return (acc * scale).to(dtype)
    acc = xs[0].clone()
    for x in xs[1:]:
        acc = acc + x
    if dtype.is_floating_point:
        return acc * torch.tensor(scale, dtype=dtype, device=acc.device) if dtype == torch.float64 else acc * scale
    if idiv > 1:
        return torch.div(acc, idiv, rounding_mode="trunc").to(dtype)
    return acc


@pytest.fixture(scope="module")
def emu():
    from tensorflow_allreduce_b200.ops.emulated import EmulatedGroup

    groups = {}

    def get(n, nbytes=8 << 20):
        key = (n, nbytes)
        if key not in groups:
            groups[key] = EmulatedGroup(n, nbytes)
        return groups[key]

    yield get
    # Guard regions around every emulated buffer and signal pad: no kernel of this module may
    # have stored out of bounds (sizes 0 .. a few packs, odd tails, every dtype and algorithm).
    damaged = {k: g.damaged_guard_bytes() for k, g in groups.items()}
    for g in groups.values():
        g.close()
    assert all(v == 0 for v in damaged.values()), damaged


@pytest.mark.parametrize("nranks", [2, 4, 8])
@pytest.mark.parametrize("algo", ["one_shot", "two_shot"])
@pytest.mark.parametrize("dtype", DTYPES)
def test_allreduce_matches_reference(emu, nranks, algo, dtype):
    g = emu(nranks)
    e = PACK[dtype]
    sizes = [0, 1, e - 1, e, e + 1, 3 * e * nranks + 5, 4096 + 3, (1 << 18) + 7]
    for n in sizes:
        bufs = [g.buffer(r, dtype, max(n, 1)) for r in range(nranks)]
        xs = [_fill(dtype, n, 100 * r + 7) for r in range(nranks)]
        for r in range(nranks):
            bufs[r][:n].copy_(xs[r])
        want = _reference_sum(xs, dtype)
        if algo == "one_shot":
            outs = [torch.empty(max(n, 1), dtype=dtype, device="cuda") for _ in range(nranks)]
            g.allreduce(n, dtype, "one_shot", outs=outs, blocks=3)
            got = [o[:n] for o in outs]
            # one-shot must leave the inputs untouched
            for r in range(nranks):
                assert torch.equal(bufs[r][:n], xs[r])
        else:
            g.allreduce(n, dtype, "two_shot", blocks=3)
            got = [b[:n] for b in bufs]
        torch.cuda.synchronize()
        assert g.status == 0
        for r in range(nranks):
            assert torch.equal(got[r], want), f"rank {r} n={n} {dtype} {algo}"


@pytest.mark.parametrize("nranks", [2, 3, 8])
@pytest.mark.parametrize("algo", ["one_shot", "two_shot"])
@pytest.mark.parametrize("op", ["prod", "min", "max"])
def test_prod_min_max_match_reference(emu, nranks, algo, op):
    g = emu(nranks)
    fn = {"prod": lambda a, b: a * b, "min": torch.minimum, "max": torch.maximum}[op]
    for dtype in (torch.float32, torch.bfloat16, torch.int32, torch.int64, torch.float64):
        e = PACK[dtype]
        for n in (1, e + 1, 3 * e * nranks + 5, (1 << 16) + 3):
            xs = [_fill(dtype, n, 100 * r + 11) for r in range(nranks)]
            if op == "prod" and not dtype.is_floating_point:
                xs = [x % 3 for x in xs]      # keep integer products small
            bufs = [g.buffer(r, dtype, n) for r in range(nranks)]
            for r in range(nranks):
                bufs[r][:n].copy_(xs[r])
            if dtype == torch.bfloat16:       # the kernels combine in fp32 and round once
                want = xs[0].float()
                for x in xs[1:]:
                    want = fn(want, x.float())
                want = want.to(dtype)
            else:
                want = xs[0].clone()
                for x in xs[1:]:
                    want = fn(want, x)
            if algo == "one_shot":
                outs = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(nranks)]
                g.allreduce(n, dtype, "one_shot", outs=outs, blocks=3, op=op)
                got = outs
            else:
                g.allreduce(n, dtype, "two_shot", blocks=3, op=op)
                got = [b[:n] for b in bufs]
            torch.cuda.synchronize()
            assert g.status == 0
            for r in range(nranks):
                assert torch.equal(got[r], want), f"rank {r} n={n} {dtype} {algo} {op}"


@pytest.mark.parametrize("nranks", [2, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_allreduce_exhaustive_small_sizes(emu, nranks, dtype):
    g = emu(nranks)
    e = PACK[dtype]
    for n in range(0, 4 * nranks * e + 1):
        xs = [_fill(dtype, n, 31 * r + n) for r in range(nranks)]
        bufs = [g.buffer(r, dtype, max(n, 1)) for r in range(nranks)]
        for r in range(nranks):
            bufs[r][:n].copy_(xs[r])
        g.allreduce(n, dtype, "two_shot", blocks=2, scale=1.0 / nranks)
        want = _reference_sum(xs, dtype, scale=1.0 / nranks)
        for r in range(nranks):
            assert torch.equal(bufs[r][:n], want), f"n={n} rank={r}"
    assert g.status == 0


def test_allreduce_average_and_separate_output(emu):
    g = emu(4)
    n = 10007
    for dtype, idiv in ((torch.float32, 1), (torch.int32, 4)):
        xs = [_fill(dtype, n, r) for r in range(4)]
        for r in range(4):
            g.buffer(r, dtype, n).copy_(xs[r])
        outs = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(4)]
        g.allreduce(n, dtype, "two_shot", outs=outs, scale=0.25, idiv=idiv, blocks=5)
        want = _reference_sum(xs, dtype, scale=0.25, idiv=idiv)
        for r in range(4):
            assert torch.equal(outs[r], want)


def test_allreduce_many_blocks_and_reuse(emu):
    # Back-to-back launches on the same pads: epochs must keep the barriers apart.
    g = emu(8, 16 << 20)
    n = (1 << 20) + 13
    blocks = min(16, g.max_blocks())
    for it in range(20):
        xs = [_fill(torch.float32, n, it * 10 + r) for r in range(8)]
        for r in range(8):
            g.buffer(r, torch.float32, n).copy_(xs[r])
        g.allreduce(n, torch.float32, "two_shot", blocks=blocks)
        want = _reference_sum(xs, torch.float32)
        assert torch.equal(g.buffer(3, torch.float32, n), want)
    assert g.status == 0


@pytest.mark.parametrize("nranks", [2, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("opt", ["sgd", "sgd_nesterov_wd", "adamw", "adam_l2", "adam_tf"])
def test_fused_update_matches_reference(emu, nranks, dtype, opt):
    from tensorflow_allreduce_b200.ops import fused_optim as fo

    g = emu(nranks)
    n = 5003
    torch.manual_seed(0)
    p0 = torch.randn(n, device="cuda")
    m0 = torch.randn(n, device="cuda") * 0.1
    v0 = torch.rand(n, device="cuda") * 0.01
    grads = [_fill(dtype, n, 5 + r) for r in range(nranks)]
    for r in range(nranks):
        g.buffer(r, dtype, n).copy_(grads[r])
    gavg = _reference_sum(grads, dtype, scale=1.0 / nranks).float()
    if dtype == torch.float32:
        params = [p0.clone() for _ in range(nranks)]
        masters = None
    else:
        params = [p0.to(dtype) for _ in range(nranks)]
        masters = [p0.clone() for _ in range(nranks)]
    s1 = [m0.clone() for _ in range(nranks)]
    s2 = [v0.clone() for _ in range(nranks)]
    if opt.startswith("sgd"):
        kw = dict(lr=0.1, momentum=0.9) if opt == "sgd" else dict(lr=0.05, momentum=0.8, weight_decay=0.01, nesterov=True)
        h = fo.sgd_hyper(zero_grad=True, **kw)
        want_p, want_m = fo.sgd_reference(p0, gavg, m0, **kw)
        want_v = v0
    else:
        kw = dict(lr=1e-2, step=3, weight_decay=0.1, decoupled=(opt != "adam_l2"), tf_epsilon_hat=(opt == "adam_tf"))
        h = fo.adam_hyper(zero_grad=True, **kw)
        want_p, want_m, want_v = fo.adam_reference(p0, gavg, m0, v0, **kw)
    g.fused_step(n, dtype, params, h, masters=masters, state1=s1, state2=s2, scale=1.0 / nranks, blocks=3)
    torch.cuda.synchronize()
    assert g.status == 0
    for r in range(nranks):
        fp32_p = params[r] if dtype == torch.float32 else masters[r]
        torch.testing.assert_close(fp32_p, want_p, rtol=1e-5, atol=1e-5)
        torch.testing.assert_close(s1[r], want_m, rtol=1e-5, atol=1e-6)
        if not opt.startswith("sgd"):
            torch.testing.assert_close(s2[r], want_v, rtol=2e-5, atol=1e-7)
        if dtype != torch.float32:
            assert torch.equal(params[r], masters[r].to(dtype))
        # every rank must hold bit-identical parameters, and the gradient must be zeroed
        assert torch.equal(fp32_p, params[0] if dtype == torch.float32 else masters[0])
        assert int(g.buffer(r, dtype, n).count_nonzero()) == 0


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_allgatherv_device_displacements(emu, nranks):
    g = emu(nranks)
    sizes = [17, 32, 81, 12, 15, 23, 22, 0][:nranks]
    for dtype, cols in ((torch.float32, 17), (torch.uint8, 3), (torch.int64, 1), (torch.bfloat16, 5)):
        ins = [(_fill(dtype, sizes[r] * cols, r + 1)) for r in range(nranks)]
        total = sum(sizes) * cols
        # every rank places its output at a different offset of its buffer (not symmetric on purpose)
        esize = ins[0].element_size()
        offs = [256 * (r + 1) + (esize * r if dtype == torch.uint8 else 0) for r in range(nranks)]
        for r in range(nranks):
            g.buffer(r, torch.uint8, g.bytes_per_rank).zero_()
        g.allgatherv(ins, offs, blocks=2)
        torch.cuda.synchronize()
        assert g.status == 0
        want = torch.cat(ins)
        for r in range(nranks):
            got = g.buffer(r, torch.uint8, total * esize, offset_bytes=offs[r]).clone().view(dtype)
            assert torch.equal(got, want), f"rank {r} {dtype}"


def test_bounded_wait_reports_status_and_returns():
    # One rank never arrives: the others give up after the limit, record a status word and the
    # kernel returns; the context stays usable.
    from tensorflow_allreduce_b200.ops.emulated import EmulatedGroup

    g = EmulatedGroup(4, 1 << 20)
    g.barrier_probe(absent=-1, timeout_s=5.0)
    torch.cuda.synchronize()
    assert g.status == 0
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    g.barrier_probe(absent=2, timeout_s=0.3)
    t1.record()
    torch.cuda.synchronize()
    st = g.status
    assert st & 0x80000000, hex(st)
    assert st & (1 << 2), hex(st)          # the missing peer is named
    assert 200 < t0.elapsed_time(t1) < 5000
    x = torch.ones(10, device="cuda") * 2  # the device still works
    assert float(x.sum()) == 20.0
    g.close()


@pytest.mark.parametrize("nranks", [2, 3, 8])
@pytest.mark.parametrize("algo", ["one_shot", "two_shot"])
def test_staged_inputs_are_copied_in_by_the_kernel(emu, nranks, algo):
    # The staged path of a real group: the inputs are private tensors, the kernel copies them into
    # the ranks' symmetric buffers before the first barrier and writes the result to separate
    # outputs. The buffers hold garbage beforehand; the private inputs must stay untouched.
    g = emu(nranks)
    for dtype in (torch.float32, torch.bfloat16, torch.int64, torch.uint8):
        e = PACK[dtype]
        for n, blocks in ((1, 1), (e - 1, 2), (e, 1), (5 * e * nranks + 3, 3), ((1 << 18) + 7, 4), ((1 << 18) + 7, 1)):
            xs = [_fill(dtype, n, 31 * r + n % 13) for r in range(nranks)]
            keep = [x.clone() for x in xs]
            for r in range(nranks):
                g.buffer(r, torch.uint8, max(n, 1) * torch.empty((), dtype=dtype).element_size()).fill_(0x5A)
            outs = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(nranks)]
            g.allreduce(n, dtype, algo, outs=outs, blocks=blocks, srcs=xs)
            torch.cuda.synchronize()
            assert g.status == 0
            want = _reference_sum(keep, dtype)
            for r in range(nranks):
                assert torch.equal(outs[r], want), f"rank {r} n={n} {dtype} {algo}"
                assert torch.equal(xs[r], keep[r])


def test_ranks_that_disagree_about_the_place_are_reported(emu):
    # An in-place reduction on symmetric memory assumes the tensor at the same offset on every
    # rank. Ordered launches cannot agree on that beforehand, so the kernel compares the offsets
    # the ranks pass: equal -> nothing happens; one differs -> the layout bit of the status word.
    g = emu(4)
    n = 5000
    for r in range(4):
        g.buffer(r, torch.float32, n).fill_(float(r + 1))
    g.allreduce(n, torch.float32, "two_shot", blocks=2, places=[4097] * 4)
    torch.cuda.synchronize()
    assert g.status == 0 and float(g.buffer(3, torch.float32, n)[n - 1]) == 10.0
    g.allreduce(n, torch.float32, "two_shot", blocks=2, places=[4097, 4097, 8193, 4097])
    torch.cuda.synchronize()
    assert g.status & 0x20000000, hex(g.status)
    assert not g.status & 0x80000000          # nobody waited in vain: the barriers still work
    g.clear_status()
    g.allreduce(n, torch.float32, "two_shot", blocks=2, places=[1] * 4)    # the group stays usable
    torch.cuda.synchronize()
    assert g.status == 0


def test_profile_stamps_are_ordered(emu):
    g = emu(8)
    n = 1 << 20
    stamps = torch.zeros(8, dtype=torch.int64, device="cuda")
    for algo, outs in (("two_shot", None), ("one_shot", [torch.empty(n, device="cuda") for _ in range(8)])):
        stamps.zero_()
        g.allreduce(n, torch.float32, algo, outs=outs, blocks=4, profile=stamps)
        torch.cuda.synchronize()
        t = stamps[:5].tolist()
        assert t[0] > 0 and all(b >= a for a, b in zip(t, t[1:])), t
        assert t[4] - t[0] < 1e9


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_mixed_grid_runs_the_cross_rank_phase_on_a_few_blocks(emu, nranks):
    # NVLS launches of real groups use a mixed grid: every block copies in and runs the local
    # epilogue, only the first few talk to the peers, and the blocks of a rank meet at two local
    # barriers in between. Same kernel code here with peer loads: staged inputs, separate outputs,
    # several launches in a row (the barrier counter runs on), then a fused update.
    g = emu(nranks)
    for dtype in (torch.float32, torch.bfloat16):
        e = PACK[dtype]
        for n, blocks, p1 in (((1 << 18) + 7, 6, 2), (5 * e * nranks + 3, 4, 1), ((1 << 16) + 1, 5, 3), (e - 1, 3, 1)):
            xs = [_fill(dtype, n, 77 * r + n % 11) for r in range(nranks)]
            keep = [x.clone() for x in xs]
            outs = [torch.empty(n, dtype=dtype, device="cuda") for _ in range(nranks)]
            g.allreduce(n, dtype, "two_shot", outs=outs, blocks=blocks, srcs=xs, phase1_blocks=p1)
            torch.cuda.synchronize()
            assert g.status == 0, hex(g.status)
            want = _reference_sum(keep, dtype)
            for r in range(nranks):
                assert torch.equal(outs[r], want), f"rank {r} n={n} {dtype}"
    # fused momentum-SGD with a mixed grid equals the same step with a plain grid
    from tensorflow_allreduce_b200.ops import fused_optim as fo

    n = (1 << 17) + 5
    results = []
    for p1 in (0, 2):
        grads = [_fill(torch.float32, n, 5 * r + 1) for r in range(nranks)]
        for r in range(nranks):
            g.buffer(r, torch.float32, n).copy_(grads[r])
        params = [torch.linspace(-1, 1, n, device="cuda") for _ in range(nranks)]
        mom = [torch.full((n,), 0.25, device="cuda") for _ in range(nranks)]
        g.fused_step(n, torch.float32, params, fo.sgd_hyper(0.1, momentum=0.9, weight_decay=0.01, zero_grad=True), state1=mom,
                     scale=1.0 / nranks, blocks=6, phase1_blocks=p1)
        torch.cuda.synchronize()
        assert g.status == 0
        results.append((params[0].clone(), mom[nranks - 1].clone()))
        assert float(g.buffer(0, torch.float32, n).abs().max()) == 0.0        # gradients zeroed
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


@pytest.mark.parametrize("nranks", [2, 4, 8])
def test_staged_pipeline_kernel_with_copier_and_reducer_blocks(emu, nranks):
    # Ordinary tensors of real groups go through ONE launch whose blocks have roles: copiers bring
    # chunks into a ring inside the staging area and finished chunks out again, reducers reduce
    # chunk after chunk, and progress words (not barriers) order them. Same kernel here with peer
    # loads: one chunk, a ring that is exactly full, a ring that wraps several times with a ragged
    # last chunk, in place and into separate outputs, launches in a row (the words run on), one
    # group of blocks per role or several that take every groups-th chunk each; reducer blocks that
    # drain after every chunk, and streaming ones (15 warps move data through ONE software pipeline
    # over all chunks, one warp polls the progress words and publishes; a group of 40 chunks takes
    # the block's ring of "done" counters around five times).
    g = emu(nranks)
    chunk = 4096
    packs_per_chunk = chunk // 16
    for dtype in (torch.float32, torch.bfloat16, torch.int32):
        e = PACK[dtype]
        for packs, slots, lag, red, cop, gr, gc in ((1, 4, 2, 2, 3, 1, 1), (packs_per_chunk - 1, 4, 2, 1, 1, 1, 1),
                                                    (4 * packs_per_chunk, 4, 2, 2, 3, 1, 1), (11 * packs_per_chunk + 37, 4, 2, 3, 2, 3, 2),
                                                    (7 * packs_per_chunk + 1, 2, 1, 2, 4, 2, 1), (3 * packs_per_chunk, 8, 5, 2, 2, 1, 1),
                                                    (29 * packs_per_chunk + 5, 8, 4, 4, 8, 4, 4), (2 * packs_per_chunk, 6, 3, 4, 6, 2, 3),
                                                    (13 * packs_per_chunk, 6, 3, 2, 3, 2, 3), (40 * packs_per_chunk - 9, 8, 4, 2, 4, 1, 4)):
            n = packs * e
            xs = [_fill(dtype, n, 31 * r + packs % 13) for r in range(nranks)]
            keep = [x.clone() for x in xs]
            scale, idiv = (1.0 / nranks, 1) if dtype.is_floating_point else (1.0, 1)
            want = _reference_sum(keep, dtype, scale=scale, idiv=idiv)
            outs = [torch.full((n,), 3, dtype=dtype, device="cuda") for _ in range(nranks)]
            kw = dict(scale=scale, idiv=idiv, chunk_bytes=chunk, slots=slots, lag=lag, reducers=red, copiers=cop, rgroups=gr, cgroups=gc)
            for streaming in (False, True):
                outs = [torch.full((n,), 3, dtype=dtype, device="cuda") for _ in range(nranks)]
                g.staged_pipeline(xs, outs, streaming=streaming, **kw)
                torch.cuda.synchronize()
                assert g.status == 0, hex(g.status)
                for r in range(nranks):
                    assert torch.equal(outs[r], want), f"rank {r} packs={packs} {dtype} streaming={streaming}"
                    assert torch.equal(xs[r], keep[r])
            g.staged_pipeline(xs, xs, streaming=True, **kw)
            torch.cuda.synchronize()
            assert g.status == 0, hex(g.status)
            for r in range(nranks):
                assert torch.equal(xs[r], want), f"in place: rank {r} packs={packs} {dtype}"
    # a ring that would be overwritten before it is copied out is refused on the host
    xs = [_fill(torch.float32, 64 * packs_per_chunk, r) for r in range(nranks)]
    with pytest.raises(RuntimeError):
        g.staged_pipeline(xs, xs, chunk_bytes=chunk, slots=2, lag=2)
    with pytest.raises(RuntimeError):                       # a slot would change hands between groups of copiers
        g.staged_pipeline(xs, xs, chunk_bytes=chunk, slots=5, lag=2, copiers=4, cgroups=2)
