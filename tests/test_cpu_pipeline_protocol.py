"""The synchronisation protocol of the staged pipeline kernel (csrc/cuda/staged_pipeline.cu) as a model
on the CPU: copier groups, reducer groups, the ring of slots and the progress words of every rank
as state machines that a random scheduler interleaves, with the words reaching each peer after a
delay of their own. What is checked is the design, not the CUDA code: with the ring sizes and lags
that the library's planner (`bc_plan_pipeline`, the real one) hands out, no agent ever reads a
slot that does not hold what it expects, nothing is overwritten while somebody still needs it,
nobody waits for ever, and every chunk leaves fully reduced.

The kernel has no counterpart in the reference, whose allreduce of a framework-owned tensor is one
copy followed by a ring with a stream synchronise per step
(tensorflow/contrib/mpi_collectives/ring.h:136-228)."""
import ctypes as C
import random

import pytest


class Hazard(AssertionError):
    pass


class Model:
    """P ranks. Rank r's ring: slots[r][s] = {"chunk": c, "share": [state per owner q]} with state
    "raw" (rank r's own input of chunk c) or "red" (the reduced share, written by its owner q)."""

    def __init__(self, P, nchunks, slots, lag, GR, GC, rng):
        self.P, self.N, self.S, self.lag, self.GR, self.GC, self.rng = P, nchunks, slots, lag, GR, GC, rng
        self.ring = [[None] * slots for _ in range(P)]
        # words as seen by rank `dst`: seen[dst][kind][group][src]; in flight: list of (dst, kind, group, src, value)
        self.seen = [[[[0] * P for _ in range(max(GR, GC))] for _ in range(2)] for _ in range(P)]
        self.flight = []
        self.out_done = [[False] * nchunks for _ in range(P)]
        self.agents = []
        for r in range(P):
            for g in range(GC):
                self.agents.append(self.copier(r, g))
            for g in range(GR):
                self.agents.append(self.reducer(r, g))

    def publish(self, src, kind, group, value):
        for dst in range(self.P):
            self.flight.append((dst, kind, group, src, value))

    def all_seen(self, me, kind, group, value):
        return all(self.seen[me][kind][group][q] >= value for q in range(self.P))

    # Agents are generators: they yield a predicate to wait for (or None to give up the turn).
    def copier(self, r, g):
        for ch in range(g, self.N + self.lag, self.GC):
            if ch < self.N:
                s = ch % self.S
                old = self.ring[r][s]
                if old is not None:
                    # the chunk that lived here must have left this rank, and no reducer may still want it
                    if not self.out_done[r][old["chunk"]]:
                        raise Hazard(f"rank {r}: chunk {ch} overwrites chunk {old['chunk']} before it was copied out")
                    if any(st != "red" for st in old["share"]):
                        raise Hazard(f"rank {r}: chunk {ch} overwrites a share of chunk {old['chunk']} that was never reduced")
                self.ring[r][s] = {"chunk": ch, "share": ["raw"] * self.P}
                yield None
                self.publish(r, 0, g, ch // self.GC + 1)
                yield None
            o = ch - self.lag
            if 0 <= o < self.N:
                yield lambda o=o: self.all_seen(r, 1, o % self.GR, o // self.GR + 1)
                slot = self.ring[r][o % self.S]
                if slot is None or slot["chunk"] != o or any(st != "red" for st in slot["share"]):
                    raise Hazard(f"rank {r}: copy-out of chunk {o} finds {slot}")
                self.out_done[r][o] = True
                yield None

    def reducer(self, q, g):
        for ch in range(g, self.N, self.GR):
            yield lambda ch=ch: self.all_seen(q, 0, ch % self.GC, ch // self.GC + 1)
            for r in range(self.P):              # load share q of every rank's slot
                slot = self.ring[r][ch % self.S]
                if slot is None or slot["chunk"] != ch or slot["share"][q] != "raw":
                    raise Hazard(f"rank {q}: reduction of chunk {ch} reads {slot} from rank {r}")
                yield None
            for r in range(self.P):              # store the result into every rank's slot
                slot = self.ring[r][ch % self.S]
                if slot is None or slot["chunk"] != ch:
                    raise Hazard(f"rank {q}: result of chunk {ch} lands on {slot} of rank {r}")
                slot["share"][q] = "red"
                yield None
            self.publish(q, 1, g, ch // self.GR + 1)
            yield None

    def run(self, max_steps=2_000_000):
        waiting = {}                 # agent -> predicate
        live = list(self.agents)
        steps = 0
        while live:
            steps += 1
            if steps > max_steps:
                raise Hazard("the model did not finish")
            # deliver a word, or move an agent
            movable = [a for a in live if a not in waiting or waiting[a]()]
            if self.flight and (not movable or self.rng.random() < 0.4):
                i = self.rng.randrange(len(self.flight))
                dst, kind, group, src, value = self.flight.pop(i)
                # stores of one thread to one address arrive in order: a later value never loses to an earlier one
                self.seen[dst][kind][group][src] = max(self.seen[dst][kind][group][src], value)
                continue
            if not movable:
                raise Hazard(f"deadlock with {len(live)} agents waiting")
            a = self.rng.choice(movable)
            waiting.pop(a, None)
            try:
                pred = next(a)
            except StopIteration:
                live.remove(a)
                continue
            if pred is not None:
                waiting[a] = pred
        if not all(all(row) for row in self.out_done):
            raise Hazard("a chunk never left its ring")


@pytest.fixture(scope="module")
def plan():
    from tensorflow_allreduce_b200 import _lib

    lib = _lib.lib()

    def get(nbytes, slice_bytes, chunk, slots, cgroups, unit=0):
        out = (C.c_longlong * 4)()
        assert lib.bc_plan_pipeline(nbytes, slice_bytes, chunk, slots, cgroups, unit, out) == 0
        return tuple(out)

    return get


def test_rings_and_lags_of_the_planner_are_safe_under_any_interleaving(plan):
    rng = random.Random(20240611)
    cases = 0
    for trial in range(160):
        P = rng.choice([2, 3, 4, 8])
        GC = rng.choice([1, 2, 3, 4, 8])
        GR = rng.choice([1, 2, 4, 8])
        slots_cfg = rng.choice([0, 2, 4, 6, 16, 24])
        chunk_cfg = rng.choice([64 << 10, 256 << 10])
        nchunks_want = rng.choice([1, 2, 3, 7, 16, 17, 33, 50])
        nbytes = nchunks_want * chunk_cfg - rng.choice([0, 16, 4096])
        chunk_bytes, nchunks, slots, lag = plan(max(nbytes, 16), 64 << 20, chunk_cfg, slots_cfg, GC)
        if nchunks == 0:
            continue
        Model(P, nchunks, slots, lag, GR, GC, random.Random(trial)).run()
        cases += 1
    assert cases > 100


def test_the_model_sees_what_the_launch_check_refuses():
    # The launch refuses a ring that wraps with a lag of at least its size, and one whose slots
    # change hands between copier groups; the model shows why (it must not pass them silently).
    with pytest.raises(Hazard):
        for seed in range(20):
            Model(4, 12, 2, 2, 1, 1, random.Random(seed)).run()
    with pytest.raises(Hazard):
        for seed in range(50):
            Model(2, 40, 5, 2, 2, 2, random.Random(seed)).run()


def test_streaming_units_give_rings_that_fit(plan):
    # With streaming reducers a chunk is a whole number of steps of all ranks' reducer blocks, which
    # can be megabytes: the plan must still fit the slice or say that there is none.
    for world in (4, 8):
        unit = world * 16 * 512 * 4 * 16
        for slice_mb in (2, 8, 64, 256):
            for nbytes in (48 << 20, 64 << 20, (96 << 20) + 16, 1 << 30, 3 << 30):
                chunk_bytes, nchunks, slots, lag = plan(nbytes, slice_mb << 20, 0, 0, 0, unit)
                if nchunks == 0:
                    assert 2 * unit * 8 > slice_mb << 20 or slots * chunk_bytes > slice_mb << 20
                    continue
                assert chunk_bytes % unit == 0 and slots * chunk_bytes <= slice_mb << 20
                if 16 * 2 * unit <= slice_mb << 20:          # room for 16 slots of two steps each
                    assert chunk_bytes >= 2 * unit
                Model(world, min(nchunks, 40), min(slots, min(nchunks, 40)), lag, 1, 4, random.Random(nbytes % 97)).run()
