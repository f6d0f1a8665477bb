"""Model check of the producer / consumer handshake that orders the fused multi-GPU kernels.

The CUDA kernels wait on and advance monotonic counters exactly as `makani_b200.parallel.peer.sync_descriptor` lays them
out (consumer: ready[p] >= n_read + 1 for every peer, then n_read += 1 and free[me] += 1 on every peer; producer:
free[p] >= n_prod, then n_prod += 1 and ready[me] += 1 on every peer).  This test runs that protocol for the kernel
sequence of the distributed spectral convolution on a 2 x 2 process grid under thousands of random interleavings and
checks the three properties the design relies on: no deadlock, every consumer sees exactly the generation it expects
from every rank, and no segment is overwritten while (or before) a peer reads it.
"""

import random

import pytest


class SlotState:
    """One rank's copy of a slot: flags, counters and the generation tag of every rank's segment."""

    def __init__(self, members):
        self.members = members
        self.ready = {p: 0 for p in members}
        self.free = {p: 0 for p in members}
        self.n_prod = 0
        self.n_read = 0
        self.data = {p: 0 for p in members}       # generation of the segment written by rank p
        self.reading = None                       # snapshot while a consumer kernel of this rank is in flight


class Kernel:
    """A launch that consumes slot `cons` and / or produces slot `prod`; three observable events: start (all waits
    passed, reads begin), write (the epilogue stores reach the peers' copies), end (last CTA: bump + signal)."""

    def __init__(self, rank, cons, prod):
        self.rank, self.cons, self.prod = rank, cons, prod
        self.phase = 0

    def enabled(self, world):
        if self.phase > 0:
            return True
        r = self.rank
        if self.cons is not None:
            s = world[self.cons][r]
            if any(s.ready[p] < s.n_read + 1 for p in s.members):
                return False
        if self.prod is not None:
            s = world[self.prod][r]
            if any(s.free[p] < s.n_prod for p in s.members):
                return False
        return True

    def advance(self, world):
        r = self.rank
        if self.phase == 0:                                   # start: reads of the consumed slot begin
            if self.cons is not None:
                s = world[self.cons][r]
                want = s.n_read + 1
                assert all(g == want for g in s.data.values()), f"rank {r} reads {self.cons}: {s.data} != generation {want}"
                s.reading = dict(s.data)
        elif self.phase == 1:                                 # stores of the produced segment land in every copy
            if self.prod is not None:
                gen = world[self.prod][r].n_prod + 1
                for p in world[self.prod][r].members:
                    peer = world[self.prod][p]
                    assert peer.reading is None or self.prod != self._reading_slot(world, p), \
                        f"rank {r} overwrites {self.prod} while rank {p} reads it"
                    assert peer.n_read >= gen - 1, f"rank {r} overwrites generation {gen - 1} of {self.prod} before rank {p} consumed it"
                    peer.data[r] = gen
        else:                                                 # end: last CTA bumps the counters and signals the peers
            if self.cons is not None:
                s = world[self.cons][r]
                assert s.reading == s.data, f"{self.cons} changed under rank {r}'s reads"
                s.reading = None
                s.n_read += 1
                for p in s.members:
                    world[self.cons][p].free[r] += 1
            if self.prod is not None:
                s = world[self.prod][r]
                s.n_prod += 1
                for p in s.members:
                    world[self.prod][p].ready[r] += 1
        self.phase += 1
        return self.phase == 3

    def _reading_slot(self, world, p):
        for name, per_rank in world.items():
            if p in per_rank and per_rank[p].reading is not None:
                return name
        return None


def _grid(ph, pw):
    ranks = [(h, w) for h in range(ph) for w in range(pw)]
    idx = {c: i for i, c in enumerate(ranks)}
    hgroup = {idx[(h, w)]: [idx[(q, w)] for q in range(ph)] for h, w in ranks}     # ranks that differ in h
    wgroup = {idx[(h, w)]: [idx[(h, q)] for q in range(pw)] for h, w in ranks}
    return len(ranks), hgroup, wgroup


def _spectral_conv_sequence(rank, layers):
    """Forward and backward kernel sequence of one rank: (consumed slot, produced slot) per launch."""
    fwd = [(None, "xw"), ("xw", "t1"), ("t1", None), (None, "t3"), ("t3", "t4"), ("t4", None)]
    seq = []
    for _ in range(layers):
        seq += fwd
    for _ in range(layers):
        seq += fwd          # the adjoint chain uses the same buffers in the same roles
    return [Kernel(rank, c, p) for c, p in seq]


@pytest.mark.parametrize("ph,pw", [(2, 2), (4, 2), (1, 2), (3, 1)])
def test_random_interleavings_are_safe_and_complete(ph, pw):
    n, hgroup, wgroup = _grid(ph, pw)
    slot_group = {"xw": wgroup, "t1": hgroup, "t3": hgroup, "t4": wgroup}
    for seed in range(300):
        rng = random.Random(seed)
        world = {name: {r: SlotState(groups[r]) for r in range(n)} for name, groups in slot_group.items()}
        queues = {r: _spectral_conv_sequence(r, layers=3) for r in range(n)}
        steps = 0
        while any(queues.values()):
            runnable = [r for r, q in queues.items() if q and q[0].enabled(world)]
            assert runnable, f"deadlock (seed {seed}): heads {[ (r, q[0].cons, q[0].prod, q[0].phase) for r, q in queues.items() if q]}"
            # skewed scheduling: sometimes one rank races far ahead of the others
            r = rng.choice(runnable) if rng.random() < 0.7 else runnable[0]
            if queues[r][0].advance(world):
                queues[r].pop(0)
            steps += 1
            assert steps < 10 ** 6
        for name, per_rank in world.items():
            for r, s in per_rank.items():
                assert s.n_prod == s.n_read == 6, (name, r, s.n_prod, s.n_read)


def test_a_missing_wait_is_caught_by_the_model():
    """Sanity of the checker itself: a producer that does not wait for `free` is flagged."""
    n, hgroup, wgroup = _grid(1, 2)
    world = {"xw": {r: SlotState(wgroup[r]) for r in range(n)}}

    class Rogue(Kernel):
        def enabled(self, world):
            return True

    seq0 = [Rogue(0, None, "xw"), Rogue(0, None, "xw")]
    with pytest.raises(AssertionError, match="before rank"):
        for k in seq0:
            while not k.advance(world):
                pass


def test_norm_and_matmul_exchanges_interleaved_with_the_transform_chain():
    """All slot users of one SFNO block on a 2 x 2 grid: instance-norm statistics over the whole spatial group
    (produce, consume), the transform chain, and a second norm; several blocks back to back."""
    n, hgroup, wgroup = _grid(2, 2)
    everyone = {r: list(range(n)) for r in range(n)}
    slot_group = {"xw": wgroup, "t1": hgroup, "t3": hgroup, "t4": wgroup, "inorm": everyone}
    block = [(None, "inorm"), ("inorm", None),                                    # norm 0
             (None, "xw"), ("xw", "t1"), ("t1", None), (None, "t3"), ("t3", "t4"), ("t4", None),
             (None, "inorm"), ("inorm", None)]                                    # norm 1
    for seed in range(200):
        rng = random.Random(1000 + seed)
        world = {name: {r: SlotState(groups[r]) for r in range(n)} for name, groups in slot_group.items()}
        queues = {r: [Kernel(r, c, p) for _ in range(4) for c, p in block] for r in range(n)}
        while any(queues.values()):
            runnable = [r for r, q in queues.items() if q and q[0].enabled(world)]
            assert runnable, f"deadlock (seed {seed})"
            r = rng.choice(runnable)
            if queues[r][0].advance(world):
                queues[r].pop(0)
        assert all(s.n_prod == s.n_read == 8 for s in world["inorm"].values())
