"""Model of the peer-store all-gather protocol (sparsewave_b200/csrc/swb_peer_window.cu) under random
interleavings: R ranks, each running step after step one exchange kernel of G CTAs (of which only a few are
resident at a time) followed by a consumer that reads its whole window.  Checks that every schedule
finishes (no wait depends on a CTA that cannot run) and that a consumer never sees a chunk of another
epoch (nothing is overwritten while it is read, nothing is read before it has landed).  A step names the
one of the window's two buffers that it fills; the ready-flag round trip (steps 1 and 2) is taken only
when the step before it filled the same buffer."""
import random

import pytest


class Rank:
    def __init__(self, ranks, slices):
        self.ready = [0] * ranks
        self.arrivals = [0, 0]  # per buffer: CTAs of any rank whose slice has landed in it, ever
        self.fills = [0, 0]     # per buffer: finished steps that filled it
        self.epoch = 0
        self.count = 0          # CTAs of this rank's current kernel that have finished
        self.last = None        # buffer of the last finished step
        self.flag_writes = 0    # ready flags this rank has sent, ever
        # data[buffer][source rank][slice] = epoch of the content
        self.data = [[[0] * slices for _ in range(ranks)] for _ in range(2)]


def exchange_cta(world, r, b, grid, buf=0):
    ranks = len(world)
    me = world[r]
    epoch = me.epoch + 1
    handshake = me.last == buf                   # the step before filled this buffer: wait for its readers
    fill = me.fills[buf] + 1
    yield
    if handshake and b == 0:                     # 1. ready flags out
        for k in range(ranks):
            world[k].ready[r] = epoch
            me.flag_writes += 1
            yield
    for k in range(ranks):                       # 2. ready flags in (not its own)
        while handshake and k != r and me.ready[k] < epoch:
            yield
    dst, piece = b % ranks, b // ranks           # 3. this CTA's slice of the chunk into window dst
    world[dst].data[buf][r][piece] = epoch
    yield
    world[dst].arrivals[buf] += 1                # 4. the slice has landed: one arrival at the destination
    yield
    me.count += 1                                #    the CTA of this rank that finishes last waits
    if me.count != grid:
        return
    while me.arrivals[buf] < fill * grid:        # 5. every rank's CTAs aimed at this buffer have arrived
        yield
    me.fills[buf] = fill
    me.count = 0
    me.last = buf
    me.epoch = epoch


def consumer(world, r, step, errors, buf=0):
    for k in range(len(world)):
        for piece, seen in enumerate(world[r].data[buf][k]):
            if seen != step:
                errors.append((r, step, k, piece, seen))
            yield


def rank_program(world, r, steps, grid, resident, rng, errors, buffers=None):
    """One rank's stream: kernels in order; inside an exchange kernel at most `resident` CTAs run at a
    time, started in index order, each advanced in random order.  buffers[step - 1]: the buffer of a step."""
    for step in range(1, steps + 1):
        buf = buffers[step - 1] if buffers else 0
        waiting = [exchange_cta(world, r, b, grid, buf) for b in range(grid)]
        running = []
        while waiting or running:
            while waiting and len(running) < resident:
                running.append(waiting.pop(0))
            g = rng.choice(running)
            try:
                next(g)
            except StopIteration:
                running.remove(g)
            yield
        yield from consumer(world, r, step, errors, buf)


# the buffer of each step: always the first (swb_comm_window_allgather), taking turns (the sharded operators),
# a replayed graph of three alternating steps (the replay's first step meets the buffer of its last), mixed use
BUFFER_SEQUENCES = {"first only": [0] * 6, "alternating": [0, 1] * 3, "odd graph replayed": [0, 1, 0] * 2,
                    "mixed": [0, 0, 1, 1, 0, 1]}


@pytest.mark.parametrize("sequence", sorted(BUFFER_SEQUENCES))
@pytest.mark.parametrize("ranks,slices,resident", [(2, 3, 1), (2, 4, 8), (4, 2, 2), (8, 1, 3), (3, 2, 1)])
def test_every_schedule_finishes_and_windows_are_consistent(ranks, slices, resident, sequence):
    grid = ranks * slices
    buffers = BUFFER_SEQUENCES[sequence]
    steps = len(buffers)
    handshakes = sum(1 for i in range(1, steps) if buffers[i] == buffers[i - 1])
    for seed in range(30):
        rng = random.Random(seed)
        world = [Rank(ranks, slices) for _ in range(ranks)]
        errors = []
        programs = [rank_program(world, r, steps, grid, resident, rng, errors, buffers) for r in range(ranks)]
        live = list(range(ranks))
        ticks = 0
        while live:
            # uneven progress: one rank may run far ahead of the others within what the protocol allows
            r = rng.choice(live) if rng.random() < 0.7 else live[0]
            try:
                next(programs[r])
            except StopIteration:
                live.remove(r)
            ticks += 1
            assert ticks < 2_000_000, "a schedule did not finish"
        assert not errors, errors[:3]
        assert all(w.epoch == steps and w.count == 0 and sum(w.arrivals) == steps * grid for w in world)
        # the round trip is taken exactly where a buffer is filled twice in a row: never when they take turns
        assert all(w.flag_writes == handshakes * ranks for w in world)


def test_the_model_detects_a_missing_ready_wait():
    """The same model without step 2 lets a fast rank overwrite a window that is still being read."""
    def broken_cta(world, r, b, grid):
        g = exchange_cta(world, r, b, grid)
        me = world[r]
        saved = me.ready
        me.ready = [1 << 30] * len(world)  # every ready flag looks raised
        try:
            yield from g
        finally:
            me.ready = saved
    found = False
    for seed in range(40):
        rng = random.Random(seed)
        world = [Rank(2, 2) for _ in range(2)]
        errors = []

        def program(r):
            for step in range(1, 6):
                ctas = [broken_cta(world, r, b, 4) for b in range(4)]
                while ctas:
                    g = rng.choice(ctas)
                    try:
                        next(g)
                    except StopIteration:
                        ctas.remove(g)
                    yield
                yield from consumer(world, r, step, errors)
        programs = [program(0), program(1)]
        live = [0, 1]
        for _ in range(100000):
            if not live:
                break
            r = rng.choice(live)
            try:
                next(programs[r])
            except StopIteration:
                live.remove(r)
        found = found or bool(errors)
    assert found
