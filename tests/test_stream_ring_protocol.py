"""The barrier protocol of the streaming decode attention kernel
(arle_b200/csrc/attention_decode_stream.cu), as a model on the CPU: two producer warps that
fill a ring of stages, two groups of four consumer warps that take alternate tiles, "full"
barriers with a transaction count and "empty" barriers, all with one phase bit, and copies
that land in any order.  The kernel takes only even ring depths; this shows why (with an odd
depth a group's waits on a stage all carry the same parity, and a group that comes back before
the other group's load has landed reads the stage as it is), and that even depths are safe
whatever the order in which copies land and warps run.  The model follows the kernel's loops
line by line; it does not run the kernel."""
import random

import pytest


class Barrier:
    """An mbarrier: arrivals expected per phase, bytes outstanding, phases completed."""

    def __init__(self, count):
        self.count, self.pending, self.tx, self.phase = count, count, 0, 0

    def arrive(self, tx=0):
        self.tx += tx
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the phase expects"
        self._check()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self._check()

    def _check(self):
        if self.pending == 0 and self.tx == 0:
            self.phase += 1
            self.pending = self.count

    def passed(self, parity):          # try_wait.parity: has the phase of this parity completed?
        return (self.phase & 1) != parity


def run_cta(tiles_per_piece, depth, seed, land_probability):
    """One CTA walking pieces of ``tiles_per_piece`` tiles each.  Returns None, or what went wrong."""
    rng = random.Random(seed)
    full = [Barrier(2) for _ in range(depth)]
    empty = [Barrier(4) for _ in range(depth)]
    in_flight = []
    named = {"count": 0, "generation": 0}

    def producer():
        st, par = 0, 0
        for ntile in tiles_per_piece:
            for _ in range(ntile):
                while not empty[st].passed(par ^ 1):
                    yield
                full[st].arrive(tx=16384)
                in_flight.append((full[st], 16384))
                st += 1
                if st == depth:
                    st, par = 0, par ^ 1
                yield

    def consumer(warp):
        group = warp >> 2
        st, par, n = 0, 0, 0
        for ntile in tiles_per_piece:
            for _ in range(ntile):
                my_st, my_par = st, par
                st += 1
                if st == depth:
                    st, par = 0, par ^ 1
                mine = (n & 1) == group
                n += 1
                if not mine:
                    continue
                while not full[my_st].passed(my_par):
                    yield
                use = (n - 1) // depth                     # which load into this stage the warp is about to read
                if full[my_st].phase < use + 1:
                    raise AssertionError(f"warp {warp} read stage {my_st} for load {use} after {full[my_st].phase} loads had landed")
                yield
                empty[my_st].arrive()
            for _ in range(2):                             # the merge: the consumers' named barrier, twice
                generation = named["generation"]
                named["count"] += 1
                if named["count"] == 8:
                    named["count"] = 0
                    named["generation"] += 1
                while named["generation"] == generation:
                    yield

    threads = [producer(), producer()] + [consumer(w) for w in range(8)]
    alive = list(range(len(threads)))
    for _ in range(4_000_000):
        if not alive:
            break
        if in_flight and rng.random() < land_probability:
            bar, nbytes = in_flight.pop(rng.randrange(len(in_flight)))       # copies land in any order
            bar.complete_tx(nbytes)
        i = rng.choice(alive)
        try:
            next(threads[i])
        except StopIteration:
            alive.remove(i)
        except AssertionError as e:
            return str(e)
    if alive:
        return f"no progress: threads {alive} still running"
    if in_flight:
        return "copies still in flight when the CTA ends"
    return None


PIECES = [32, 32, 32, 15]          # 111 tiles: three whole pairs and a piece, as at 64 rows of 2,048 keys


@pytest.mark.parametrize("depth", [2, 4, 6, 8])
def test_even_ring_depths_never_read_a_stage_early(depth):
    for land in (0.5, 0.1, 0.03):
        for seed in range(12):
            assert run_cta(PIECES, depth, seed, land) is None, (depth, land, seed)


@pytest.mark.parametrize("depth", [3, 5, 7])
def test_odd_ring_depths_do(depth):
    """Why the kernel rounds the depth down to an even number: with slow, disordered copies an odd
    depth lets a consumer group pass a wait that belongs to the other group's load."""
    faults = [run_cta(PIECES, depth, seed, 0.05) for seed in range(12)]
    assert any(f is not None and "read stage" in f for f in faults)


def test_the_kernel_keeps_the_depth_even():
    import os
    src = open(os.path.join(os.path.dirname(__file__), "..", "arle_b200", "csrc", "attention_decode_stream.cu")).read()
    assert "stages &= ~1;" in src
