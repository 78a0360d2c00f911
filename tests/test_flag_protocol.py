"""Model check of the epoch-flag protocol behind the peer-memory collectives (CPU only).

The runtime (``parallel/sharded.py`` with ``parallel/symm.py``) orders cross-GPU reads and writes of
one sharded unit with three flag channels per unit, each a row of per-rank epoch counters that a
rank writes into every peer's arena:

  shard-ready     rank r has finished writing its parameter shard for optimizer step e
  grads-ready     rank r's gradient staging buffer holds micro-step g
  grads-consumed  rank r has finished reading everybody's staging buffer of micro-step g

Here every rank is a coroutine that yields before each access to shared state, and a seeded
scheduler interleaves them at random.  The invariants: a gather reads only shards of the current
step; a reduce reads only staging buffers of the current micro-step; nobody overwrites a buffer
that a peer has still to read.  The same run with one of the waits removed must be caught, which
shows that the checker can see the races the waits are there to prevent.
"""
import random

import pytest

SHARD, GRAD, DONE = 0, 1, 2


class World:
    def __init__(self, W):
        self.W = W
        self.flags = [[[0] * W for _ in range(3)] for _ in range(W)]     # flags[owner][channel][writer]
        self.shard = [("init", 0)] * W                                    # (tag, step) of each rank's shard
        self.stage = [("none", 0)] * W                                    # (tag, micro-step) of each staging buffer
        self.errors = []


def rank_program(w: World, r: int, steps: int, micro: int = 2, wait_done: bool = True, wait_shard: bool = True):
    W = w.W
    shard_epoch, grad_epoch = 1, 0
    # step 0: the initial shards are announced
    w.shard[r] = ("shard", shard_epoch)
    yield
    for p in range(W):
        w.flags[p][SHARD][r] = shard_epoch
        yield
    for step in range(steps):
        # ---- gather: wait for every peer's shard of this step, then read them
        for p in range(W):
            if wait_shard:
                while w.flags[r][SHARD][p] < shard_epoch:
                    yield
            yield
            tag, e = w.shard[p]
            if e != shard_epoch:
                w.errors.append(f"rank {r} step {step}: gathered shard of rank {p} from step {e}, wanted {shard_epoch}")
        # ---- `micro` backward passes (gradient accumulation; parameters stay gathered in between):
        # publish gradients, reduce, mark consumed
        for _ in range(micro):
            grad_epoch += 1
            if grad_epoch > 1 and wait_done:
                for p in range(W):
                    while w.flags[r][DONE][p] < grad_epoch - 1:      # peers have read my previous staging buffer
                        yield
            yield
            w.stage[r] = ("grad", grad_epoch)
            yield
            for p in range(W):
                w.flags[p][GRAD][r] = grad_epoch
                yield
            for p in range(W):
                while w.flags[r][GRAD][p] < grad_epoch:
                    yield
                yield
                tag, e = w.stage[p]
                if e != grad_epoch:
                    w.errors.append(f"rank {r} step {step}: reduced staging buffer of rank {p} from micro-step {e}, wanted {grad_epoch}")
            for p in range(W):
                w.flags[p][DONE][r] = grad_epoch
                yield
        # ---- optimizer step on the own shard, then announce it
        shard_epoch += 1
        yield
        w.shard[r] = ("shard", shard_epoch)
        yield
        for p in range(W):
            w.flags[p][SHARD][r] = shard_epoch
            yield


def run(seed: int, W: int = 3, steps: int = 3, **kw):
    rng = random.Random(seed)
    w = World(W)
    progs = [rank_program(w, r, steps, **kw) for r in range(W)]
    live = list(range(W))
    budget = 200000
    while live and budget:
        budget -= 1
        r = rng.choice(live)
        try:
            next(progs[r])
        except StopIteration:
            live.remove(r)
    assert budget, "the protocol did not terminate (a rank waits for a flag nobody writes)"
    return w.errors


def test_protocol_holds_under_random_interleavings():
    for seed in range(300):
        assert run(seed) == [], seed
    for seed in range(50):
        assert run(1000 + seed, W=4, steps=2) == []


@pytest.mark.parametrize("mutation", ["wait_done", "wait_shard"])
def test_checker_catches_a_missing_wait(mutation):
    """Without the grads-consumed wait a fast rank overwrites its staging buffer with the next
    micro-batch while a slow peer is still to read it (between optimizer steps the next gather
    happens to order the two, within a step nothing else does); without the shard-ready wait a
    gather reads a shard of the previous step."""
    caught = sum(1 for seed in range(300) if run(seed, **{mutation: False}))
    assert caught > 0
