"""Pure-Python model of the peer data plane's epoch protocol, explored over
random interleavings.

Every rank runs the same program per training step (``parallel/peer.py``):

    forward    wait PUB_READY[owner] >= e for each owner, pull its slots,
               then signal PUB_CONSUMED[self] = e.  Slots of modules whose
               forward did not run in a step are pulled late, right before the
               optimizer (the signal always follows the last pull)
    backward   wait GRAD_CONSUMED[all] >= g (first write of the step only),
               write the local gradient slots, signal GRAD_READY[self] = g + 1
    optimizer  wait GRAD_READY[all] >= g + 1, read every rank's slots of the
               owned parameters, signal GRAD_CONSUMED[self] = g + 1,
               wait PUB_CONSUMED[all] >= e, write the owned publish slots,
               signal PUB_READY[self] = e + 1

Flags only grow; a wait blocks until the flag reaches the wanted value.  The
model checks, for any interleaving the waits allow, that no rank ever reads a
slot of the wrong epoch and that no slot is overwritten while a reader of the
previous epoch has not finished -- and that dropping any one of the four waits
is caught (so the checks are not vacuous).
"""
import random

import pytest

PUB_READY, PUB_CONSUMED, GRAD_READY, GRAD_CONSUMED = range(4)


class Violation(AssertionError):
    pass


def _program(rank, world, steps, drop=None):
    """The op list of one rank; ``drop`` names a wait to leave out."""
    ops = []
    for s in range(steps):
        e = s + 1                      # publish epoch consumed by this step's forward (epoch 1 = initial publish)
        g = s                          # gradient epochs completed before this step
        # modules that sat this forward out; now and then a rank's forward touches no
        # dedicated module at all (then nothing but GRAD_CONSUMED orders its next gradient write)
        late = [o for o in range(world) if s >= 1 and ((o + rank + s) % 3 == 0 or rank == 0)]

        def pull(owner):
            if drop != "pub_ready":
                ops.append(("wait", PUB_READY, [owner], e))
            ops.append(("read_pub", owner, e))

        for owner in range(world):
            if owner not in late:
                pull(owner)
        if not late:
            ops.append(("signal", PUB_CONSUMED, e))
        if drop != "grad_consumed":
            ops.append(("wait", GRAD_CONSUMED, list(range(world)), g))
        ops.append(("write_grad", g + 1))
        ops.append(("signal", GRAD_READY, g + 1))
        if drop != "grad_ready":
            ops.append(("wait", GRAD_READY, list(range(world)), g + 1))
        for src in range(world):
            ops.append(("read_grad", src, g + 1))
        ops.append(("signal", GRAD_CONSUMED, g + 1))
        for owner in late:
            pull(owner)
        if late:
            ops.append(("signal", PUB_CONSUMED, e))
        if drop != "pub_consumed":
            ops.append(("wait", PUB_CONSUMED, list(range(world)), e))
        ops.append(("write_pub", e + 1))
        ops.append(("signal", PUB_READY, e + 1))
    return ops


def simulate(world, steps, seed, drop=None):
    rng = random.Random(seed)
    flags = [[0] * world for _ in range(4)]
    for r in range(world):
        flags[PUB_READY][r] = 1                      # the constructor publishes epoch 1 behind a barrier
    pub = [1] * world                                # epoch held by each owner's publish slots
    grad = [0] * world                               # gradient epoch held by each rank's arena
    pub_reads_done = [[0] * world for _ in range(world)]     # [owner][reader]: last epoch fully read
    grad_reads_done = [[0] * world for _ in range(world)]    # [src][owner]
    progs = [_program(r, world, steps, drop) for r in range(world)]
    pc = [0] * world
    while any(pc[r] < len(progs[r]) for r in range(world)):
        runnable = []
        for r in range(world):
            if pc[r] >= len(progs[r]):
                continue
            op = progs[r][pc[r]]
            if op[0] == "wait" and not all(flags[op[1]][i] >= op[3] for i in op[2]):
                continue
            runnable.append(r)
        if not runnable:
            raise Violation("deadlock")
        r = rng.choice(runnable)
        op = progs[r][pc[r]]
        pc[r] += 1
        kind = op[0]
        if kind == "signal":
            flags[op[1]][r] = op[2]
        elif kind == "read_pub":
            owner, want = op[1], op[2]
            if pub[owner] != want:
                raise Violation(f"rank {r} read publish epoch {pub[owner]} of owner {owner}, wanted {want}")
            pub_reads_done[owner][r] = want
        elif kind == "write_pub":
            new = op[1]
            if any(pub_reads_done[r][reader] < new - 1 for reader in range(world)):
                raise Violation(f"owner {r} overwrote publish epoch {new - 1} before every reader had it")
            pub[r] = new
        elif kind == "write_grad":
            new = op[1]
            if any(grad_reads_done[r][owner] < new - 1 for owner in range(world)):
                raise Violation(f"rank {r} overwrote gradient epoch {new - 1} before every owner read it")
            grad[r] = new
        elif kind == "read_grad":
            src, want = op[1], op[2]
            if grad[src] != want:
                raise Violation(f"owner {r} read gradient epoch {grad[src]} of rank {src}, wanted {want}")
            grad_reads_done[src][r] = want
    return True


@pytest.mark.parametrize("world", [2, 3, 8])
def test_protocol_is_safe_and_live_under_random_interleavings(world):
    for seed in range(300 if world < 8 else 60):
        assert simulate(world, steps=3, seed=seed)


@pytest.mark.parametrize("drop", ["pub_ready", "pub_consumed", "grad_ready", "grad_consumed"])
def test_every_wait_is_necessary(drop):
    caught = 0
    for seed in range(400):
        try:
            simulate(3, steps=3, seed=seed, drop=drop)
        except Violation:
            caught += 1
    assert caught > 0, f"leaving out the {drop} wait was never noticed: the model checks nothing"
