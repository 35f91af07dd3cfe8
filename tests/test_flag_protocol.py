"""A host-side model check of the epoch-flag protocol of the fused all-gather GEMM (``parallel/tp.py``): ranks run the calls of
one buffer pair in lock-free fashion under random interleavings; every pull must observe the data of its own call (never a
stale shard, never one already overwritten by a later call), and no rank may wait forever.

The model: per call k a rank (1) writes its shard into buffer k % 2, (2) raises its flag for call k at every peer, then for
each peer p (3) waits until p's flag has reached k and (4) reads p's shard of buffer k % 2.  Steps of different ranks interleave
arbitrarily; steps of one rank are ordered (stream order).  With one buffer instead of two the check must fail: that is the
counter-example showing the alternation is needed."""
import random

import pytest


def run(world: int, calls: int, nbuf: int, seed: int):
    rnd = random.Random(seed)
    data = [[None] * nbuf for _ in range(world)]            # data[r][b]: which call's shard rank r holds in buffer b
    flags = [[[0] * world for _ in range(nbuf)] for _ in range(world)]   # flags[r][set][src]
    # program of a rank: list of (op, args)
    prog = []
    for r in range(world):
        steps = []
        for k in range(1, calls + 1):
            steps.append(("write", k))
            steps.append(("signal", k))
            for p in range(world):
                if p != r:
                    steps.append(("pull", k, p))
        prog.append(steps)
    pc = [0] * world
    violations = []
    for _ in range(100000):
        runnable = []
        for r in range(world):
            if pc[r] >= len(prog[r]):
                continue
            op = prog[r][pc[r]]
            if op[0] == "pull" and flags[r][op[1] % nbuf][op[2]] < op[1]:
                continue                                      # bounded wait in the kernel: not runnable yet
            runnable.append(r)
        if not runnable:
            break
        r = rnd.choice(runnable)
        op = prog[r][pc[r]]
        if op[0] == "write":
            data[r][op[1] % nbuf] = op[1]
        elif op[0] == "signal":
            for p in range(world):
                flags[p][op[1] % nbuf][r] = op[1]
        else:
            seen = data[op[2]][op[1] % nbuf]
            if seen != op[1]:
                violations.append((r, op, seen))
        pc[r] += 1
    done = all(pc[r] == len(prog[r]) for r in range(world))
    return done, violations


@pytest.mark.parametrize("world", [2, 3, 4])
def test_alternating_buffers_are_safe_under_any_interleaving(world):
    for seed in range(200):
        done, bad = run(world, calls=6, nbuf=2, seed=seed)
        assert done, "a rank waits forever"
        assert not bad, bad[:3]


def test_a_single_buffer_can_be_overwritten_before_it_is_read():
    assert any(run(2, calls=4, nbuf=1, seed=s)[1] for s in range(200))
