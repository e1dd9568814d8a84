"""The two hand-shakes behind the row-shard gathers of wf_comm.cu, replayed on the CPU under random schedules.

Small gathers: every rank pushes its words, tagged with the gather's number, into the peers' landing buffers and
then pulls the peers' words out of its own; the landing buffer has two halves used by even and odd gathers and
nothing else orders the ranks.  Large gathers: a rank writes its block into its own staging area, tells the peers
"ready", reads their staging areas, tells them "done"; before it overwrites its staging area it waits for every
peer's "done" of the gather before.  The claims checked here, for many random interleavings of the ranks' steps:
no rank ever reads a word or a block of another gather than the one it is in, nothing is overwritten before its
last reader is through, and every rank finishes (no schedule leaves all ranks waiting).
"""
import random

import pytest


def run_small(world, gathers, rng):
    # landing[r][half][src] = tag of the word rank src last stored into rank r's landing buffer
    landing = [[[0] * world for _ in range(2)] for _ in range(world)]
    unread = [[[False] * world for _ in range(2)] for _ in range(world)]  # stored and not yet pulled
    step = [0] * world  # 2 * g: about to push gather g; 2 * g + 1: about to pull it
    while any(s < 2 * gathers for s in step):
        able = []
        for r in range(world):
            if step[r] >= 2 * gathers:
                continue
            g, pulling = divmod(step[r], 2)
            if not pulling or all(landing[r][g & 1][s] == g + 1 for s in range(world) if s != r):
                able.append(r)
        assert able, f"every rank waits: {step}"
        r = rng.choice(able)
        g, pulling = divmod(step[r], 2)
        half = g & 1
        if not pulling:
            for d in range(world):
                if d != r:
                    assert not unread[d][half][r], f"rank {r} overwrites gather {landing[d][half][r] - 1} in rank {d} before it was read"
                    landing[d][half][r] = g + 1
                    unread[d][half][r] = True
        else:
            for s in range(world):
                if s != r:
                    assert landing[r][half][s] == g + 1
                    unread[r][half][s] = False
        step[r] += 1


def run_large(world, gathers, rng):
    stage = [0] * world                       # gather whose block the staging area of rank r holds (1-based)
    readers = [set() for _ in range(world)]   # ranks that still have to read stage[r]
    ready = [[0] * world for _ in range(world)]  # ready[r][s]: last "ready" rank s told rank r
    done = [[0] * world for _ in range(world)]
    step = [0] * world  # 3 * g: wait for "done" of g - 1 and write the block; + 1: publish ready and wait; + 2: read, then "done"
    while any(s < 3 * gathers for s in step):
        able = []
        for r in range(world):
            if step[r] >= 3 * gathers:
                continue
            g, phase = divmod(step[r], 3)
            if phase == 0 and all(done[r][s] >= g for s in range(world) if s != r):
                able.append(r)
            elif phase == 1:
                able.append(r)
            elif phase == 2 and all(ready[r][s] >= g + 1 for s in range(world) if s != r):
                able.append(r)
        assert able, f"every rank waits: {step}"
        r = rng.choice(able)
        g, phase = divmod(step[r], 3)
        if phase == 0:
            assert not readers[r], f"rank {r} overwrites its block of gather {stage[r] - 1} while {readers[r]} still read it"
            stage[r] = g + 1
            readers[r] = {s for s in range(world) if s != r}
        elif phase == 1:
            for d in range(world):
                if d != r:
                    ready[d][r] = g + 1
        else:
            for s in range(world):
                if s != r:
                    assert stage[s] == g + 1, f"rank {r} in gather {g} reads rank {s}'s block of gather {stage[s] - 1}"
                    readers[s].discard(r)
            for d in range(world):
                if d != r:
                    done[d][r] = g + 1
        step[r] += 1


@pytest.mark.parametrize("world", [2, 3, 8])
def test_two_landing_halves_order_the_small_gathers(world):
    rng = random.Random(20261125 + world)
    for _ in range(200):
        run_small(world, 7, rng)


@pytest.mark.parametrize("world", [2, 3, 8])
def test_ready_and_done_flags_order_the_large_gathers(world):
    rng = random.Random(20261126 + world)
    for _ in range(200):
        run_large(world, 6, rng)


def test_one_landing_half_would_not_be_enough():
    """The checker itself: with a single half, some schedule overwrites a word before it was read."""
    def run_one_half(world, gathers, rng):
        landing = [[0] * world for _ in range(world)]
        unread = [[False] * world for _ in range(world)]
        step = [0] * world
        while any(s < 2 * gathers for s in step):
            able = [r for r in range(world) if step[r] < 2 * gathers and
                    (step[r] % 2 == 0 or all(landing[r][s] == step[r] // 2 + 1 for s in range(world) if s != r))]
            if not able:
                return "stuck"
            r = rng.choice(able)
            g, pulling = divmod(step[r], 2)
            if not pulling:
                for d in range(world):
                    if d != r:
                        if unread[d][r]:
                            return "overwritten"
                        landing[d][r], unread[d][r] = g + 1, True
            else:
                for s in range(world):
                    if s != r:
                        unread[r][s] = False
            step[r] += 1
        return "ok"

    rng = random.Random(7)
    assert any(run_one_half(2, 5, rng) != "ok" for _ in range(200))
