"""Model check of the fused all-reduce's slot protocol (host-side reasoning, no GPU).

Every rank runs the same program: publish(seq) - one tagged store into slot seq % SLOTS of every
rank's inbox, the stores of one publish landing in any order and interleaved with everybody else's
- then consume(seq), which waits until all ranks' tags for seq are in its own inbox and reads them.
A publish may only overwrite a slot entry whose previous all-reduce (seq - SLOTS) the destination
has already consumed.  Random schedules show that two slots are enough and one is not."""
import random

import pytest


def _run(world, slots, n_reduces, rng):
    """Returns the first violated (seq, src, dst) or None."""
    inbox = [[[0] * world for _ in range(slots)] for _ in range(world)]   # [dst][slot][src] = tag
    consumed = [-1] * world          # last sequence number each rank has finished consuming
    # per-rank program counter: (seq, phase); phase 0 = publishing (pending destinations), 1 = consuming
    seq = [0] * world
    pending = [list(range(world)) for _ in range(world)]
    phase = [0] * world
    while any(s < n_reduces for s in seq):
        runnable = []
        for r in range(world):
            if seq[r] >= n_reduces:
                continue
            if phase[r] == 0:
                runnable.append(r)
            elif all(inbox[r][seq[r] % slots][src] == seq[r] + 1 for src in range(world)):
                runnable.append(r)
        assert runnable, "deadlock"
        r = rng.choice(runnable)
        if phase[r] == 0:
            dst = pending[r].pop(rng.randrange(len(pending[r])))
            if seq[r] - slots >= 0 and consumed[dst] < seq[r] - slots:
                return (seq[r], r, dst)          # overwrote data the destination still needs
            inbox[dst][seq[r] % slots][r] = seq[r] + 1
            if not pending[r]:
                phase[r] = 1
        else:
            consumed[r] = seq[r]
            seq[r] += 1
            phase[r] = 0
            pending[r] = list(range(world))
    return None


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_slots_are_never_overwritten_early(world):
    rng = random.Random(world)
    for _ in range(300):
        assert _run(world, 2, 40, rng) is None


def test_one_slot_would_be_overwritten_early():
    rng = random.Random(1)
    assert any(_run(2, 1, 40, rng) is not None for _ in range(300))
