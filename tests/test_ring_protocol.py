"""Host-side model of the ring bookkeeping the W4A16 kernel's roles use (csrc/gemm_w4a16.cu): slots and phases
advanced by addition, K blocks dealt to convert groups and issuer threads by running count across work items.

The kernel cannot be single-stepped, so the arithmetic it relies on is restated here and checked against the
definitions it replaced (slot = count % depth, phase = (count / depth) & 1) over long sequences of work items of
uneven length, together with the two properties the barrier protocol needs:

  * a parity wait is only meaningful when the waiter is at most one phase ahead of the barrier — so every
    packed-weight slot must always be consumed by the SAME convert group (ring depth a multiple of the group count);
  * the look-ahead of the scale queue names exactly the K blocks the group visits next, across item boundaries.
"""
import itertools
import random

import pytest

# (activation-row tile, convert groups DQ, issuers NI, activation ring SA, operand ring AST, packed-weight ring SW)
CONFIGS = {
    16: dict(DQ=2, NI=4, SA=16, AST=8, SW=32),
    64: dict(DQ=2, NI=2, SA=12, AST=8, SW=16),
    128: dict(DQ=4, NI=2, SA=8, AST=8, SW=16),
    256: dict(DQ=3, NI=1, SA=5, AST=5, SW=6),
    "pair": dict(DQ=3, NI=1, SA=8, AST=8, SW=9),
}


def item_lengths(seed, n_items):
    rng = random.Random(seed)
    return [rng.choice([4, 5, 7, 64, 128, 3, 9]) for _ in range(n_items)]


class Ring:
    """slot / phase of a running position, advanced by `step` with wrap-around — the kernel's form."""

    def __init__(self, start, depth, step):
        assert step <= depth and start < depth
        self.slot, self.phase, self.depth, self.step = start, 0, depth, step

    def advance(self):
        self.slot += self.step
        if self.slot >= self.depth:
            self.slot -= self.depth
            self.phase ^= 1


@pytest.mark.parametrize("name", list(CONFIGS))
def test_issuer_slots_and_phases_follow_the_running_count(name):
    c = CONFIGS[name]
    for me in range(c["NI"]):
        act, op = Ring(me, c["SA"], c["NI"]), Ring(me, c["AST"], c["NI"])
        my_it, it0 = me, 0
        seen = []
        for length in item_lengths(1, 40):
            it_end = it0 + length
            while my_it < it_end:
                assert act.slot == my_it % c["SA"] and act.phase == (my_it // c["SA"]) & 1
                assert op.slot == my_it % c["AST"] and op.phase == (my_it // c["AST"]) & 1
                seen.append(my_it)
                act.advance(); op.advance()
                my_it += c["NI"]
            it0 = it_end
        assert seen == list(range(me, it0, c["NI"]))          # every NI-th block, none skipped, none twice


@pytest.mark.parametrize("name", list(CONFIGS))
def test_convert_group_rings_and_operand_reuse_wait(name):
    c = CONFIGS[name]
    DQ, SA, AST, SW = c["DQ"], c["SA"], c["AST"], c["SW"]
    for grp in range(DQ):
        w = Ring(grp, SW, DQ)
        os_slot = grp
        first_reuse = grp
        while first_reuse < AST:
            first_reuse += DQ
        done = Ring((first_reuse - AST) % SA, SA, DQ)
        done.phase = ((first_reuse - AST) // SA) & 1
        my_it, it0 = grp, 0
        for length in item_lengths(2, 60):
            it_end = it0 + length
            while my_it < it_end:
                assert w.slot == my_it % SW and w.phase == (my_it // SW) & 1
                assert os_slot == my_it % AST
                if my_it >= AST:                              # the block that used this operand slot before
                    j = my_it - AST
                    assert done.slot == j % SA and done.phase == (j // SA) & 1
                    done.advance()
                w.advance()
                os_slot = (os_slot + DQ) % AST
                my_it += DQ
            it0 = it_end


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_packed_weight_slot_belongs_to_one_convert_group(name):
    c = CONFIGS[name]
    owner = {}
    for it in range(10 * c["SW"] * c["DQ"]):
        slot, grp = it % c["SW"], it % c["DQ"]
        assert owner.setdefault(slot, grp) == grp, f"slot {slot} is consumed by groups {owner[slot]} and {grp}"
    # ... and the operand-slot wait can never be two phases ahead: a group's previous visit already waited for a
    # block at most one ring turn older (needs AST >= DQ)
    assert c["AST"] >= c["DQ"] and c["SW"] % c["DQ"] == 0


@pytest.mark.parametrize("name", list(CONFIGS))
def test_scale_queue_look_ahead_names_the_next_visits(name):
    """The queue holds the scales of this group's current and next two visits; at an item boundary the first three
    of the next item were fetched while the current one ran."""
    c = CONFIGS[name]
    DQ = c["DQ"]
    lengths = item_lengths(3, 50)
    starts = list(itertools.accumulate([0] + lengths))
    kb0 = [7 * i for i in range(len(lengths))]                  # arbitrary first K block per item
    for grp in range(DQ):
        my_it = grp
        # prefetch for the first item
        nxt = [kb0[0] + grp + j * DQ for j in range(3)]
        for i, length in enumerate(lengths):
            it0, it_end = starts[i], starts[i + 1]
            queue = list(nxt)
            if i + 1 < len(lengths):
                rem = max(it_end - my_it, 0)
                my_next = my_it + (rem + DQ - 1) // DQ * DQ
                kbf = kb0[i + 1] + (my_next - it_end)
                nxt = [kbf + j * DQ for j in range(3)]
            while my_it < it_end:
                kb = kb0[i] + (my_it - it0)
                assert queue[0] == kb, "the scale used is the one of the K block being converted"
                queue = [queue[1], queue[2], kb + 3 * DQ]
                my_it += DQ
            # the group's first block of the next item is what the prefetch assumed
            if i + 1 < len(lengths) and my_it < starts[i + 2]:
                assert nxt[0] == kb0[i + 1] + (my_it - it_end)
