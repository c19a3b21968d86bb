"""The static memory planner against the reference's golden vectors
(test/mlir/unittests/Transforms/StaticMemoryPlanning.cpp:14-205) and as a property test.  Host only."""
import random

import pytest

from gc_b200 import api

F, Z = "free", "zero_offset"


def test_best_fit_and_hot_first_golden():
    # TestStaticMemoryPlanning: nine buffers, three layers of reuse
    tr = [(0, 100), (1, 120), (2, 100), (0, 0), (3, 50), (4, 60), (2, 0), (4, 0), (8, 100), (8, 0), (5, 60), (5, 0), (1, 0),
          (6, 350), (3, 0), (7, 100)]
    want = {0: 0, 1: 160, 2: 280, 3: 0, 4: 100, 5: 100, 6: 100, 7: 0, 8: 280}
    for hot in (False, True):
        total, off, reused = api.schedule_memory(tr, 1, hot)
        assert total == 450 and off == want and reused == {}


GOLDEN_INPLACE = [
    # (traces, hints, expected offsets, expected total, expected selection) — TestStaticMemoryPlanningInplace
    ([(1, 120), (2, 100), (3, 200), (1, 0), (2, 0), (3, 0), (4, 220), (4, 0)], {3: [(1, F), (2, F)]},
     {1: 0, 2: 120, 3: 0, 4: 0}, 220, {3: [1, 2]}),                                      # merge + split
    ([(1, 120), (2, 100), (4, 250), (3, 250), (1, 0), (2, 0), (3, 0), (4, 0)], {3: [(1, F), (2, F)]},
     {1: 0, 2: 120, 3: 0, 4: 250}, 500, {3: [1, 2]}),                                    # extend
    ([(1, 120), (2, 100), (3, 150), (4, 50), (5, 10), (1, 0), (2, 0), (3, 0), (4, 0), (5, 0)],
     {3: [(1, F), (2, F)], 4: [(1, F), (2, F)]}, {1: 0, 2: 120, 3: 0, 4: 150, 5: 220}, 230, {3: [1, 2], 4: [2]}),
    ([(1, 120), (2, 100), (3, 150), (4, 50), (5, 10), (1, 0), (2, 0), (3, 0), (4, 0), (5, 0)],
     {3: [(1, F), (2, Z)], 4: [(1, F), (2, F)]}, {1: 0, 2: 150, 3: 0, 4: 150, 5: 250}, 260, {3: [1], 4: [2]}),
    ([(1, 120), (2, 100), (3, 150), (4, 50), (5, 10), (1, 0), (2, 0), (3, 0), (4, 0), (5, 0)],
     {3: [(1, F), (2, F)], 4: [(1, F), (2, Z)]}, {1: 0, 2: 120, 3: 0, 4: 220, 5: 270}, 280, {3: [1, 2]}),
    ([(1, 120), (2, 100), (3, 150), (2, 0), (4, 150), (5, 10), (1, 0), (3, 0), (4, 0), (5, 0)], {4: [(1, F)]},
     {1: 0, 2: 120, 3: 220, 4: 0, 5: 150}, 370, {4: [1]}),                               # merge free to the right
    ([(1, 120), (2, 100), (3, 100), (4, 120), (1, 0), (2, 0), (3, 0), (4, 0), (5, 200), (5, 0)],
     {3: [(1, F), (2, F)], 4: [(1, F), (2, F)]}, {1: 0, 2: 120, 3: 120, 4: 0, 5: 0}, 220, {3: [2], 4: [1]}),   # perfect matches
    ([(1, 120), (2, 100), (3, 100), (4, 120), (1, 0), (2, 0), (3, 0), (4, 0), (5, 200), (5, 0)],
     {3: [(1, F)], 4: [(2, F)]}, {1: 0, 2: 120, 3: 0, 4: 120, 5: 0}, 240, {3: [1], 4: [2]}),                    # selected inputs
]


@pytest.mark.parametrize("case", range(len(GOLDEN_INPLACE)))
def test_inplace_golden(case):
    tr, hints, want_off, want_total, want_sel = GOLDEN_INPLACE[case]
    total, off, reused = api.schedule_memory(tr, 1, False, hints)
    assert (total, off, reused) == (want_total, want_off, want_sel)


@pytest.mark.parametrize("hot", [False, True])
@pytest.mark.parametrize("seed", range(8))
def test_random_traces_never_overlap_and_respect_alignment(seed, hot):
    rnd = random.Random(seed)
    live, tr, spans, t = {}, [], {}, 0
    for b in range(1, 120):
        while live and (len(live) > 6 or rnd.random() < 0.4):
            victim = rnd.choice(sorted(live))
            tr.append((victim, 0)); spans[victim][2] = t; t += 1
            del live[victim]
        size = rnd.choice([1, 7, 64, 100, 1000, 4096, 333])
        tr.append((b, size)); live[b] = size; spans[b] = [size, t, None]; t += 1
    for victim in sorted(live):
        tr.append((victim, 0)); spans[victim][2] = t; t += 1
    align = 64
    total, off, _ = api.schedule_memory(tr, align, hot)
    up = lambda v: (v + align - 1) // align * align
    assert all(o % align == 0 for o in off.values())
    assert total >= max(off[b] + up(s[0]) for b, s in spans.items())
    ids = sorted(spans)
    for i, a in enumerate(ids):
        for b in ids[i + 1:]:
            sa, sb = spans[a], spans[b]
            if sa[1] < sb[2] and sb[1] < sa[2]:                                        # lifetimes overlap
                assert off[a] + up(sa[0]) <= off[b] or off[b] + up(sb[0]) <= off[a], (a, b)
    # reuse happens: far less than the sum of all buffers
    assert total < sum(up(s[0]) for s in spans.values()) / 3


def test_release_of_unknown_buffer_is_an_error():
    with pytest.raises(ValueError):
        api.schedule_memory([(1, 0)])
