"""Prefill scheduling search: the native implementation and the oracle restatement against tables produced by the
reference's own compiled search (tests/golden/scheduler_dp.npz), and the one-call planner against a walk through
those tables done the way router/manager.py:714-757 does it."""
import os

import numpy as np
import pytest

from loongserve_b200 import scheduler
from oracle import esp_oracle as O

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "scheduler_dp.npz"))
N = int(GOLD["n"])


def _inputs(k):
    lens, room, abc = GOLD[f"c{k}_lens"], GOLD[f"c{k}_room"], GOLD[f"c{k}_abc"]
    R, I = len(lens), len(room)
    best = np.full((R + 1, I + 1), np.inf)
    choice = np.full((R + 1, I + 1, 2), -1, dtype=np.int32)
    return (R, I, best, choice, np.cumsum(lens), np.cumsum(lens ** 2), np.cumsum(1.0 / lens.astype(np.float64)), np.cumsum(room), abc)


def _same_tables(best, choice, k):
    assert np.array_equal(choice, GOLD[f"c{k}_choice"])
    assert best.tobytes() == GOLD[f"c{k}_best"].tobytes()            # costs bit for bit, +inf cells included


@pytest.mark.parametrize("k", range(N))
def test_native_search_matches_reference_tables(k):
    args = _inputs(k)
    scheduler.minimize_prefill_iteration_time(*args)
    _same_tables(args[2], args[3], k)


@pytest.mark.parametrize("k", [k for k in range(N) if len(GOLD[f"c{k}_lens"]) <= 16])
def test_oracle_search_matches_reference_tables(k):
    args = _inputs(k)
    O.minimize_prefill_iteration_time(*args)
    _same_tables(args[2], args[3], k)


@pytest.mark.parametrize("k", range(N))
def test_one_call_planner_matches_walk_through_reference_tables(k):
    lens, room, abc = GOLD[f"c{k}_lens"], GOLD[f"c{k}_room"], GOLD[f"c{k}_abc"]
    best, choice = GOLD[f"c{k}_best"], GOLD[f"c{k}_choice"]
    R, I = len(lens), len(room)
    m = 1 + int(np.argmin(best[R, 1:]))               # first strict minimum, as the loop at manager.py:716-719 finds it
    want, n, longest = [], R, 0.0
    while n > 0:
        b, u = (int(x) for x in choice[n, m])
        seg = lens[n - b:n]
        longest = max(longest, abc[u, 0] + abc[u, 1] * float(seg.sum()) + abc[u, 2] * float((seg ** 2).sum()))
        want.append((slice(n - b, n), slice(m - u, m)))
        n, m = n - b, m - u
    assert m == 0
    got, cost, got_longest = scheduler.plan_prefill_batches(lens, room, abc)
    assert got == want
    assert cost == best[R, 1:].min() and got_longest == longest


def test_native_search_matches_oracle_on_random_small_cases():
    rng = np.random.RandomState(5)
    for _ in range(30):
        R, I = int(rng.randint(1, 9)), int(rng.randint(1, 6))
        lens = np.sort(rng.randint(1, 5000, size=R).astype(np.int64))[::-1].copy()
        room = np.sort(rng.randint(0, 6000, size=I).astype(np.int64))[::-1].copy()
        if room.sum() < lens.sum():
            room[0] += lens.sum() - room.sum()
        abc = np.vstack([[np.nan] * 3, rng.uniform(0.0, 1.0, size=(I, 3)) * [1.0, 1e-3, 1e-7]])
        tables = []
        for fn in (scheduler.minimize_prefill_iteration_time, O.minimize_prefill_iteration_time):
            best = np.full((R + 1, I + 1), np.inf)
            choice = np.full((R + 1, I + 1, 2), -1, dtype=np.int32)
            fn(R, I, best, choice, np.cumsum(lens), np.cumsum(lens ** 2), np.cumsum(1.0 / lens.astype(np.float64)), np.cumsum(room), abc)
            tables.append((best, choice))
        assert tables[0][0].tobytes() == tables[1][0].tobytes() and np.array_equal(tables[0][1], tables[1][1])


def test_planner_rejects_requests_that_do_not_fit():
    abc = np.array([[np.nan] * 3, [0.1, 1e-5, 1e-10]])
    with pytest.raises(RuntimeError):
        scheduler.plan_prefill_batches([100, 50], [120], abc)
    with pytest.raises(TypeError):
        scheduler.minimize_prefill_iteration_time(1, 1, np.full((2, 2), np.inf, dtype=np.float32), np.full((2, 2, 2), -1, dtype=np.int32),
                                                  np.array([5]), np.array([25]), np.array([0.2]), np.array([10]), abc)
