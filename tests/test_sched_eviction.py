"""CPU: admission with eviction at page granularity against the reference's own planner cases.

The reference's `plan_evictions` (crates/eidola-app-core/src/local_models.rs:653-701) is pinned by unit tests at
local_models.rs:2255-2310.  Their cases are restated here with one page per GiB (budget 16, footprints 4/5/4, ...):
the scheduler's planner must choose the same victims in the same order, and refuse in the same situations without
changing anything.  oracle/sched.py holds the Python restatement of the reference function; both are checked."""
import ctypes as C

import numpy as np
import pytest

from oracle import sched as osched

PAGE = 16


def _sched(budget, max_seqs=8):
    import eidola_b200 as eb  # host-only entry points: no GPU needed
    return eb.Scheduler(budget, PAGE, max_seqs, budget, seed=1)


def _load(s, entries):
    """entries: (pages, last_used, pinned, in_flight) -> slots in order."""
    from eidola_b200 import capi
    slots = []
    for pages, used, pinned, busy in entries:
        slot = s.admit(pages * PAGE)
        capi.call("eb_sched_touch", s._h, C.c_int32(slot), C.c_int64(used))
        capi.call("eb_sched_set_flags", s._h, C.c_int32(slot), C.c_int32(int(pinned)), C.c_int32(int(busy)))
        slots.append(slot)
    return slots


def _plan(s, pages):
    from eidola_b200 import capi
    out = (C.c_int32 * 16)()
    n = C.c_int32(0)
    rc = capi.call_rc("eb_sched_plan_evictions", s._h, C.c_int32(pages * PAGE), out, C.c_int32(16), C.byref(n))
    return rc, [int(out[i]) for i in range(n.value)]


def _ref(required, budget, entries, slots):
    return osched.plan_evictions(required, budget, [(slots[i], e[0], e[1], e[2], e[3]) for i, e in enumerate(entries)])


def test_no_eviction_when_it_fits():          # local_models.rs:2255-2261
    entries = [(4, 1, False, False)]
    s = _sched(16)
    slots = _load(s, entries)
    assert _plan(s, 3) == (0, []) and _ref(3, 16, entries, slots) == []


def test_evicts_lru_first_and_only_as_needed():   # local_models.rs:2263-2286
    entries = [(4, 300, False, False), (5, 100, False, False), (4, 200, False, False)]  # a, b, c
    s = _sched(16)
    a, b, c = _load(s, entries)
    assert _plan(s, 6) == (0, [b]) and _ref(6, 16, entries, [a, b, c]) == [b]
    assert _plan(s, 10) == (0, [b, c]) and _ref(10, 16, entries, [a, b, c]) == [b, c]
    before = s.block_tables().copy()
    assert s.free_pages() == 3 and np.array_equal(s.block_tables(), before)   # planning changes nothing


def test_never_touches_pinned_or_in_flight():     # local_models.rs:2288-2304
    entries = [(6, 1, True, False), (6, 2, False, True), (3, 900, False, False)]  # pinned-old, busy-old, idle
    s = _sched(16)
    slots = _load(s, entries)
    assert _plan(s, 4) == (0, [slots[2]]) and _ref(4, 16, entries, slots) == [slots[2]]
    import eidola_b200 as eb
    rc, victims = _plan(s, 8)
    assert rc == -3 and victims == [] and "pinned or in-use" in eb.capi.last_error()
    assert _ref(8, 16, entries, slots) == "held"
    assert s.free_pages() == 1


def test_refuses_more_than_the_budget():          # local_models.rs:2306-2310
    import eidola_b200 as eb
    s = _sched(16)
    rc, _ = _plan(s, 20)
    assert rc == -3 and "budget" in eb.capi.last_error()
    assert osched.plan_evictions(20, 16, []) == "budget"


def test_admit_evicting_is_plan_and_reserve_in_one_step():   # local_models.rs:441-485 (reserve_engine)
    from eidola_b200 import capi
    entries = [(4, 300, False, False), (5, 100, False, False), (4, 200, False, False)]
    s = _sched(16)
    a, b, c = _load(s, entries)
    out, n, slot = (C.c_int32 * 16)(), C.c_int32(0), C.c_int32(-1)
    capi.call("eb_sched_admit_evicting", s._h, C.c_int32(10 * PAGE), C.c_int64(1000), C.byref(slot), out, C.c_int32(16), C.byref(n))
    assert [out[i] for i in range(n.value)] == [b, c] and s.seq_len(slot.value) == 10 * PAGE and s.seq_len(a) == 4 * PAGE
    assert s.free_pages() == 16 - 4 - 10
    # a request that cannot be met leaves the pool exactly as it was
    capi.call("eb_sched_set_flags", s._h, C.c_int32(a), C.c_int32(1), C.c_int32(-1))
    capi.call("eb_sched_set_flags", s._h, slot, C.c_int32(-1), C.c_int32(1))
    before = s.block_tables().copy()
    rc = capi.call_rc("eb_sched_admit_evicting", s._h, C.c_int32(5 * PAGE), C.c_int64(1001), C.byref(slot), out, C.c_int32(16), C.byref(n))
    assert rc == -3 and np.array_equal(s.block_tables(), before) and s.free_pages() == 2


@pytest.mark.parametrize("seed", range(6))
def test_random_pools_match_the_restated_reference_planner(seed):
    rng = np.random.default_rng(seed)
    budget = 40
    s = _sched(budget, max_seqs=12)
    entries = []
    while sum(e[0] for e in entries) < budget - 6 and len(entries) < 9:
        entries.append((int(rng.integers(1, 7)), int(rng.integers(0, 50)) * 10 + len(entries), bool(rng.random() < 0.25), bool(rng.random() < 0.25)))
    entries = [e for i, e in enumerate(entries) if sum(x[0] for x in entries[:i + 1]) <= budget]
    slots = _load(s, entries)
    for need in (1, 5, 9, 17, 30, 41):
        rc, victims = _plan(s, need)
        want = _ref(need, budget, entries, slots)
        if isinstance(want, str):
            assert rc == -3, (need, want)
        else:
            assert rc == 0 and victims == want, (need, victims, want)
