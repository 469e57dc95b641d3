"""The host scheduler against its pure-Python restatement: block tables, packing and plans are bit-exact.

Style follows the reference's planner tests (crates/eidola-app-core/src/local_models.rs:2255-2310): a pure
planner, injected inputs, refusal without side effects.
"""
import numpy as np
import pytest

import eidola_b200 as eb
from oracle import sched as osched


def _same_tables(s, o):
    assert np.array_equal(s.block_tables(), np.array(o.tables, np.int32))
    assert s.free_pages() == len(o.free)


def test_shuffled_pages_match_oracle_and_are_a_permutation():
    s = eb.Scheduler(64, 16, 4, 16, seed=0)
    o = osched.Sched(64, 16, 4, 16, 0)
    a = s.admit(250)
    assert a == o.admit(250) == 0
    _same_tables(s, o)
    row = s.block_tables()[0, :16]
    assert len(set(row.tolist())) == 16 and not np.array_equal(row, np.sort(row))


def test_tiny_decode_config_block_tables():
    """Contexts {7,33,128,250}, page 16, seed 0: the tiny CPU decode configuration."""
    s = eb.Scheduler(40, 16, 4, 17, seed=0)
    o = osched.Sched(40, 16, 4, 17, 0)
    for L in (7, 33, 128, 250):
        assert s.admit(L) == o.admit(L)
    _same_tables(s, o)
    for slot in range(4):
        s.extend(slot, s.seq_len(slot) + 1)
        o.extend(slot, o.len[slot] + 1)
    _same_tables(s, o)
    p = s.pack([0, 1, 2, 3], [1, 1, 1, 1])
    po = o.pack([0, 1, 2, 3], [1, 1, 1, 1])
    assert p["positions"].tolist() == [7, 33, 128, 250] == po["positions"]
    assert p["ctx_lens"].tolist() == [8, 34, 129, 251] == po["ctx_lens"]


def test_refusal_has_no_side_effects():
    s = eb.Scheduler(8, 16, 2, 8, seed=3)
    a = s.admit(100)  # 7 pages
    before = s.block_tables().copy()
    with pytest.raises(eb.EbError) as e:
        s.admit(40)  # needs 3, 1 free
    assert e.value.code == -3
    with pytest.raises(eb.EbError):
        s.extend(a, 200)
    assert np.array_equal(s.block_tables(), before) and s.free_pages() == 1 and s.seq_len(a) == 100
    s.extend(a, 128)
    assert s.free_pages() == 0
    b = s.admit(0)
    assert b == 1
    with pytest.raises(eb.EbError) as e:
        s.admit(0)  # slots exhausted
    assert e.value.code == -3
    with pytest.raises(eb.EbError) as e:
        s.release(5)
    assert e.value.code == -5


def test_random_walk_matches_oracle():
    rng = np.random.default_rng(11)
    s = eb.Scheduler(300, 16, 12, 40, seed=5)
    o = osched.Sched(300, 16, 12, 40, 5)
    live = []
    for _ in range(400):
        op = rng.integers(0, 4)
        if op == 0 or not live:
            L = int(rng.integers(0, 500))
            want = o.admit(L)
            if want is None:
                with pytest.raises(eb.EbError):
                    s.admit(L)
            else:
                assert s.admit(L) == want
                live.append(want)
        elif op == 1:
            slot = live[int(rng.integers(len(live)))]
            n = o.len[slot] + int(rng.integers(0, 40))
            if o.extend(slot, n):
                s.extend(slot, n)
            else:
                with pytest.raises(eb.EbError):
                    s.extend(slot, n)
        elif op == 2:
            slot = live[int(rng.integers(len(live)))]
            n = int(rng.integers(0, o.len[slot] + 1))
            o.truncate(slot, n)
            s.truncate(slot, n)
        else:
            slot = live.pop(int(rng.integers(len(live))))
            o.release(slot)
            s.release(slot)
        _same_tables(s, o)
    if live:
        slots = live[:5]
        q_lens = [min(max(1, o.len[x]), 1 + i % 5) for i, x in enumerate(slots)]
        ok = all(o.len[x] >= q for x, q in zip(slots, q_lens))
        if ok:
            p, po = s.pack(slots, q_lens), o.pack(slots, q_lens)
            for k in ("q_off", "ctx_lens", "tok_seq", "tok_slot", "positions"):
                assert p[k].tolist() == po[k], k


@pytest.mark.parametrize("window", [0, 128])
@pytest.mark.parametrize("chunk", [0, 8, 64])
@pytest.mark.parametrize("ppi", [1, 4])
def test_attn_plan_matches_oracle(window, chunk, ppi):
    rng = np.random.default_rng(2)
    ctx = rng.integers(1, 5000, size=37).astype(np.int32)
    ql = np.minimum(ctx, rng.integers(1, 6, size=37)).astype(np.int32)
    got = eb.attn_plan(ctx, ql, 16, window, 148, chunk, ppi)
    want = osched.attn_plan(ctx.tolist(), ql.tolist(), 16, window, 148, chunk, ppi)
    assert got["items"].tolist() == [list(x) for x in want["items"]]
    assert got["seq_part"].tolist() == want["seq_part"] and got["n_parts"] == want["n_parts"]
    # every visible page of every sequence is covered exactly once
    cover = {}
    for seq, pb, pe, _ in got["items"].tolist():
        cover.setdefault(seq, []).append((pb, pe))
    for i in range(37):
        runs = sorted(cover[i])
        lo = max(0, ctx[i] - ql[i] - window + 1) // 16 if window else 0
        assert runs[0][0] == lo and runs[-1][1] == (ctx[i] + 15) // 16
        assert all(a[1] == b[0] for a, b in zip(runs, runs[1:]))


def test_attn_plan_leaves_short_ranges_whole_when_they_fill_the_sms():
    rng = np.random.default_rng(3)
    ctx = rng.integers(128, 8192, size=256).astype(np.int32)
    ql = np.ones(256, np.int32)
    got = eb.attn_plan(ctx, ql, 16, 128, 148)
    want = osched.attn_plan(ctx.tolist(), ql.tolist(), 16, 128, 148)
    assert got["items"].tolist() == [list(x) for x in want["items"]]
    assert got["n_parts"] == 256 and len(got["items"]) == 256  # one item per sequence: no merge launch
    full = eb.attn_plan(ctx, ql, 16, 0, 148)  # full layers of the same batch are still split
    assert len(full["items"]) > 256
    few = eb.attn_plan(ctx[:40], ql[:40], 16, 128, 148)  # fewer sequences than SMs: split for parallelism
    assert len(few["items"]) > 40


def test_attn_plan_sm_count_follows_the_kernel_choice():
    """The planner's granularity hint: one CTA per item for decode shapes and short windows, one CTA per (item, KV head),
    two per SM, for verify shapes on long items; and a plan made with the hint has about 4 x 2 x SMs / n_kv items."""
    sm = 148
    assert eb.attn_plan_sm_count(sm, 1, 64, 8, 0) == sm
    assert eb.attn_plan_sm_count(sm, 2, 64, 8, 0) == sm            # 16 rows still fit the decode tile
    assert eb.attn_plan_sm_count(sm, 5, 64, 8, 0) == 2 * sm // 8
    assert eb.attn_plan_sm_count(sm, 5, 16, 2, 0) == sm
    assert eb.attn_plan_sm_count(sm, 5, 8, 1, 0) == 2 * sm
    assert eb.attn_plan_sm_count(sm, 5, 64, 8, 128) == sm          # short window: the one-CTA-per-item kernel
    assert eb.attn_plan_sm_count(sm, 5, 64, 8, 4096) == 2 * sm // 8
    assert eb.attn_plan_sm_count(2, 6, 64, 8, 0) == 1              # never below one
    rng = np.random.default_rng(5)
    ctx = rng.integers(2048, 8192, size=256).astype(np.int32)
    ql = np.full(256, 5, np.int32)
    coarse = eb.attn_plan(ctx, ql, 16, 0, eb.attn_plan_sm_count(sm, 5, 64, 8, 0))
    fine = eb.attn_plan(ctx, ql, 16, 0, sm)
    assert len(coarse["items"]) < len(fine["items"])
    assert 256 <= len(coarse["items"]) <= 2 * 256                 # 4 x 37 = 148 wanted, one item per sequence at least


def test_attn_plan_rejects_bad_input():
    with pytest.raises(eb.EbError):
        eb.attn_plan([5], [6], 16, 0, 148)
