"""GPU parity of the whole decode step: the engine (C ABI) against the CPU oracle decoder and the golden vectors."""
from pathlib import Path

import numpy as np
import pytest

from oracle import binding as orc
from oracle import sched as osched
from tests.decoder_cases import (TINY_CONTEXTS, assert_unbiased, compare_forced_step, free_running_error, mid_config,
                                 tiny_config)

pytestmark = pytest.mark.gpu
GOLD = np.load(Path(__file__).parent / "golden" / "tiny_decode.npz")


def _engine_step(eng, slots, q_lens, tokens):
    nxt, mg = eng.step(slots, q_lens, tokens)
    cfg = eng.cfg
    return {"next": nxt, "margin": mg, "logits": eng.read_logits(),
            "route_idx": [eng.read_routing(l) for l in range(cfg.n_layers)],
            "hidden": [eng.read_hidden(l) for l in range(-1, cfg.n_layers)]}


def _oracle_step(model, sch, slots, q_lens, tokens):
    for s, q in zip(slots, q_lens):
        sch.extend(s, sch.len[s] + q)
    p = sch.pack(slots, q_lens)
    p.update(slots=slots, n_tokens=int(sum(q_lens)))
    return model.step(p, tokens, np.array(sch.tables, np.int32), want_debug=True), p


def _force_all(eng, ref):
    for l in range(eng.cfg.n_layers + 1):
        eng.force_hidden(l, ref["hidden"][l])


def _clear_forcing(eng):
    for l in range(eng.cfg.n_layers + 1):
        eng.force_hidden(l, None)


# Free-running bound.  FP8 activation quantisation amplifies a one-ulp difference (the engine's attention output
# differs from the oracle's in ~0.1 % of its bf16 elements) into percent-level differences one layer later, so a
# free-running step is held to a statistical bound; the tight comparison is the teacher-forced one.
FREE_LOGIT_ABS = {"tiny": 0.1, "mid": 0.75}  # mid: three times the measured 0.24
FREE_HIDDEN_REL = 0.15


def test_tiny_decode_step_matches_golden_and_oracle(gpu):
    import eidola_b200 as eb
    cfg = tiny_config()
    model = orc.Model(cfg)
    model.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    oslots = [sch.admit(L) for L in TINY_CONTEXTS]
    toks = np.array([11, 222, 3333, 4000], np.int32)
    ref, _ = _oracle_step(model, sch, oslots, [1, 1, 1, 1], toks)
    assert np.array_equal(ref["logits"], GOLD["logits0"]) and np.array_equal(ref["route_idx"], GOLD["route_idx0"])

    # (1) teacher-forced: every layer and the head start from the oracle's input
    eng = eb.Engine(cfg)
    eng.kv_fill_synth()
    slots = [eng.admit(L) for L in TINY_CONTEXTS]
    _force_all(eng, ref)
    got = _engine_step(eng, slots, [1, 1, 1, 1], toks)
    assert np.array_equal(eng.block_tables(), GOLD["tables0"])  # integer work: bit-exact against the golden vectors
    assert np.array_equal(got["hidden"][0], GOLD["hidden0"][0])  # embedding gather
    worst_h, worst_l = compare_forced_step(got, ref, cfg, what="tiny forced")
    ms, launches = eng.last_step_stats()
    assert ms > 0 and launches > 20
    eng.close()

    # (2) free-running: the same step with nothing imposed
    eng = eb.Engine(cfg)
    eng.kv_fill_synth()
    slots = [eng.admit(L) for L in TINY_CONTEXTS]
    got = _engine_step(eng, slots, [1, 1, 1, 1], toks)
    dl, rel = free_running_error(got, ref)
    assert dl.max() <= FREE_LOGIT_ABS["tiny"] and rel <= FREE_HIDDEN_REL, (dl, rel)
    assert_unbiased(got["logits"], ref["logits"], "tiny free-running logits")
    assert_unbiased(got["hidden"][-1], ref["hidden"][-1], "tiny free-running hidden")
    assert np.array_equal(got["route_idx"][0], GOLD["route_idx0"][0])  # layer 0 routing sees identical inputs
    print(f"tiny: forced hidden err {worst_h:.4f} logits err {worst_l:.4f}; free logits err {dl.max():.4f} hidden rel {rel:.4f}")


def test_tiny_greedy_64_steps(gpu):
    """Greedy decode for 64 steps, teacher-forced on the golden token stream: the engine's token equals the golden
    one wherever the oracle's top-2 margin exceeds the free-running logit noise; block tables stay bit-exact."""
    import eidola_b200 as eb
    cfg = tiny_config()
    eng = eb.Engine(cfg)
    eng.kv_fill_synth()
    slots = [eng.admit(L) for L in TINY_CONTEXTS]
    toks = np.array([11, 222, 3333, 4000], np.int32)
    matched = clear = clear_matched = 0
    for step in range(64):
        nxt, _ = eng.step(slots, [1, 1, 1, 1], toks)
        want, margin = GOLD["tokens"][step], GOLD["margins"][step]
        for i in range(4):
            matched += int(nxt[i] == want[i])
            if margin[i] > 2 * FREE_LOGIT_ABS["tiny"]:
                clear += 1
                clear_matched += int(nxt[i] == want[i])
        toks = want.copy()
    assert np.array_equal(eng.block_tables(), GOLD["tables_end"])
    assert clear_matched == clear, (clear_matched, clear)
    assert matched >= 0.6 * 256, matched
    print(f"greedy: {matched}/256 tokens equal the golden stream; {clear_matched}/{clear} where the margin is clear")


def test_tiny_greedy_64_steps_free_running(gpu):
    """Greedy decode for 64 steps with the engine's own tokens fed back (nothing imposed).  The golden stream is the
    oracle's own free run, so a sequence can be compared until its first disagreement; that disagreement must sit
    where the oracle's top-2 margin is within the free-running logit noise (two logits each off by at most the
    bound), i.e. the engine never picks a different token at a clear margin."""
    import eidola_b200 as eb
    cfg = tiny_config()
    eng = eb.Engine(cfg)
    eng.kv_fill_synth()
    slots = [eng.admit(L) for L in TINY_CONTEXTS]
    toks = np.array([11, 222, 3333, 4000], np.int32)
    alive = [True] * 4
    agreed = [0] * 4
    for step in range(64):
        nxt, _ = eng.step(slots, [1, 1, 1, 1], toks)
        for i in range(4):
            if not alive[i]:
                continue
            if nxt[i] == GOLD["tokens"][step][i]:
                agreed[i] += 1
            else:
                alive[i] = False
                assert GOLD["margins"][step][i] <= 2 * FREE_LOGIT_ABS["tiny"], (
                    f"sequence {i} leaves the oracle's stream at step {step} where the oracle's margin is "
                    f"{GOLD['margins'][step][i]:.3f}")
        toks = nxt.copy()
    print(f"free-running greedy: steps in agreement with the oracle's stream per sequence {agreed} (of 64)")
    # with N(0, 0.02) random weights the logits are nearly flat, so a sub-noise margin turns up within a few steps
    assert all(a >= 1 for a in agreed)


def test_mid_config_ragged_verify_steps(gpu):
    """Benchmark-shaped layers (hidden 2880, 64q/8kv, top-4 of 8 experts), ragged q_len 1..5, three steps with a
    rejected-draft rollback in between; each step teacher-forced layer by layer against the oracle."""
    import eidola_b200 as eb
    cfg = mid_config()
    eng = eb.Engine(cfg)
    eng.kv_fill_synth()
    model = orc.Model(cfg)
    model.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    ctx = [5, 40, 130, 300, 17, 1000, 64, 2, 511, 128, 33, 250]
    slots = [eng.admit(L) for L in ctx]
    assert slots == [sch.admit(L) for L in ctx]
    rng = np.random.default_rng(0)
    for step, q_lens in enumerate(([1] * 12, [5, 1, 3, 5, 2, 5, 1, 1, 4, 5, 5, 2], [1, 5, 1, 1, 1, 5, 1, 1, 1, 1, 1, 1])):
        T = sum(q_lens)
        toks = rng.integers(0, cfg.vocab, size=T).astype(np.int32)
        ref, _ = _oracle_step(model, sch, slots, q_lens, toks)
        _force_all(eng, ref)
        got = _engine_step(eng, slots, q_lens, toks)
        assert np.array_equal(eng.block_tables(), np.array(sch.tables, np.int32))
        wh, wl = compare_forced_step(got, ref, cfg, what=f"mid step {step}")
        print(f"mid step {step}: forced hidden err {wh:.4f} logits err {wl:.4f}")
        if step == 1:  # reject some draft tokens: roll three sequences back
            for s, drop in ((slots[0], 3), (slots[3], 4), (slots[5], 1)):
                eng.truncate(s, eng.seq_len(s) - drop)
                sch.truncate(s, sch.len[s] - drop)
    _clear_forcing(eng)
    q_lens = [1] * 12
    toks = rng.integers(0, cfg.vocab, size=12).astype(np.int32)
    ref, _ = _oracle_step(model, sch, slots, q_lens, toks)
    got = _engine_step(eng, slots, q_lens, toks)
    dl, rel = free_running_error(got, ref)
    ml, rl = assert_unbiased(got["logits"], ref["logits"], "mid free-running logits")
    mh, rh = assert_unbiased(got["hidden"][-1], ref["hidden"][-1], "mid free-running hidden")
    print(f"mid free-running: logits err max {dl.max():.4f} mean {ml:+.2e} rms {rl:.2e}; hidden rel {rel:.4f} mean {mh:+.2e} rms {rh:.2e}")
    assert dl.max() <= FREE_LOGIT_ABS["mid"] and rel <= FREE_HIDDEN_REL, (dl, rel)


def test_refused_step_leaves_no_trace(gpu):
    import eidola_b200 as eb
    cfg = tiny_config(num_pages=6, max_pages_per_seq=4)
    eng = eb.Engine(cfg)
    a, b = eng.admit(40), eng.admit(47)  # 3 + 3 pages: pool exhausted
    before = eng.block_tables().copy()
    with pytest.raises(eb.EbError) as e:
        eng.step([a, b], [1, 2], [1, 2, 3])  # b would need a 4th page
    assert e.value.code == -3
    assert np.array_equal(eng.block_tables(), before) and eng.seq_len(a) == 40 and eng.seq_len(b) == 47
    with pytest.raises(eb.EbError):
        eng.step([a, a], [1, 1], [1, 2])
    with pytest.raises(eb.EbError):
        eng.step([a], [1], [cfg.vocab])
    eng.step([a], [1], [5])
    assert eng.seq_len(a) == 41


def test_window_ring_is_bit_identical_to_full_pages(gpu):
    """Sliding-window layers that keep only a ring of pages per sequence produce the same tokens and logits as
    layers that keep the whole context: 170 decode steps from empty contexts (the ring of 10 pages wraps) and
    verify steps with rollbacks in between."""
    import eidola_b200 as eb
    engines = []
    for ring in (0, 1):
        cfg = tiny_config(window_ring=ring, num_pages=96, max_pages_per_seq=24)
        eng = eb.Engine(cfg)
        slots = [eng.admit(0) for _ in range(4)]
        engines.append((eng, slots))
    toks = np.array([1, 2, 3, 4], np.int32)
    for step in range(170):
        outs = []
        for eng, slots in engines:
            if step % 23 == 7:  # a verify step with 5 tokens per sequence, then reject three of them
                nxt, _ = eng.step(slots, [5] * 4, np.repeat(toks, 5))
                for s in slots:
                    eng.truncate(s, eng.seq_len(s) - 3)
                nxt = nxt[4::5]
            else:
                nxt, _ = eng.step(slots, [1] * 4, toks)
            outs.append((nxt.copy(), eng.read_logits()))
        assert np.array_equal(outs[0][0], outs[1][0]), f"step {step}"
        assert np.array_equal(outs[0][1], outs[1][1]), f"step {step}"
        toks = outs[0][0]
    mem_full, mem_ring = engines[0][0].memory()["kv"], engines[1][0].memory()["kv"]
    assert mem_ring < mem_full


def test_page_rings_refuse_a_cut_they_no_longer_cover(gpu):
    """Sliding-window layers with page rings hold the window plus one chunk: rolling back a few rejected drafts is fine, a
    cut far below the longest the sequence has been is refused (the ring pages there have been overwritten) and changes
    nothing; without rings any cut is fine."""
    import eidola_b200 as eb
    for ring in (1, 0):
        cfg = tiny_config(window_ring=ring, num_pages=96, max_pages_per_seq=40, max_tokens=20)
        eng = eb.Engine(cfg)
        eng.kv_fill_synth()
        slot = eng.admit(40)
        rng = np.random.default_rng(1)
        for _ in range(30):  # 150 more tokens: far more than window + chunk
            eng.step([slot], [5], rng.integers(0, cfg.vocab, size=5).astype(np.int32))
        assert eng.seq_len(slot) == 190
        eng.truncate(slot, 187)  # rejected drafts
        assert eng.seq_len(slot) == 187
        if ring:
            with pytest.raises(eb.EbError) as err:
                eng.truncate(slot, 20)
            assert "ring" in str(err.value) and eng.seq_len(slot) == 187
        else:
            eng.truncate(slot, 20)
            assert eng.seq_len(slot) == 20
        eng.step([slot], [1], np.array([3], np.int32))
        assert int(eb.status_read()) == 0
