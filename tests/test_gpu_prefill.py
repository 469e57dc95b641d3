"""GPU: chunked prefill through the decode / verify kernels -- the cache the engine fills itself must be the cache the
oracle fills, and chunking must not matter."""
import numpy as np
import pytest

from oracle import binding as orc
from oracle import sched as osched
from tests.decoder_cases import assert_unbiased, tiny_config
from tests.helpers import bf16_to_f32

pytestmark = pytest.mark.gpu

PROMPTS = [7, 33, 12, 50]


def _prompts(cfg, seed=3):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, cfg.vocab, size=n).astype(np.int32) for n in PROMPTS]


def _oracle_prefill(cfg, prompts, chunk_cap):
    """The oracle fed the chunks eb_engine_prefill makes (sequences in order, each taking what it still needs, at most
    chunk_cap, or what is left of the step's max_tokens rows unless that is less than one attention entry): returns
    (first generated tokens, margins, the model and scheduler afterwards, steps)."""
    model = orc.Model(cfg)
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    slots = [sch.admit(0) for _ in prompts]
    done = [0] * len(prompts)
    first, margin = [None] * len(prompts), [None] * len(prompts)
    steps, start = 0, 0
    while any(d < len(p) for d, p in zip(done, prompts)):
        b, q, rows, skipped = [], [], 0, False
        for k in range(len(prompts)):
            i = (start + k) % len(prompts)
            rem = len(prompts[i]) - done[i]
            if rem <= 0:
                continue
            qq = min(rem, chunk_cap, cfg.max_tokens - rows)
            if qq < rem and qq < min(rem, cfg.max_q_len):
                skipped = True
                continue
            b.append(i)
            q.append(qq)
            rows += qq
        toks = np.concatenate([prompts[i][done[i]:done[i] + qq] for i, qq in zip(b, q)])
        for i, qq in zip(b, q):
            sch.extend(slots[i], sch.len[slots[i]] + qq)
        p = sch.pack([slots[i] for i in b], q)
        p.update(slots=[slots[i] for i in b], n_tokens=int(sum(q)))
        r = model.step(p, toks, np.array(sch.tables, np.int32))
        steps += 1
        row = 0
        for i, qq in zip(b, q):
            row += qq
            done[i] += qq
            if done[i] == len(prompts[i]):
                first[i], margin[i] = int(r["next"][row - 1]), float(r["margin"][row - 1])
        if skipped:
            start = (start + 1) % len(prompts)
    return first, margin, model, sch, slots, steps


@pytest.mark.parametrize("kw", [dict(), dict(max_tokens=128), dict(max_tokens=128, window_ring=1), dict(max_tokens=40, window_ring=1)],
                         ids=["steps_of_20_rows", "whole_prompts_in_one_step", "one_step_window_rings", "steps_of_40_rows_window_rings"])
def test_prefill_fills_the_cache_the_oracle_fills(gpu, kw):
    import eidola_b200 as eb
    cfg = tiny_config(**kw)
    prompts = _prompts(cfg)
    eng = eb.Engine(cfg)
    cap = eng.chunk_tokens()
    assert cap == (min(cfg.max_tokens, 256) if cfg.window_ring else cfg.max_tokens)
    want_first, want_margin, model, sch, oslots, want_steps = _oracle_prefill(cfg, prompts, cap)
    slots = [eng.admit(0) for _ in prompts]
    first, margin, steps, ms = eng.prefill(slots, prompts)
    assert steps == want_steps and ms > 0
    if cfg.max_tokens >= sum(PROMPTS):
        assert steps == 1
    assert [eng.seq_len(s) for s in slots] == PROMPTS
    assert np.array_equal(eng.block_tables(), np.array(sch.tables, np.int32))  # the same pages in the same order
    for i in range(len(prompts)):
        if want_margin[i] > 0.05:
            assert first[i] == want_first[i], (i, first[i], want_first[i], want_margin[i])
    # one more decode step on both: the logits depend on every K and V the prefill wrote
    toks = np.array(want_first, np.int32)
    nxt, _ = eng.step(slots, [1] * 4, toks)
    for s in oslots:
        sch.extend(s, sch.len[s] + 1)
    p = sch.pack(oslots, [1] * 4)
    p.update(slots=oslots, n_tokens=4)
    ref = model.step(p, toks, np.array(sch.tables, np.int32))
    err = np.abs(bf16_to_f32(eng.read_logits()) - bf16_to_f32(ref["logits"])).max()
    print(f"prefill {kw}: {steps} steps; decode step after it: max |logit diff| vs oracle {err:.4f}")
    assert err <= 0.1
    assert int(eb.status_read()) == 0


def test_prefill_chunking_does_not_matter(gpu):
    """Prefill chunks and token-by-token decode steps leave the same context behind: the next step's logits agree
    (different kernels shapes computed them, so to rounding, not bit for bit)."""
    import eidola_b200 as eb
    cfg = tiny_config()
    prompts = _prompts(cfg, seed=4)
    a = eb.Engine(cfg)
    sa = [a.admit(0) for _ in prompts]
    first_a, _, _, _ = a.prefill(sa, prompts)
    b = eb.Engine(cfg)
    sb = [b.admit(0) for _ in prompts]
    for t in range(max(PROMPTS)):
        live = [i for i in range(4) if t < PROMPTS[i]]
        b.step([sb[i] for i in live], [1] * len(live), [int(prompts[i][t]) for i in live])
    toks = np.array(first_a, np.int32)
    a.step(sa, [1] * 4, toks)
    b.step(sb, [1] * 4, toks)
    err = np.abs(bf16_to_f32(a.read_logits()) - bf16_to_f32(b.read_logits())).max()
    print(f"chunked vs token-by-token prefill: max |logit diff| {err:.4f}")
    # 50 positions of K and V were computed by differently shaped kernels and requantised on the way: noise, not bias
    assert err <= 0.25
    assert_unbiased(a.read_logits(), b.read_logits(), "chunked vs token-by-token prefill")
    with pytest.raises(eb.EbError):
        a.prefill(sa[:1], [np.zeros(0, np.int32)])
