"""CPU: the oracle decoder reproduces the committed golden vectors of the tiny decode configuration, and basic
invariants of the decoder hold (packing order does not matter, a windowed layer ignores old tokens)."""
import numpy as np

from oracle import binding as orc
from oracle import sched as osched
from tests.decoder_cases import TINY_CONTEXTS, tiny_config
from tests.golden.make_golden import run_tiny
from pathlib import Path

GOLD = np.load(Path(__file__).parent / "golden" / "tiny_decode.npz")


def test_oracle_reproduces_golden():
    cfg, first, out = run_tiny(steps=8)
    assert np.array_equal(out["tables0"], GOLD["tables0"])
    assert np.array_equal(out["positions0"], GOLD["positions0"]) and GOLD["positions0"].tolist() == TINY_CONTEXTS
    assert np.array_equal(first["route_idx"], GOLD["route_idx0"])
    assert np.array_equal(first["logits"], GOLD["logits0"])
    assert np.array_equal(first["hidden"], GOLD["hidden0"])
    assert np.array_equal(np.stack(out["tokens"]), GOLD["tokens"][:8])
    assert np.array_equal(np.stack(out["margins"]), GOLD["margins"][:8])


def test_golden_block_tables_are_shuffled_and_disjoint():
    t = GOLD["tables0"]
    used = t[t >= 0]
    assert len(used) == len(set(used.tolist())) == sum((L + 1 + 15) // 16 for L in TINY_CONTEXTS)
    assert not np.array_equal(used, np.sort(used))


def test_sequences_are_independent_of_batch_composition():
    """A sequence's logits do not depend on which other sequences share the step, except through the shared
    128-token activation scale block -- so compare a step of one sequence with itself under another slot order."""
    cfg = tiny_config()
    a, b = orc.Model(cfg), orc.Model(cfg)
    a.kv_fill_synth()
    b.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    slots = [sch.admit(L) for L in TINY_CONTEXTS]
    for s in slots:
        sch.extend(s, sch.len[s] + 1)
    bt = np.array(sch.tables, np.int32)
    toks = np.array([11, 222, 3333, 4000], np.int32)
    p = sch.pack(slots, [1, 1, 1, 1])
    p.update(slots=slots, n_tokens=4)
    r1 = a.step(p, toks, bt)
    order = [2, 0, 3, 1]
    p2 = sch.pack([slots[i] for i in order], [1, 1, 1, 1])
    p2.update(slots=[slots[i] for i in order], n_tokens=4)
    r2 = b.step(p2, toks[order], bt)
    assert np.array_equal(r2["logits"], r1["logits"][order])
    assert np.array_equal(r2["next"], r1["next"][order])
