"""GPU parity on the shapes the benchmarks run, teacher-forced layer by layer against the CPU oracle.

The small decoder cases never reach the kernels the headline configurations dispatch to: the 201088-row LM head at
256 tokens (the 128-token x 256-row GEMM), 32 experts with 1024 routed rows, 128 experts with 10240 routed rows, the
router above 640 tokens.  Here one layer pair + head of the 20b-shaped decoder and one layer of the 120b-shaped
verify step run at the benchmark's own widths and token counts; only the context lengths are shorter (U[16,1500]
instead of thousands), which keeps the oracle's attention to seconds -- long contexts are covered by the attention
tests.  Building the oracle's weights (billions of seeded values) takes most of the time of these tests."""
import numpy as np
import pytest

from oracle import binding as orc
from oracle import sched as osched
from tests.decoder_cases import compare_forced_step

pytestmark = pytest.mark.gpu


def _forced_step(cfg, ctx, q_lens, seed, what):
    import eidola_b200 as eb
    n = len(ctx)
    model = orc.Model(cfg)
    model.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    slots = [sch.admit(int(L)) for L in ctx]
    for s, q in zip(slots, q_lens):
        sch.extend(s, sch.len[s] + q)
    T = int(sum(q_lens))
    p = sch.pack(slots, q_lens)
    p.update(slots=slots, n_tokens=T)
    toks = np.random.default_rng(seed).integers(0, cfg.vocab, size=T).astype(np.int32)
    ref = model.step(p, toks, np.array(sch.tables, np.int32), want_debug=True)
    del model
    eng = eb.Engine(cfg)
    eng.kv_fill_synth()
    assert [eng.admit(int(L)) for L in ctx] == slots
    for l in range(cfg.n_layers + 1):
        eng.force_hidden(l, ref["hidden"][l])
    nxt, mg = eng.step(slots, q_lens, toks)
    got = {"next": nxt, "margin": mg, "logits": eng.read_logits(),
           "route_idx": [eng.read_routing(l) for l in range(cfg.n_layers)],
           "hidden": [eng.read_hidden(l) for l in range(-1, cfg.n_layers)]}
    assert np.array_equal(eng.block_tables(), np.array(sch.tables, np.int32))
    assert np.array_equal(got["hidden"][0], ref["hidden"][0])  # embedding gather: bit-exact
    exact = sum(int(np.array_equal(got["route_idx"][l], ref["route_idx"][l])) for l in range(cfg.n_layers))
    wh, wl = compare_forced_step(got, ref, cfg, what=what)
    agree = float((nxt == ref["next"]).mean())
    print(f"{what}: routing bit-exact in {exact}/{cfg.n_layers} layers, forced hidden err {wh:.4f}, logits err {wl:.4f}, "
          f"greedy tokens equal on {agree:.3f} of {T} rows")
    eng.close()
    assert eb.status_read() == 0
    return got, ref


def test_20b_shaped_layer_pair_and_full_vocabulary_head(gpu):
    """256 sequences x 1 token, hidden 2880, 64q/8kv, 32 experts top-4 (1024 routed rows), vocabulary 201088."""
    from eidola_b200.capi import make_config
    n = 256
    ctx = np.random.default_rng(4).integers(16, 1500, size=n)
    cfg = make_config(n_layers=2, hidden=2880, n_q_heads=64, n_kv_heads=8, window=128, n_experts=32, top_k=4, inter=2880,
                      vocab=201088, num_pages=int(((ctx + 1 + 16) // 16 + 1).sum()) + 8, max_seqs=n, max_pages_per_seq=100,
                      max_tokens=n, max_q_len=1, seed=4, debug=1)
    got, ref = _forced_step(cfg, ctx, [1] * n, seed=0, what="20b-shaped layer pair + head")
    # every expert is hit at 1024 routed rows, as the benchmark's byte count assumes
    assert len(np.unique(ref["route_idx"][0])) == 32


def test_120b_shaped_verify_layer(gpu):
    """512 sequences x q_len 5 = 2560 rows, 128 experts top-4 (10240 routed rows), the router's many-token path, verify-
    shaped attention on a sliding-window layer.  (Whole pages, not the ring the benchmark keeps: the seeded stand-in
    for prefill fills ring pages differently from the oracle's cache; the ring is checked bit for bit against whole
    pages in test_gpu_engine.py.)"""
    from eidola_b200.capi import make_config
    n = 512
    ctx = np.random.default_rng(5).integers(16, 1500, size=n)
    cfg = make_config(n_layers=1, hidden=2880, n_q_heads=64, n_kv_heads=8, window=128, n_experts=128, top_k=4, inter=2880,
                      vocab=8192, num_pages=int(((ctx + 5 + 16) // 16 + 1).sum()) + 8, max_seqs=n, max_pages_per_seq=100,
                      max_tokens=5 * n, max_q_len=5, seed=5, debug=1)
    _forced_step(cfg, ctx, [5] * n, seed=1, what="120b-shaped verify layer")
