"""Generate tests/golden/tiny_decode.npz from the CPU oracle (run from the repository root):

    python tests/golden/make_golden.py

The reference project holds no golden vectors for this path (it contains no decoder), so these pin the oracle
itself: a later change to the oracle that alters a block table, a routing decision, a logit or a greedy token of
the tiny decode configuration fails tests/test_decoder_oracle.py.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import binding as orc  # noqa: E402
from oracle import sched as osched  # noqa: E402
from tests.decoder_cases import TINY_CONTEXTS, tiny_config  # noqa: E402


def run_tiny(steps=64):
    cfg = tiny_config()
    model = orc.Model(cfg)
    model.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    slots = [sch.admit(L) for L in TINY_CONTEXTS]
    tokens = np.array([11, 222, 3333, 4000], np.int32)  # the first new token of each sequence
    out = {"tables0": None, "tokens": [], "margins": []}
    first = None
    for step in range(steps):
        for s in slots:
            sch.extend(s, sch.len[s] + 1)
        p = sch.pack(slots, [1] * len(slots))
        p.update(slots=slots, n_tokens=len(slots))
        bt = np.array(sch.tables, np.int32)
        if step == 0:
            out["tables0"] = bt.copy()
            out["positions0"] = np.array(p["positions"], np.int32)
            out["ctx0"] = np.array(p["ctx_lens"], np.int32)
        r = model.step(p, tokens, bt, want_logits=(step == 0), want_debug=(step == 0))
        if step == 0:
            first = r
        out["tokens"].append(r["next"].copy())
        out["margins"].append(r["margin"].copy())
        tokens = r["next"].copy()
    out["tables_end"] = np.array(sch.tables, np.int32)
    return cfg, first, out


if __name__ == "__main__":
    cfg, first, out = run_tiny()
    np.savez_compressed(
        ROOT / "tests" / "golden" / "tiny_decode.npz",
        tables0=out["tables0"], tables_end=out["tables_end"], positions0=out["positions0"], ctx0=out["ctx0"],
        route_idx0=first["route_idx"], logits0=first["logits"], hidden0=first["hidden"],
        tokens=np.stack(out["tokens"]), margins=np.stack(out["margins"]))
    print("wrote tiny_decode.npz; first tokens", out["tokens"][0], "min margin", float(np.min(out["margins"])))
