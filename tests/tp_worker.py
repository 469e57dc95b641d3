"""One rank of the tensor-/expert-parallel parity run (started by tests/test_gpu_tp.py, one process per GPU).

    python tests/tp_worker.py <rank> <world> <id_file> <out_file> <config: tp_small|tp_mid>

Every rank drives an engine created with eb_engine_create_tp over an NCCL communicator whose 128-byte id rank 0
writes to <id_file>.  Each rank saves what it computed; the parent compares ranks with each other, with a
single-GPU engine and with the CPU oracle.
"""
import os
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))


def tp_config(name):
    from eidola_b200.capi import make_config
    if name == "tp_small":  # 16 query / 2 KV heads over 2 ranks: one KV head per rank, K/V bands shared with the neighbour
        return make_config(n_layers=2, hidden=512, n_q_heads=16, n_kv_heads=2, window=128, n_experts=8, top_k=4,
                           inter=512, vocab=2048, num_pages=96, max_seqs=4, max_pages_per_seq=24, max_tokens=20,
                           max_q_len=5, seed=7, debug=1)
    return make_config(n_layers=2, hidden=2880, n_q_heads=64, n_kv_heads=8, window=128, n_experts=8, top_k=4,
                       inter=2880, vocab=8192, num_pages=600, max_seqs=12, max_pages_per_seq=80, max_tokens=60,
                       max_q_len=5, seed=3, debug=1)


def vocab_slice(vocab, rank, world):
    """Vocabulary rows of the LM head that live on `rank`: whole 128-row scale blocks, dealt in order."""
    blocks = (vocab + 127) // 128
    per = (blocks + world - 1) // world
    return min(vocab, rank * per * 128), min(vocab, (rank + 1) * per * 128)


CONTEXTS = {"tp_small": [7, 33, 128, 250], "tp_mid": [5, 40, 130, 300, 17, 1000, 64, 2, 511, 128, 33, 250]}


def run_steps(eng, name, force=None, rank=0, world=1):
    """Two steps (decode, then ragged verify).  `force`: per step the oracle's hidden states to impose.  Under tensor
    parallelism a rank holds the logits of its vocabulary slice only: the other columns are saved as zeros."""
    cfg = eng.cfg
    ctx = CONTEXTS[name]
    slots = [eng.admit(L) for L in ctx]
    rng = np.random.default_rng(0)
    out = []
    for step, q_lens in enumerate(([1] * len(ctx), [(i % 5) + 1 for i in range(len(ctx))])):
        T = sum(q_lens)
        toks = rng.integers(0, cfg.vocab, size=T).astype(np.int32)
        if force is not None:
            for l in range(cfg.n_layers + 1):
                eng.force_hidden(l, force[step][l])
        nxt, mg = eng.step(slots, q_lens, toks)
        logits = eng.read_logits()
        if world > 1:
            v0, v1 = vocab_slice(cfg.vocab, rank, world)
            logits[:, :v0] = 0
            logits[:, v1:] = 0
        out.append({"next": nxt, "margin": mg, "logits": logits,
                    "route_idx": np.stack([eng.read_routing(l) for l in range(cfg.n_layers)]),
                    "hidden": np.stack([eng.read_hidden(l) for l in range(-1, cfg.n_layers)]),
                    "tokens": toks, "q_lens": np.array(q_lens, np.int32)})
    return slots, out


PREFILL_PROMPTS = [7, 133, 12, 50, 300]


def run_prefill(eng, rank=0, world=1):
    """Whole prompts through eb_engine_prefill (steps of max_tokens rows), then one decode step on seeded tokens."""
    cfg = eng.cfg
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, cfg.vocab, size=n).astype(np.int32) for n in PREFILL_PROMPTS]
    slots = [eng.admit(0) for _ in prompts]
    first, margin, steps, _ = eng.prefill(slots, prompts)
    nxt, mg = eng.step(slots, [1] * len(slots), rng.integers(0, cfg.vocab, size=len(slots)).astype(np.int32))  # the same everywhere
    logits = eng.read_logits()
    if world > 1:
        v0, v1 = vocab_slice(cfg.vocab, rank, world)
        logits[:, :v0] = 0
        logits[:, v1:] = 0
    return {"first": first, "first_margin": margin, "steps": np.array([steps], np.int32), "next": nxt, "margin": mg, "logits": logits}


def main():
    rank, world, id_file, out_file, name = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
    force_file = sys.argv[6] if len(sys.argv) > 6 else None
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(rank))
    if rank == 0:
        uid = eb.Comm.unique_id()
        tmp = id_file + ".tmp"
        Path(tmp).write_bytes(uid)
        os.replace(tmp, id_file)
    else:
        t0 = time.time()
        while not os.path.exists(id_file):
            if time.time() - t0 > 120:
                raise TimeoutError("no NCCL id from rank 0")
            time.sleep(0.05)
        uid = Path(id_file).read_bytes()
    comm = eb.Comm(uid, rank, world)
    if name.endswith("+prefill"):
        cfg = tp_config(name[:-len("+prefill")])
        cfg.max_tokens = 256
        eng = eb.Engine(cfg, rank, world, comm)
        flat = run_prefill(eng, rank, world)
        flat["status"] = np.array([eb.status_read()], np.int32)
        np.savez(out_file, **flat)
        eng.close()
        comm.close()
        return
    cfg = tp_config(name)
    eng = eb.Engine(cfg, rank, world, comm)
    eng.kv_fill_synth()
    force = None
    if force_file:
        f = np.load(force_file)
        force = [[f[f"s{s}_l{l}"] for l in range(cfg.n_layers + 1)] for s in range(2)]
    _, out = run_steps(eng, name, force, rank, world)
    flat = {}
    for s, o in enumerate(out):
        for k, v in o.items():
            flat[f"s{s}_{k}"] = v
    flat["status"] = np.array([eb.status_read()], np.int32)
    flat["comm_async_error"] = np.array([comm.async_error()], np.int32)
    np.savez(out_file, **flat)
    eng.close()
    comm.close()


if __name__ == "__main__":
    main()
