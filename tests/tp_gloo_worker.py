"""One CPU rank of the tensor-/expert-parallel decomposition check (started by tests/test_tp_gloo.py).

    RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT in the environment;  argv: <out_file>

Each rank computes its shard of every decoder layer with the CPU oracle's operators -- its query heads, its KV heads
(with the 128-row K/V weight bands a rank shares with its neighbour when it holds a single KV head), its slice of
the O projection's K dimension, its experts -- and the per-layer exchanges go through torch.distributed (gloo) in
the engine's form: the two fp32 sums are reduce-scatters over token slices (gloo has no reduce-scatter: an
all-reduce of which a rank keeps its slice; with TP_GLOO_C1=gather the first one is replaced by the gathered-operand
form: the ranks' quantised attention bands are all-gathered and every rank multiplies full-K rows by the whole W_o), the slice's owner adds the residual, normalises and routes its tokens,
and the rows and the routing are all-gathered.  The LM head is split over the vocabulary and the ranks' argmax
candidates are merged.  Every layer starts from the unsharded oracle's input (teacher forcing); rank 0 saves the
outputs.
"""
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import binding as orc  # noqa: E402
from oracle import sched as osched  # noqa: E402
from tests.helpers import bf16_to_f32  # noqa: E402
from tests.tp_worker import CONTEXTS, tp_config  # noqa: E402


def sid(layer, kind, expert=0):
    return ((layer + 1) << 20) | (kind << 12) | expert


def main():
    import torch
    import torch.distributed as dist
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = tp_config("tp_small")
    H, I, E, K, D = cfg.hidden, cfg.inter, cfg.n_experts, cfg.top_k, cfg.head_dim
    HQ, HKV = cfg.n_q_heads, cfg.n_kv_heads
    hq_l, hkv_l, e_l = HQ // world, HKV // world, E // world
    hqd_l, hqd_g, hkd_g = hq_l * D, HQ * D, HKV * D
    kv_band = -(-hkv_l * D // 128) * 128
    kv_row0 = (rank * hkv_l * D) // 128 * 128
    koff = (rank * hkv_l * D) % 128
    k_col0, v_col0 = hqd_l + koff, hqd_l + kv_band + koff
    nqkv_l = hqd_l + 2 * kv_band

    # the unsharded oracle gives every layer's input and the expected output
    model = orc.Model(cfg)
    model.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, cfg.page_size, cfg.max_seqs, cfg.max_pages_per_seq, cfg.seed)
    ctx = CONTEXTS["tp_small"]
    slots = [sch.admit(L) for L in ctx]
    q_lens = [1, 3, 5, 2]
    for s, q in zip(slots, q_lens):
        sch.extend(s, sch.len[s] + q)
    T = sum(q_lens)
    p = sch.pack(slots, q_lens)
    p.update(slots=slots, n_tokens=T)
    bt = np.array(sch.tables, np.int32)
    toks = np.random.default_rng(1).integers(0, cfg.vocab, size=T).astype(np.int32)
    ref = model.step(p, toks, bt, want_debug=True)

    chunk = -(-T // world)                                   # token slice of this rank: equal chunks, the last may be short
    t0, t1 = min(T, rank * chunk), min(T, (rank + 1) * chunk)

    def gather_rows(mine, width, dtype):
        """All-gather of equal chunks of rows; returns the first T rows."""
        buf = np.zeros((chunk, width), dtype)
        buf[: t1 - t0] = mine
        wire = buf.view(np.uint8)                                  # gloo has no 16-bit integer types: send the bytes
        parts = [torch.zeros(wire.shape, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(wire))
        return np.concatenate([q.numpy() for q in parts]).view(dtype)[:T]

    cos, sin = orc.rope_table(cfg.max_pages_per_seq * cfg.page_size, D, float(cfg.rope_theta))
    ones = np.ones(H, np.float32)
    outs = []
    for l in range(cfg.n_layers):
        x = ref["hidden"][l].copy()
        # ---- attention half, this rank's heads
        wg, sg = orc.synth_weight_fp8(cfg.seed, sid(l, 1), hqd_g + 2 * hkd_g, H, 0, hqd_g + 2 * hkd_g, cfg.init_std)
        bands = [(rank * hqd_l, hqd_l), (hqd_g + kv_row0, kv_band), (hqd_g + hkd_g + kv_row0, kv_band)]
        wl = np.concatenate([wg[a:a + n] for a, n in bands])
        sl = np.concatenate([sg[a // 128:(a + n) // 128] for a, n in bands])
        assert wl.shape[0] == nqkv_l
        h = orc.rmsnorm(x, ones, cfg.rms_eps)
        h8, sh = orc.quant_act_block128(h)
        qkv = orc.gemm_fp8_block(h8, sh, wl, sl)
        orc.rope_inplace(qkv, 0, hq_l, D, p["positions"], cos, sin)
        orc.rope_inplace(qkv, k_col0, hkv_l, D, p["positions"], cos, sin)
        cache_g = orc.synth_normal_bf16(cfg.seed, 20000 + l, 0, cfg.num_pages * 2 * HKV * 16 * D).reshape(cfg.num_pages, 2, HKV, 16, D)
        cache_l = np.ascontiguousarray(cache_g[:, :, rank * hkv_l:(rank + 1) * hkv_l])
        orc.kv_append(cache_l, hkv_l, D, 16, qkv[:, k_col0:], qkv[:, v_col0:], nqkv_l, bt, p["tok_slot"], p["positions"])
        sinks = orc.synth_normal_f32(cfg.seed, sid(l, 6), 0, HQ)[rank * hq_l:(rank + 1) * hq_l]
        window = cfg.window if l % 2 == 0 else 0
        att = orc.attn_paged_sink(np.ascontiguousarray(qkv[:, :hqd_l]), cache_l, bt, slots, p["q_off"], p["ctx_lens"], sinks,
                                  window, hq_l, hkv_l)
        a8, sa = orc.quant_act_block128(att)
        wo, so = orc.synth_weight_fp8(cfg.seed, sid(l, 2), H, hqd_g, 0, H, cfg.init_std)
        c0 = rank * hqd_l
        o_part = bf16_to_f32(orc.gemm_fp8_block(a8, sa, np.ascontiguousarray(wo[:, c0:c0 + hqd_l]),
                                                np.ascontiguousarray(so[:, c0 // 128:(c0 + hqd_l) // 128]))).copy()
        xs = np.ascontiguousarray(x[t0:t1])
        if os.environ.get("TP_GLOO_C1") == "gather":
            # C1 on the gathered operand: the ranks' code bands and scale columns side by side ARE the quantised whole
            # attention output (scale blocks are 128 columns wide), and full-K rows of the projection are the unsharded ones
            def all_cols(mine):
                parts = [torch.zeros(mine.view(np.uint8).shape, dtype=torch.uint8) for _ in range(world)]
                dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(mine).view(np.uint8)))
                return np.concatenate([q.numpy().view(mine.dtype) for q in parts], axis=1)
            a8_g, sa_g = all_cols(a8), all_cols(sa)
            a8_w, sa_w = orc.quant_act_block128(all_cols(att))   # what one GPU quantises: the whole attention output
            assert np.array_equal(a8_g, a8_w) and np.array_equal(sa_g, sa_w), "gathered bands differ from the whole operand"
            o_full = orc.gemm_fp8_block(a8_g, sa_g, wo, so)     # hence the unsharded projection, bit for bit
            orc.residual_add(xs, np.ascontiguousarray(o_full[t0:t1]))
        else:
            t_o = torch.from_numpy(o_part)
            dist.all_reduce(t_o)                               # C1: sum over the ranks' heads; this rank keeps rows [t0, t1)
            orc.residual_add(xs, orc.bf16_encode(t_o.numpy()[t0:t1]))
        # ---- expert half: the slice's owner normalises and routes, rows and routing are gathered
        h2s = orc.rmsnorm(xs, ones, cfg.rms_eps) if t1 > t0 else np.zeros((0, H), np.uint16)
        wr = orc.synth_normal_bf16(cfg.seed, sid(l, 3), 0, E * H, cfg.init_std).reshape(E, H)
        if t1 > t0:
            idx_s, wts_s, _ = orc.router_topk(h2s, wr, K)
        else:
            idx_s, wts_s = np.zeros((0, K), np.int32), np.zeros((0, K), np.float32)
        h2 = gather_rows(h2s, H, np.uint16)
        idx = gather_rows(idx_s, K, np.int32)
        wts = gather_rows(wts_s, K, np.float32)
        x = gather_rows(xs, H, np.uint16)                      # (the engine keeps the residual sliced; the check wants it whole)
        idx_all, wts_all, _ = orc.router_topk(h2, wr, K)       # routing a slice gives the bits of routing everything
        assert np.array_equal(idx, idx_all) and np.array_equal(wts, wts_all)
        mine = (idx >= rank * e_l) & (idx < (rank + 1) * e_l)
        w1 = [orc.synth_weight_fp8(cfg.seed, sid(l, 4, e), 2 * I, H, 0, 2 * I, cfg.init_std) for e in range(E)]
        w2 = [orc.synth_weight_fp8(cfg.seed, sid(l, 5, e), H, I, 0, H, cfg.init_std) for e in range(E)]
        part = bf16_to_f32(orc.moe_forward(h2, idx, np.where(mine, wts, 0).astype(np.float32),
                                           np.stack([a for a, _ in w1]), np.stack([b for _, b in w1]),
                                           np.stack([a for a, _ in w2]), np.stack([b for _, b in w2]))).copy()
        t_m = torch.from_numpy(part)
        dist.all_reduce(t_m)                                   # C2: sum over the ranks' experts; rows [t0, t1) kept
        xs = np.ascontiguousarray(x[t0:t1])
        orc.residual_add(xs, orc.bf16_encode(t_m.numpy()[t0:t1]))
        x = gather_rows(xs, H, np.uint16)
        outs.append(x)
        gathered = [None] * world
        dist.all_gather_object(gathered, idx.tobytes())
        assert all(g == gathered[0] for g in gathered), "routing differs between ranks"
    # ---- vocabulary-parallel LM head on the oracle's final hidden state: candidates {top1, top2, id} per rank, merged
    blocks = (cfg.vocab + 127) // 128
    per = -(-blocks // world)
    v0, v1 = min(cfg.vocab, rank * per * 128), min(cfg.vocab, (rank + 1) * per * 128)
    hf = orc.rmsnorm(ref["hidden"][cfg.n_layers], ones, cfg.rms_eps)
    hf8, shf = orc.quant_act_block128(hf)
    wlm, slm = orc.synth_weight_fp8(cfg.seed, sid(-1, 2), cfg.vocab, H, v0, v1 - v0, cfg.init_std)
    lg = bf16_to_f32(orc.gemm_fp8_block(hf8, shf, wlm, slm))
    order = np.argsort(-lg, axis=1, kind="stable")           # stable: ties keep the lower id first
    cand = np.stack([lg[np.arange(T), order[:, 0]], lg[np.arange(T), order[:, 1]], (order[:, 0] + v0).astype(np.float32)], axis=1)
    parts = [torch.zeros(T, 3) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(cand.astype(np.float32)))
    best = np.full(T, -np.inf, np.float32)
    second = np.full(T, -np.inf, np.float32)
    tok = np.zeros(T, np.int64)
    for q in parts:                                           # ranks in ascending vocabulary order: strict > keeps the lower id
        c = q.numpy()
        win = c[:, 0] > best
        second = np.where(win, np.maximum(best, c[:, 1]), np.maximum(second, c[:, 0]))
        tok = np.where(win, c[:, 2].astype(np.int64), tok)
        best = np.where(win, c[:, 0], best)
    full = bf16_to_f32(ref["logits"])
    want_tok = full.argmax(axis=1)
    top2 = np.sort(full, axis=1)[:, -2:]
    assert np.array_equal(tok, want_tok), "merged vocabulary-parallel argmax differs from the whole-row argmax"
    assert np.array_equal(best - second, top2[:, 1] - top2[:, 0])
    if rank == 0:
        np.savez(sys.argv[1], got=np.stack(outs), want=ref["hidden"][1:], route=ref["route_idx"])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
