#!/usr/bin/env python
"""Benchmark of the decode hot path on B200 through the C ABI of libeidola_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decoder|attn|spec120b|gemm|peak]

Prints ONE JSON line.  With one GPU the default workload also carries the other two parts of the metric as
sub-records (`attn`: the paged sink-attention benchmark; `gemm_sweep`: the FP8 GEMM sweep against the measured FP8
issue-rate ceiling `fp8_peak`; `sampler`: top-p sampling beside argmax on 256 rows of the vocabulary).  Under torchrun with N > 1 ranks the SAME 256 sequences are decoded by ONE engine
spread over the N GPUs -- query/KV heads tensor-parallel, experts expert-parallel, LM head vocabulary-parallel, over
NCCL -- so the figure scales strongly; the line then also carries `spec120b` (the 120b-shaped speculative-verify
step on the same ranks) and `parity` (a two-layer slice of the N-rank engine against the single-GPU engine).

decoder (default): the gpt-oss-20b-shaped random-init FP8 decoder -- 24 layers (even: 128-token sliding window,
    odd: full attention), hidden 2880, 64 query / 8 KV heads, head_dim 64, 32 experts top-4 (intermediate 2880),
    vocabulary 201088 -- decoding 256 concurrent ragged sequences greedily, prompt lengths uniform in [128, 8192]
    (seed 4 + rank).  Prefill is stood in for by filling the KV pages with seeded N(0,1) values.  One step = one
    new token for every sequence, through eb_engine_step: token ids go in from host memory, greedy tokens come
    back to host memory and are fed to the next step.
spec120b: the gpt-oss-120b-shaped decoder (36 layers, 128 experts) with tensor-parallel heads and expert-parallel
    experts over 2, 4 or 8 GPUs (torchrun), verifying k=4 draft tokens per sequence on 512 ragged sequences.
attn: one layer of paged sink-attention on 256 ragged sequences with lognormal(median 2048, sigma 1) context lengths
    clipped to [16, 32768] (seed 1 + rank); the kernel-level benchmark of the attention path.  --sigma, --window 128
    and --qlen 5 (speculative verify) select the variants.
gemm: the FP8 block-scaled GEMM sweep X[M,2880] x W[5120,2880]^T, M in {1, 8, 64, 256, 1024, 4096} (--m picks some):
    GB/s for the small M, TFLOP/s for the large ones.

Inputs are synthetic (seeded, generated on the device).  The per-step working set (weights 20 GB + KV 28 GB for
the decoder, 1.5 GB of KV for attn) is far larger than the L2, so nothing is flushed between iterations.

--impl reference times the CPU oracle on the host cores: the reference project has no implementation of this path
(it delegates inference to a third-party process), so the committed CPU restatement is the CPU arm.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HEAD_DIM, PAGE = 64, 16
S_KV, S_Q, S_SINK = 101, 102, 103
# dram bytes read + written per launch / algorithmic bytes of attn_kernel, from an ncu capture of a 64-sequence case
# (0.36 GB, larger than the L2), scaled by the bytes processed
NCU_TRAFFIC_RATIO_ATTN = 1.028
METRIC = "decode tokens/s @256 ragged seqs"


def lognormal_lengths(n, median, sigma, lo, hi, seed):
    rng = np.random.default_rng(seed)
    L = np.rint(np.exp(rng.normal(np.log(median), sigma, size=n)))
    return np.clip(L, lo, hi).astype(np.int32)


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def rank_device(rank: int) -> int:
    return int(os.environ.get("LOCAL_RANK", rank))


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.rows, self.proc = device, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, pw, reasons = [], [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                pw.append(float(r[2]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------ decoder workload

def decoder_config(make_config, n_layers=24, n_seqs=256, max_ctx=8192, steps=0, n_experts=32, debug=0, seed=4, max_q_len=1,
                   max_tokens=0):
    """eb_config of the 20b-shaped decoder; `make_config` is the binding's (engine arm) or the CPU checker's (CPU arm)."""
    pages_per_seq = (max_ctx + steps + PAGE) // PAGE + 1
    return make_config(n_layers=n_layers, hidden=2880, n_q_heads=64, n_kv_heads=8, window=128, n_experts=n_experts,
                       top_k=4, inter=2880, vocab=201088, num_pages=1, max_seqs=n_seqs,
                       max_pages_per_seq=pages_per_seq, max_tokens=max(max_tokens, n_seqs * max_q_len), max_q_len=max_q_len, seed=seed,
                       debug=debug)


PREFILL_STEP_ROWS = 4096  # token rows of a prefill step (--prefill real): whole prompts, several sequences per step

DECODER_NAME = ("gpt-oss-20b-shaped random-init FP8 decoder: 24 layers (even 128-window, odd full), hidden 2880, 64q/8kv "
                "heads d64, 32 experts top-4 inter 2880, vocab 201088; 256 ragged seqs, prompts U[128,8192], greedy decode")


class DecoderWorkload:
    """The 256-sequence greedy decode.  world > 1: ONE engine over `world` ranks (heads tensor-parallel, experts
    expert-parallel); every rank is given the same sequences and tokens and returns the same tokens."""
    name = DECODER_NAME

    def __init__(self, total_steps: int, n_seqs=256, n_layers=24, profile=False, rank=0, world=1, comm=None, debug=0,
                 max_ctx=8192, min_ctx=128, prefill="synthetic"):
        import eidola_b200 as eb
        from eidola_b200.capi import make_config
        self.eb, self.rank, self.world = eb, rank, world
        seed = 4
        rng = np.random.default_rng(seed)
        self.ctx0 = rng.integers(min_ctx, max_ctx + 1, size=n_seqs).astype(np.int32)
        cfg = decoder_config(make_config, n_layers=n_layers, n_seqs=n_seqs, max_ctx=max_ctx, steps=total_steps,
                             debug=(2 if profile else 0) | debug, seed=seed, max_q_len=6 if prefill == "real" else 1,
                             max_tokens=PREFILL_STEP_ROWS if prefill == "real" else 0)
        cfg.num_pages = int(((self.ctx0.astype(np.int64) + total_steps + PAGE) // PAGE + 1).sum()) + 64
        self.cfg = cfg
        self.eng = eb.Engine(cfg, rank, world, comm)
        self.prefill_stats = None
        if prefill == "real":
            # the engine computes the cache itself: the prompts run through all layers, PREFILL_STEP_ROWS token rows per step
            self.slots = np.array([self.eng.admit(0) for _ in self.ctx0], np.int32)
            prompts = [rng.integers(0, cfg.vocab, size=int(L)).astype(np.int32) for L in self.ctx0]
            t0 = time.perf_counter()
            first, _, steps, ms = self.eng.prefill(self.slots, prompts)
            wall = time.perf_counter() - t0
            n_tok = int(self.ctx0.astype(np.int64).sum())
            self.prefill_stats = {"prompt_tokens": n_tok, "steps": steps, "device_ms": ms, "wall_ms": wall * 1e3,
                                  "prompt_tokens_per_s": n_tok / (ms * 1e-3), "chunk": self.eng.chunk_tokens(),
                                  "rows_per_step": PREFILL_STEP_ROWS,
                                  "prompts": "U[%d,%d] tokens per sequence" % (min_ctx, max_ctx)}
            self.tokens = first.astype(np.int32)
        else:
            self.eng.kv_fill_synth()
            self.slots = np.array([self.eng.admit(int(L)) for L in self.ctx0], np.int32)
            self.tokens = rng.integers(0, cfg.vocab, size=n_seqs).astype(np.int32)
        self.q_lens = np.ones(n_seqs, np.int32)
        self.steps_done = 0
        self.units_per_step = n_seqs
        self.mem = self.eng.memory()

    def step(self):
        """One greedy decode step through the host-buffer API: the returned tokens feed the next step."""
        nxt, mg = self.eng.step(self.slots, self.q_lens, self.tokens)
        self.tokens = nxt
        self.margins = mg
        self.steps_done += 1
        return nxt

    def ctx_now(self) -> np.ndarray:
        return self.ctx0.astype(np.int64) + self.steps_done

    def attn_alg_bytes_full_layer(self) -> int:
        """Algorithmic bytes of one full-attention layer launch on this rank at the current lengths: K and V of every
        context token for this rank's KV heads (2 KiB per token over all 8), Q in and O out, one block-table entry per
        page."""
        ctx = self.ctx_now() + 1
        n = len(ctx)
        return (int(ctx.sum()) * 2048 + 2 * n * 64 * HEAD_DIM * 2) // self.world + 4 * int(((ctx + PAGE - 1) // PAGE).sum())

    def step_alg_bytes(self) -> dict:
        """Bytes one step must move through this rank's HBM: every weight once (all 32 experts are hit at 1024 routed
        slots), K and V of every visible context token."""
        c, G = self.cfg, self.world
        ctx = self.ctx_now() + 1
        per_layer_dense = (64 + 16) * 64 * 2880 + 2880 * 4096          # QKV + O, e4m3
        per_layer_experts = c.n_experts * 3 * 2880 * 2880
        weights = (c.n_layers * (per_layer_dense + per_layer_experts) + c.vocab * 2880) // G + c.n_layers * c.n_experts * 2880 * 2
        kv_full = (c.n_layers // 2) * int(ctx.sum()) * 2048 // G
        kv_win = (c.n_layers - c.n_layers // 2) * int(np.minimum(ctx, 128 + PAGE).sum()) * 2048 // G
        return {"weights": weights, "kv_full": kv_full, "kv_window": kv_win, "total": weights + kv_full + kv_win}

    def config(self) -> dict:
        return {"workload": self.name, "n_seqs": int(len(self.ctx0)), "n_layers": int(self.cfg.n_layers),
                "mean_context": float(self.ctx_now().mean()),
                "device_bytes_per_rank": self.mem,
                "prefill": ("real: eb_engine_prefill ran every prompt through all layers, %d token rows per step" % PREFILL_STEP_ROWS if self.prefill_stats
                            else "KV pages filled with seeded N(0,1) values (stand-in for prefill)"),
                "l2": "per-step working set ~%.0f GB per GPU >> L2, no flush" % (self.step_alg_bytes()["total"] / 1e9)}


def host_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def decoder_cpu_sample(n_seqs=64, seed=4, reps=3):
    """CPU oracle on a bounded sample of the decoder workload: the first two layers (one windowed, one full) and the
    LM head, n_seqs of the 256 sequences, whole decode steps.  One untimed warm-up repetition, then `reps` timed
    ones; the figure is the MEDIAN step time, min and max are kept beside it.  Uses nothing of the CUDA library.
    Returns a dict(value tokens/s extrapolated to 24 layers, sample description, spread)."""
    from oracle import binding as orc
    from oracle import sched as osched
    threads = orc.set_threads_pinned(host_threads())  # every CPU this process may run on, whatever OMP_NUM_THREADS says
    n_steps = 2 * (reps + 1)
    cfg = decoder_config(orc.make_config, n_layers=2, n_seqs=n_seqs, steps=n_steps + 2, seed=seed)
    rng = np.random.default_rng(seed)
    ctx = rng.integers(128, 8193, size=256).astype(np.int32)[:: 256 // n_seqs][:n_seqs]
    cfg.num_pages = int(((ctx.astype(np.int64) + n_steps + 2 + PAGE) // PAGE + 1).sum()) + 8
    model = orc.Model(cfg)
    model.kv_fill_synth()
    sch = osched.Sched(cfg.num_pages, PAGE, n_seqs, cfg.max_pages_per_seq, seed)
    slots = [sch.admit(int(L)) for L in ctx]
    toks = rng.integers(0, cfg.vocab, size=n_seqs).astype(np.int32)

    def timed_step(n_layers_run):
        for s in slots:
            sch.extend(s, sch.len[s] + 1)
        p = sch.pack(slots, [1] * n_seqs)
        p.update(slots=slots, n_tokens=n_seqs)
        bt = np.array(sch.tables, np.int32)
        t0 = time.perf_counter()
        model.step(p, toks, bt, n_layers_run=n_layers_run, want_logits=False)
        return time.perf_counter() - t0

    per_step, cpu_s = [], 0.0
    for r in range(reps + 1):
        t_full = timed_step(2)   # 2 layers + head
        t_head = timed_step(0)   # embedding + head only
        if r == 0:
            continue             # warm-up: page in the weights, start the thread pool
        cpu_s += t_full + t_head
        per_step.append((t_full - t_head) * 12 + t_head)  # 24 layers = 12 (windowed, full) pairs
    t_med = statistics.median(per_step)
    desc = ("CPU oracle on %d pinned threads, %d of 256 sequences: 2 of 24 layers (one windowed, one full) + LM head timed "
            "per decode step (1 warm-up + %d timed repetitions, %.1f s of CPU work), layer time x12 + head -> median "
            "%.2f s per step (min %.2f, max %.2f)" % (threads, n_seqs, reps, cpu_s, t_med, min(per_step), max(per_step)))
    return {"value": n_seqs / t_med, "sample": desc, "threads": threads,
            "spread": {"min": n_seqs / max(per_step), "max": n_seqs / min(per_step)}}


# ------------------------------------------------------------------------------------------ 120b-shaped TP x EP verify

class Spec120bWorkload:
    name = ("gpt-oss-120b-shaped random-init FP8 decoder: 36 layers, hidden 2880, 64q/8kv heads d64, 128 experts top-4 "
            "inter 2880, vocab 201088; heads tensor-parallel, experts expert-parallel; speculative verification of k=4 "
            "draft tokens (+1 bonus position, q_len 5) per sequence, acceptance Bernoulli(0.7) per draft, 512 ragged "
            "seqs, context lognormal(median 4096, sigma 1) in [16,131072]")

    def __init__(self, rank, world, dist, total_steps, n_seqs=512, n_layers=36, n_experts=128, profile=False, comm=None):
        import eidola_b200 as eb
        from eidola_b200.capi import make_config
        self.eb, self.rank, self.world = eb, rank, world
        seed = 5
        self.ctx0 = lognormal_lengths(n_seqs, 4096, 1.0, 16, 131072, seed)
        grow = 5 * total_steps + 16
        max_pages = int((int(self.ctx0.max()) + grow) // PAGE + 2)
        cfg = make_config(n_layers=n_layers, hidden=2880, n_q_heads=64, n_kv_heads=8, window=128, n_experts=n_experts,
                          top_k=4, inter=2880, vocab=201088, num_pages=1, max_seqs=n_seqs, max_pages_per_seq=max_pages,
                          max_tokens=5 * n_seqs, max_q_len=5, seed=seed, debug=2 if profile else 0, window_ring=1)
        cfg.num_pages = int(((self.ctx0.astype(np.int64) + grow) // PAGE + 1).sum()) + 64
        self.cfg = cfg
        self.comm = comm
        self.eng = eb.Engine(cfg, rank, world, self.comm)
        self.eng.kv_fill_synth()
        self.slots = np.array([self.eng.admit(int(L)) for L in self.ctx0], np.int32)
        self.lens = self.ctx0.astype(np.int64).copy()
        self.q_lens = np.full(n_seqs, 5, np.int32)
        self.rng = np.random.default_rng(seed)       # same stream on every rank: identical drafts and acceptances
        self.last = self.rng.integers(0, cfg.vocab, size=n_seqs).astype(np.int32)
        self.mem = self.eng.memory()
        self.accepted_total = 0

    def step(self):
        """Verify 4 random draft tokens per sequence; accept a Bernoulli(0.7) prefix, keep the bonus token."""
        n = len(self.slots)
        drafts = self.rng.integers(0, self.cfg.vocab, size=(n, 4)).astype(np.int32)
        toks = np.concatenate([self.last[:, None], drafts], axis=1).reshape(-1)
        nxt, _ = self.eng.step(self.slots, self.q_lens, toks)
        ok = self.rng.random((n, 4)) < 0.7
        a = np.where(ok.all(axis=1), 4, np.argmin(ok, axis=1)).astype(np.int64)   # accepted drafts per sequence
        self.last = nxt.reshape(n, 5)[np.arange(n), a].astype(np.int32)           # the model's token after the last accepted
        self.lens = self.lens + a + 1
        self.eng.truncate_many(self.slots, self.lens)
        adv = int((a + 1).sum())
        self.accepted_total += adv
        return adv

    def step_alg_bytes(self) -> dict:
        c, G = self.cfg, self.world
        ctx = self.lens + 5
        dense = (64 + 16) * 64 * 2880 + 2880 * 4096
        experts = c.n_experts * 3 * 2880 * 2880
        weights = c.n_layers * (dense + experts) // G + c.n_layers * c.n_experts * 2880 * 2 // G + c.vocab * 2880 // G
        kv_full = (c.n_layers // 2) * int(ctx.sum()) * 2048 // G
        kv_win = (c.n_layers - c.n_layers // 2) * int(np.minimum(ctx, 128 + 5 + PAGE).sum()) * 2048 // G
        return {"weights": weights, "kv_full": kv_full, "kv_window": kv_win, "total": weights + kv_full + kv_win,
                "reduce_scatter_bytes_per_layer": 2 * 5 * len(ctx) * 2880 * 2,
                "allgather_bytes_per_layer": 5 * len(ctx) * (2880 * 2 + 32) + 5 * len(ctx) * 2880 + (5 * len(ctx) // 128) * 23 * 4}

    def config(self) -> dict:
        return {"workload": self.name, "n_seqs": int(len(self.ctx0)), "n_layers": int(self.cfg.n_layers),
                "mean_context": float(self.lens.mean()), "device_bytes_per_rank": self.mem,
                "prefill": "KV pages filled with seeded N(0,1) values (stand-in for prefill)",
                "parallelism": "tp%d (heads) x ep%d (experts); rows dealt to ranks in slices of whole 128-row blocks: partial "
                               "[2560, 2880] products go to the slice owners as planes (summed in rank order), residual + norm + "
                               "routing on the slice; experts by dispatch / return of rows from 4 ranks on, by partial sums at 2; "
                               "e4m3 codes + block scales gathered for the next layer; vocabulary-parallel LM head with a gather "
                               "of argmax candidates; transport: %s" % (self.world, self.world,
                               "NCCL" if os.environ.get("EIDOLA_B200_TP_NCCL") == "1" else "peer-memory stores over NVLink")}


# ------------------------------------------------------------------------------------------ attention workload

class AttnWorkload:
    def __init__(self, rank: int, n_seqs=256, window=0, sigma=1.0, q_len=1):
        import eidola_b200 as eb
        from eidola_b200 import capi
        from eidola_b200.capi import DeviceBuffer, c_f32, c_i64, c_u64, c_vp
        from eidola_b200.host import AttnLaunch
        self.eb, self.capi = eb, capi
        self.info = eb.device_info(rank_device(rank))
        seed = 1 + rank
        self.n_kv, self.n_q, self.window = 8, 64, window
        self.name = ("paged sink-attention %s, one layer: %d ragged seqs, 64q/8kv heads, d64, bf16 KV pages of 16, "
                     "ctx lognormal(median 2048, sigma %g) in [16,32768], %s"
                     % ("decode" if q_len == 1 else "verify (q_len %d)" % q_len, n_seqs, sigma,
                        "%d-token sliding window" % window if window else "full attention"))
        self.ctx = lognormal_lengths(n_seqs, 2048, sigma, 16, 32768, seed)
        n = n_seqs
        self.q_lens = np.full(n, q_len, np.int32)
        pages = int(((self.ctx.astype(np.int64) + PAGE - 1) // PAGE).sum())
        self.num_pages = pages + 8
        max_pages = int((self.ctx.max() + PAGE - 1) // PAGE)
        self.sched = eb.Scheduler(self.num_pages, PAGE, n, max_pages, seed)
        slots = [self.sched.admit(int(L)) for L in self.ctx]
        self.packed = self.sched.pack(slots, self.q_lens)
        self.bt = self.sched.block_tables()
        T = self.T = self.packed["n_tokens"]
        n_cache = self.num_pages * 2 * self.n_kv * PAGE * HEAD_DIM
        self.d_cache = DeviceBuffer(n_cache * 2)
        self.q_bytes = T * self.n_q * HEAD_DIM * 2
        self.d_q, self.d_out, self.d_sinks = DeviceBuffer(self.q_bytes), DeviceBuffer(self.q_bytes), DeviceBuffer(self.n_q * 4)
        capi.call("eb_synth_normal_bf16", c_vp(self.d_cache.ptr), c_i64(n_cache), c_u64(seed), c_u64(S_KV), c_u64(0), c_f32(1.0), None)
        capi.call("eb_synth_normal_bf16", c_vp(self.d_q.ptr), c_i64(T * self.n_q * HEAD_DIM), c_u64(seed), c_u64(S_Q), c_u64(0), c_f32(1.0), None)
        capi.call("eb_synth_normal_f32", c_vp(self.d_sinks.ptr), c_i64(self.n_q), c_u64(seed), c_u64(S_SINK), c_u64(0), c_f32(1.0), None)
        self.d_bt = DeviceBuffer.from_array(self.bt)
        self.plan = eb.attn_plan(self.ctx, self.q_lens, PAGE, window,
                                 eb.attn_plan_sm_count(self.info["sm_count"], q_len, self.n_q, self.n_kv, window), 0, 1)
        self.launch = AttnLaunch(d_q=self.d_q.ptr, q_stride=self.n_q * HEAD_DIM, d_out=self.d_out.ptr,
                                 out_stride=self.n_q * HEAD_DIM, d_cache=self.d_cache.ptr, num_pages=self.num_pages,
                                 d_block_tables=self.d_bt.ptr, bt_stride=self.bt.shape[1], packed=self.packed,
                                 plan=self.plan, d_sinks=self.d_sinks.ptr, window=window, n_q=self.n_q, n_kv=self.n_kv)
        self.h_q, self.h_out = c_vp(), c_vp()  # pinned host staging for the end-to-end leg
        capi.call("eb_host_alloc", C.byref(self.h_q), capi.c_sz(self.q_bytes))
        capi.call("eb_host_alloc", C.byref(self.h_out), capi.c_sz(self.q_bytes))
        capi.call("eb_copy_d2h", self.h_q, c_vp(self.d_q.ptr), capi.c_sz(self.q_bytes), None)
        capi.call("eb_device_sync")
        self.units_per_step = T
        visible = np.minimum(self.ctx, window + q_len - 1) if window else self.ctx
        self.alg_bytes = int(visible.astype(np.int64).sum()) * 2 * self.n_kv * HEAD_DIM * 2 + 2 * self.q_bytes \
            + 4 * int(((visible.astype(np.int64) + PAGE - 1) // PAGE).sum())
        self.launches_per_step = 2 if self.plan["n_parts"] > n else 1

    def step(self, stream=None):
        self.launch.run(stream)

    def step_e2e(self, stream=None):
        capi, c_vp, c_sz = self.capi, self.capi.c_vp, self.capi.c_sz
        capi.call("eb_copy_h2d", c_vp(self.d_q.ptr), self.h_q, c_sz(self.q_bytes), c_vp(stream))
        self.launch.run(stream)
        capi.call("eb_copy_d2h", self.h_out, c_vp(self.d_out.ptr), c_sz(self.q_bytes), c_vp(stream))
        capi.call("eb_stream_sync", c_vp(stream))

    def config(self) -> dict:
        return {"workload": self.name, "n_seqs": len(self.ctx), "sum_context_tokens": int(self.ctx.sum()),
                "attn_items": self.plan["n_items"], "split_parts": self.plan["n_parts"],
                "l2": "working set %.2f GB >> L2 %.0f MB, no flush" % (self.alg_bytes / 1e9, self.info["l2_bytes"] / 1e6)}

    def cpu_sample(self, reps=20):
        from oracle import binding as orc
        cache = self.d_cache.to_array(np.uint16, (self.num_pages, 2, self.n_kv, PAGE, HEAD_DIM))
        q = self.d_q.to_array(np.uint16, (self.T, self.n_q * HEAD_DIM))
        sinks = self.d_sinks.to_array(np.float32, self.n_q)
        p = self.packed
        t0 = time.perf_counter()
        for _ in range(reps):
            out = orc.attn_paged_sink(q, cache, self.bt, p["slots"], p["q_off"], p["ctx_lens"], sinks, self.window,
                                      self.n_q, self.n_kv)
        dt = time.perf_counter() - t0
        return self.T * reps / dt, dt, out


# ------------------------------------------------------------------------------------------ drivers

def setup_dist():
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    dist = None
    if world > 1:
        import torch.distributed as dist  # plumbing only (gloo, host tensors): barrier, max over ranks, NCCL id hand-off
        dist.init_process_group("gloo")
    return rank, world, dist


def reduce_max(dist, values):
    if dist is None:
        return values
    import torch
    t = torch.tensor(values, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def make_comm(eb, rank, world, dist):
    """The NCCL communicator of the tensor-/expert-parallel engines: rank 0 makes the id, gloo carries it."""
    if world == 1:
        return None
    # NCCL's own record of the communicator ("... rank r nranks N ...") goes to the log, so that a reader of the run
    # can check that N ranks really joined
    if os.environ.get("NCCL_DEBUG", "").upper() not in ("INFO", "TRACE"):
        os.environ["NCCL_DEBUG"] = "INFO"
        os.environ.setdefault("NCCL_DEBUG_SUBSYS", "INIT")
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # stdout carries the one JSON line and nothing else
    uid = [eb.Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(uid, src=0)
    return eb.Comm(uid[0], rank, world)


def serving_metrics(stamps, units_per_step):
    """The stream-timing figures the reference server keeps per response (crates/eidola-server/src/handlers.rs:551-687):
    time to the first token, the largest gap between consecutive tokens, tokens per second over the window from the
    first to the last token.  `stamps`: host time after each step returned, the first entry is the start."""
    gaps = np.diff(np.asarray(stamps))
    window = stamps[-1] - stamps[1] if len(stamps) > 2 else 0.0
    return {"ttft_ms": float(gaps[0] * 1e3), "max_inter_token_gap_ms": float(gaps[1:].max() * 1e3) if len(gaps) > 1 else None,
            "tokens_per_s_first_to_last": float(units_per_step * (len(gaps) - 1) / window) if window > 0 else None,
            "per_sequence_tokens_per_s": float((len(gaps) - 1) / window) if window > 0 else None,
            "note": "decode only: the first token's time excludes prefill, which the KV fill stands in for"}


def tp_parity_block(eb, rank, world, dist, comm):
    """A two-layer slice of the N-rank engine against the single-GPU engine on the same step (rank 0 holds both).
    The single-GPU engine is what the parity tests compare with the CPU oracle layer by layer."""
    n, layers = 64, 2
    kw = dict(total_steps=4, n_seqs=n, n_layers=layers, debug=1, max_ctx=2048)
    tp = DecoderWorkload(rank=rank, world=world, comm=comm, **kw)
    nxt = tp.step().copy()
    logits_tp = tp.eng.read_logits()
    hid_tp = tp.eng.read_hidden(layers - 1)
    route_tp = [tp.eng.read_routing(l) for l in range(layers)]
    mg_tp = tp.margins.copy()
    tp.eng.close()
    if rank != 0:
        return None
    one = DecoderWorkload(**kw)
    ref = one.step().copy()
    logits_1 = one.eng.read_logits()
    hid_1 = one.eng.read_hidden(layers - 1)
    route_1 = [one.eng.read_routing(l) for l in range(layers)]
    mg_1 = one.margins.copy()
    one.eng.close()
    blocks = (tp.cfg.vocab + 127) // 128
    per = (blocks + world - 1) // world
    v1 = min(tp.cfg.vocab, per * 128)  # rank 0 holds the logits of its vocabulary band only
    f = lambda a: (a.astype(np.uint32) << 16).view(np.float32).astype(np.float64)  # noqa: E731
    dl = np.abs(f(logits_tp[:, :v1]) - f(logits_1[:, :v1]))
    dh = f(hid_tp) - f(hid_1)
    clear = mg_1 > 0.2
    same_route = np.ones(n, bool)
    for l in range(layers):
        same_route &= ~(route_tp[l] != route_1[l]).any(axis=1)
    return {"what": "first decode step of a 2-layer slice, %d sequences: tp%d x ep%d engine vs the single-GPU engine" % (n, world, world),
            "greedy_tokens_equal": int((nxt == ref).sum()), "of": n,
            "tokens_equal_where_margin_above_0.2": "%d/%d" % (int((nxt[clear] == ref[clear]).sum()), int(clear.sum())),
            "max_margin_of_a_differing_token": float(mg_1[nxt != ref].max()) if (nxt != ref).any() else 0.0,
            "routing_rows_differing_per_layer": [int((route_tp[l] != route_1[l]).any(axis=1).sum()) for l in range(layers)],
            "max_abs_logit_diff_rank0_band": float(dl.max()),
            "max_abs_logit_diff_rows_with_equal_routing": float(dl[same_route].max()) if same_route.any() else None,
            "rms_logit_diff": float(np.sqrt((dl * dl).mean())), "mean_signed_logit_diff": float((f(logits_tp[:, :v1]) - f(logits_1[:, :v1])).mean()),
            "hidden_rel_l2": float(np.linalg.norm(dh) / np.linalg.norm(f(hid_1))),
            "margin_max_abs_diff": float(np.abs(mg_tp - mg_1).max())}


def run_decoder(args) -> dict:
    rank, world, dist = setup_dist()
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(rank_device(rank)))
    K, W = args.steps, args.warmup
    n_prof = 3
    comm = make_comm(eb, rank, world, dist)
    kw = {}
    if args.prefill == "real":  # a stated subset of the prompt lengths: one eighth of the range, so the run stays in seconds
        kw = dict(prefill="real", min_ctx=16, max_ctx=1024)
    wl = DecoderWorkload(total_steps=K + W + n_prof + 8, n_seqs=args.seqs, n_layers=args.layers, rank=rank, world=world, comm=comm, **kw)
    stream = wl.eng.stream()

    def barrier():
        capi.call("eb_device_sync")
        if dist is not None:
            dist.barrier()
            capi.call("eb_device_sync")

    sampler = ClockSampler(rank_device(rank))
    if rank == 0:
        sampler.start()
    for _ in range(W):
        wl.step()
    barrier()
    timer = eb.Timer(stream)
    dev_ms = 0.0
    launches = 0
    ctx_mid = None
    h2d = d2h = 0
    barrier()
    stamps = [time.perf_counter()]
    timer.start()
    for i in range(K):
        wl.step()
        stamps.append(time.perf_counter())
        ms, nl = wl.eng.last_step_stats()
        dev_ms += ms
        launches += nl
        if i == K // 2:
            ctx_mid = wl.step_alg_bytes()
            h2d, d2h = wl.eng.last_step_copies()
    e2e_ms = timer.stop()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    status = eb.status_read()
    dev_ms, e2e_ms, status = reduce_max(dist, [dev_ms, e2e_ms, float(status)])
    # ---- a few extra steps with CUDA events around each call: the breakdown and the dominant kernel's roofline
    wl.eng.profile(True)
    for _ in range(2):
        wl.step()
    acc, alg, step_ms_prof = {}, 0.0, 0.0
    for _ in range(n_prof):
        alg_bytes = wl.attn_alg_bytes_full_layer()
        wl.step()
        for k, v in wl.eng.last_step_breakdown().items():
            acc[k] = acc.get(k, 0.0) + v / n_prof
        alg += alg_bytes / n_prof
        step_ms_prof = wl.eng.last_step_stats()[0]
    wl.eng.profile(False)
    n_layers, mem_cfg = wl.cfg.n_layers, wl.config()
    wl.eng.close()
    barrier()

    units = wl.units_per_step          # one batch of sequences, whatever the number of GPUs it is spread over
    peak, peak_kind = measured_peaks()
    out = {}
    if rank == 0:
        transport = "NCCL reduce-scatter / all-gather" if os.environ.get("EIDOLA_B200_TP_NCCL") == "1" else \
            "peer-memory stores over NVLink with flag waits (whole-batch planes for steps of <= 512 rows: two exchanges per layer)"
        parallelism = ("tp %d x ep %d: one engine over %d GPUs (query/KV heads and the O projection tensor-parallel, experts "
                       "expert-parallel, LM head vocabulary-parallel); exchanges on the two shard boundaries of every layer by %s"
                       % (world, world, world, transport)) if world > 1 else "single GPU"
        out = {
            "metric": METRIC,
            "value": units * K / (dev_ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": dev_ms / K,
            "higher_is_better": True, "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
            "dtype": "fp8 e4m3 x e4m3 -> fp32 (GEMMs), bf16 (attention, activations)", "data": "synthetic",
            "config": dict(mem_cfg, parallelism=parallelism,
                           value_is="sum of per-step device time (CUDA events around the step's copies and kernels), max over ranks",
                           e2e_is="CUDA events on the engine stream around K calls of eb_engine_step with host token buffers"),
            "e2e": {"value": units * K / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "bytes_are": "what eb_engine_step staged and copied in the middle timed step (eb_engine_last_step_copies)"},
            "gpu_launches": launches,
            "serving": serving_metrics(stamps, units),
            "prefill": wl.prefill_stats,
            "step_bytes_per_rank": ctx_mid,
            "step_hbm_bound": {"bytes_per_rank": ctx_mid["total"], "floor_ms": ctx_mid["total"] / (peak * 1e6),
                               "frac_of_floor": (ctx_mid["total"] / (peak * 1e6)) / (dev_ms / K), "peak_gbs": peak, "peak_kind": peak_kind},
            "clocks": clocks, "device_status": int(status),
        }
        n_full = n_layers // 2
        per_launch_ms = acc["attn_full"] / max(n_full, 1)
        achieved = alg / (per_launch_ms * 1e-3) / 1e9 if per_launch_ms > 0 else 0.0
        out["roofline"] = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                           "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_RATIO_ATTN * alg,
                           "kernel": "attn_kernel (+ attn_merge_kernel), full-attention layers",
                           "alg_bytes_per_launch": alg, "avg_launch_ms": per_launch_ms, "launches_timed": n_prof * n_full,
                           "frac_of_nominal_8TBs": achieved / 8000.0}
        out["step_breakdown_ms"] = dict(acc, step_total=step_ms_prof, other=step_ms_prof - sum(acc.values()),
                                        note="%d extra steps with CUDA events around each call (adds event overhead)" % n_prof)
    if world > 1:
        par = tp_parity_block(eb, rank, world, dist, comm)
        barrier()
        spec = None
        if not args.no_spec:
            spec = spec120b_measure(eb, capi, rank, world, dist, comm, steps=args.spec_steps, warmup=3, n_seqs=512, n_layers=36)
        if rank == 0:
            out["parity"] = par
            if spec is not None:
                out["spec120b"] = spec
    elif not args.no_sub:
        out["fp8_peak"] = peak_subrecord(eb, capi)
        out["attn"] = attn_subrecord(eb, capi, rank)
        out["gemm_sweep"] = gemm_subrecord(eb, capi, rank, out["fp8_peak"])
        out["sampler"] = sampler_subrecord(eb, capi)
    if world == 1 and not args.no_cpu:
        cpu = decoder_cpu_sample()
        out["cpu_baseline"] = {"value": cpu["value"], "unit": "tokens/s", "cores": cpu["threads"], "kind": "port",
                               "sample": cpu["sample"], "spread": cpu["spread"]}
    if comm is not None:
        comm.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return out


def spec120b_measure(eb, capi, rank, world, dist, comm, steps, warmup, n_seqs, n_layers, own_comm=False):
    """The 120b-shaped tensor-/expert-parallel speculative-verify step: `warmup` + `steps` timed steps, then two extra
    steps with per-call CUDA events for the breakdown.  Returns the record on rank 0, None elsewhere."""
    wl = Spec120bWorkload(rank, world, dist, total_steps=steps + warmup + 6, n_seqs=n_seqs, n_layers=n_layers, comm=comm)

    def barrier():
        capi.call("eb_device_sync")
        if dist is not None:
            dist.barrier()

    for _ in range(warmup):
        wl.step()
    barrier()
    timer = eb.Timer(wl.eng.stream())
    dev_ms, accepted, launches = 0.0, 0, 0
    barrier()
    timer.start()
    for _ in range(steps):
        accepted += wl.step()
        ms, nl = wl.eng.last_step_stats()
        dev_ms += ms
        launches += nl
    e2e_ms = timer.stop()
    h2d, d2h = wl.eng.last_step_copies()
    barrier()
    dev_ms, e2e_ms = reduce_max(dist, [dev_ms, e2e_ms])
    wl.eng.profile(True)
    acc = {}
    wl.step()
    for _ in range(2):
        wl.step()
        for k, v in wl.eng.last_step_breakdown().items():
            acc[k] = acc.get(k, 0.0) + v / 2
    prof_ms = wl.eng.last_step_stats()[0]
    status = eb.status_read()
    bytes_now = wl.step_alg_bytes()
    peak, peak_kind = measured_peaks()
    rec = None
    if rank == 0:
        rec = {"metric": "accepted tokens/s, 120b-shaped TP x EP speculative verify", "value": accepted / (dev_ms * 1e-3),
               "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": dev_ms / steps,
               "scaling": "strong", "config": wl.config(),
               "e2e": {"value": accepted / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms / steps,
                       "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               "accepted_per_seq_per_step": accepted / (steps * len(wl.slots)),
               "verified_rows_per_s": 5 * len(wl.slots) * steps / (dev_ms * 1e-3), "gpu_launches": launches,
               "step_bytes_per_rank": bytes_now,
               "step_hbm_bound_per_rank": {"floor_ms": bytes_now["total"] / (peak * 1e6),
                                           "frac_of_floor": (bytes_now["total"] / (peak * 1e6)) / (dev_ms / steps),
                                           "peak_gbs": peak, "peak_kind": peak_kind},
               "step_breakdown_ms": dict(acc, step_total=prof_ms, other=prof_ms - sum(acc.values()),
                                         note="2 extra steps with CUDA events around each call (adds event overhead)"),
               "device_status": status}
    wl.eng.close()
    return rec


def run_spec120b(args) -> dict:
    rank, world, dist = setup_dist()
    if world < 2 and (args.layers == 24 or args.layers > 8):
        return {"metric": "accepted tokens/s, 120b-shaped TP x EP verify", "unavailable":
                "the 120b-shaped configuration needs at least 2 GPUs (116 GB of weights + KV); launch with torchrun, "
                "or pass --layers <= 8 for a single-GPU profile of its layer shapes"}
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(rank_device(rank)))
    comm = make_comm(eb, rank, world, dist)
    sampler = ClockSampler(rank_device(rank))
    if rank == 0:
        sampler.start()
    rec = spec120b_measure(eb, capi, rank, world, dist, comm, steps=args.steps, warmup=args.warmup,
                           n_seqs=args.seqs if args.seqs != 256 else 512, n_layers=args.layers if args.layers != 24 else 36)
    clocks = sampler.stop() if rank == 0 else None
    out = {}
    if rank == 0:
        out = dict(rec, higher_is_better=True, vs_baseline=None,
                   dtype="fp8 e4m3 x e4m3 -> fp32 (GEMMs), bf16 (attention, activations)", data="synthetic", clocks=clocks)
    if comm is not None:
        comm.close()
    if dist is not None:
        dist.destroy_process_group()
    return out


def run_attn(args) -> dict:
    rank, world, dist = setup_dist()
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(rank_device(rank)))
    wl = AttnWorkload(rank, n_seqs=args.seqs, window=args.window, sigma=args.sigma, q_len=args.qlen)
    K, W = args.steps, args.warmup

    def barrier():
        capi.call("eb_device_sync")
        if dist is not None:
            dist.barrier()
            capi.call("eb_device_sync")

    sampler = ClockSampler(rank_device(rank))
    if rank == 0:
        sampler.start()
    for _ in range(W):
        wl.step()
    barrier()
    timers = [eb.Timer() for _ in range(K)]
    total = eb.Timer()
    barrier()
    total.start()
    for t in timers:
        t.start()
        wl.step()
        capi.call("eb_event_record", t.e1, None)
    total_ms = total.stop()
    per_launch = []
    for t in timers:
        ms = capi.c_f32(0)
        capi.call("eb_event_elapsed_ms", t.e0, t.e1, C.byref(ms))
        per_launch.append(ms.value)
    barrier()
    for _ in range(min(W, 3)):
        wl.step_e2e()
    barrier()
    e2e_t = eb.Timer()
    e2e_t.start()
    for _ in range(K):
        wl.step_e2e()
    e2e_ms = e2e_t.stop()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    status = eb.status_read()
    total_ms, e2e_ms = reduce_max(dist, [total_ms, e2e_ms])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return {}
    peak, peak_kind = measured_peaks()
    avg_launch_ms = sum(per_launch) / len(per_launch)
    achieved = wl.alg_bytes / (avg_launch_ms * 1e-3) / 1e9
    units = wl.units_per_step * world
    out = {
        "metric": METRIC, "value": units * K / (total_ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": total_ms / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(wl.config(), parallelism=("replicas x%d (independent sequence sets)" % world) if world > 1 else "single GPU"),
        "e2e": {"value": units * K / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": wl.q_bytes,
                "d2h_bytes_per_step": wl.q_bytes},
        "gpu_launches": wl.launches_per_step * K,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_RATIO_ATTN * wl.alg_bytes,
                     "kernel": "attn_kernel (+ attn_merge_kernel)", "alg_bytes_per_launch": wl.alg_bytes,
                     "avg_launch_ms": avg_launch_ms, "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks, "device_status": status,
    }
    if world == 1 and not args.no_cpu:
        v, dt, cpu_out = wl.cpu_sample()
        g = (wl.d_out.to_array(np.uint16, (wl.T, wl.n_q * HEAD_DIM)).astype(np.uint32) << 16).view(np.float32)
        c = (cpu_out.astype(np.uint32) << 16).view(np.float32)
        out["cpu_baseline"] = {"value": v, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": "all 256 sequences, 20 repetitions, %.1f s" % dt,
                               "max_abs_diff_vs_gpu": float(np.abs(g - c).max())}
    if dist is not None:
        dist.destroy_process_group()
    return out


# ------------------------------------------------------------------------------------------ GEMM sweep workload

def measured_tensor_peak() -> tuple[float, str]:
    """FP8 dense peak estimate in TFLOP/s when no issue-rate measurement is at hand: twice the measured bf16 cuBLAS
    burst figure (the tensor pipe runs e4m3 at twice the bf16 rate), else twice the fallback bf16 figure."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return 2.0 * float(json.loads(p.read_text())["bf16_tflops"]), "2 x measured bf16"
        except Exception:
            pass
    return 2.0 * 1590.0, "2 x fallback bf16"


def peak_subrecord(eb, capi, blocks=8192, reps=5) -> dict:
    """The FP8 tensor path's measured ceiling on this GPU (eb_fp8_mma_peak: back-to-back tcgen05.mma.kind::f8f6f4 on
    operands resident in shared memory, no loads, no epilogue), with the SM clock sampled while it runs."""
    sampler = ClockSampler(0)
    sampler.start()
    ms, tf = capi.c_f32(0), C.c_double(0)
    vals = []
    for _ in range(4):  # ~20 ms each: long enough for nvidia-smi to see the clock under load
        capi.call("eb_fp8_mma_peak", capi.c_i32(blocks), capi.c_i32(reps), C.byref(ms), C.byref(tf))
        vals.append(float(tf.value))
    clocks = sampler.stop()
    two_bf16, kind = measured_tensor_peak()
    best = max(vals)
    return {"tflops": best, "runs": vals, "kernel_ms": float(ms.value), "blocks_per_sm": blocks,
            "shape": "M128 N256 K32 x4 per block, cta_group::1, one CTA per SM, operands in shared memory",
            "clocks": clocks, "frac_of_nominal_4500": best / 4500.0, "two_x_bf16_tflops": two_bf16, "two_x_bf16_kind": kind}


def attn_subrecord(eb, capi, rank, n_seqs=256, reps=10) -> dict:
    """Paged sink-attention on the 256-sequence lognormal batch (seed 1): full, 128-token window, verify (q_len 5)."""
    import gc
    peak, peak_kind = measured_peaks()
    out = {"peak_gbs": peak, "peak_kind": peak_kind}
    for key, kw in (("decode_full", {}), ("decode_window128", {"window": 128}), ("verify_qlen5", {"q_len": 5})):
        wl = AttnWorkload(rank, n_seqs=n_seqs, **kw)
        for _ in range(3):
            wl.step()
        capi.call("eb_device_sync")
        timers = [eb.Timer() for _ in range(reps)]
        for t in timers:
            t.start()
            wl.step()
            capi.call("eb_event_record", t.e1, None)
        per = []
        for t in timers:
            ms = capi.c_f32(0)
            capi.call("eb_event_elapsed_ms", t.e0, t.e1, C.byref(ms))
            per.append(ms.value)
        avg = sum(per) / len(per)
        gbs = wl.alg_bytes / (avg * 1e-3) / 1e9
        out[key] = {"us": avg * 1e3, "alg_bytes": wl.alg_bytes, "gbs": gbs, "frac_hbm": gbs / peak, "frac_nominal_8TBs": gbs / 8000.0,
                    "launches_per_call": wl.launches_per_step, "sum_context_tokens": int(wl.ctx.sum())}
        del wl, timers
        gc.collect()
    out["note"] = ("CUDA events around each of %d calls (attention kernel + merge); the window variant moves 71 MB and is latency "
                   "bound, its fraction is reported, not claimed as a roofline" % reps)
    return out


def sampler_subrecord(eb, capi) -> dict:
    """eb_sample_top_p beside eb_argmax on 256 rows of the benchmark's vocabulary: the cost of drawing every token of the
    batch at temperature 1, top_p 0.9, on the flattest rows there are (N(0,2) logits: every token weighs something)."""
    from eidola_b200.capi import DeviceBuffer, c_f32, c_i32, c_i64, c_u64, c_vp
    T, V = 256, 201088
    logits = DeviceBuffer(T * V * 2)
    capi.call("eb_synth_normal_bf16", c_vp(logits.ptr), c_i64(T * V), c_u64(1), c_u64(3), c_u64(0), c_f32(2.0), None)
    sc = DeviceBuffer.from_array(np.full(T, 1.4426950408889634, np.float32))
    q = DeviceBuffer.from_array(np.full(T, int(0.9 * 2 ** 24), np.uint32))
    r = DeviceBuffer.from_array((np.arange(T, dtype=np.uint64) * 2654435761 % 2 ** 32).astype(np.uint32))
    tok, mg = DeviceBuffer(T * 4), DeviceBuffer(T * 4)

    def timed(fn, n=20):
        for _ in range(3):
            fn()
        t = eb.Timer()
        capi.call("eb_device_sync")
        t.start()
        for _ in range(n):
            fn()
        return t.stop() / n * 1e3

    am = timed(lambda: capi.call("eb_argmax", c_vp(logits.ptr), c_i32(T), c_i64(V), c_i64(V), c_vp(tok.ptr), c_vp(mg.ptr), None))
    sm = timed(lambda: capi.call("eb_sample_top_p", c_vp(logits.ptr), c_i32(T), c_i64(V), c_i64(V), c_vp(sc.ptr), c_vp(q.ptr),
                                 c_vp(r.ptr), c_vp(tok.ptr), None))
    return {"rows": T, "vocab": V, "argmax_us": am, "sample_top_p_us": sm, "temperature": 1.0, "top_p": 0.9,
            "note": "20 back-to-back launches each; synthetic N(0,2) logits, the sampler's worst case"}


def gemm_subrecord(eb, capi, rank, fp8_peak) -> dict:
    """The FP8 GEMM sweep X[M,2880] x W[5120,2880]^T: per-M time, TFLOP/s against the measured FP8 ceiling (and 2 x bf16,
    and nominal), GB/s against the measured HBM peak."""
    import gc
    wl = GemmSweep(rank)
    hbm_peak, hbm_kind = measured_peaks()
    t2, t2_kind = measured_tensor_peak()
    sweep = {}
    for M in wl.MS:
        ms = wl.time_m(M, reps=20, warm=3)
        tf = wl.flops(M) / (ms * 1e-3) / 1e12
        gbs = wl.alg_bytes(M) / (ms * 1e-3) / 1e9
        sweep[str(M)] = {"us": ms * 1e3, "tflops": tf, "gbs": gbs, "frac_fp8_measured": tf / fp8_peak["tflops"],
                         "frac_2x_bf16": tf / t2, "frac_nominal_4500": tf / 4500.0, "frac_hbm": gbs / hbm_peak}
    del wl
    gc.collect()
    return {"sweep": sweep, "fp8_peak_tflops": fp8_peak["tflops"], "two_x_bf16_tflops": t2, "two_x_bf16_kind": t2_kind,
            "hbm_peak_gbs": hbm_peak, "hbm_peak_kind": hbm_kind,
            "note": "20 launches per M queued behind a fill kernel, 13 rotating copies of W so no launch finds it in L2; "
                    "M <= 256 is bound by HBM (frac_hbm), M >= 1024 by the tensor path (frac_fp8_measured)"}


def run_peak(args) -> dict:
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(0))
    rec = peak_subrecord(eb, capi)
    return {"metric": "FP8 tensor-path ceiling (tcgen05.mma.kind::f8f6f4 issue rate)", "value": rec["tflops"], "unit": "TFLOP/s",
            "n_gpus": 1, "steps": 4, "warmup": 1, "ms_per_step": rec["kernel_ms"], "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8 e4m3 x e4m3 -> fp32", "data": "synthetic", "config": {"workload": rec["shape"]},
            "fp8_peak": rec, "clocks": rec["clocks"], "gpu_launches": 4 * 6}


class GemmSweep:
    """Y = X W^T, X [M,2880] e4m3, W [5120,2880] e4m3, fp32 scales per 128x128 block uniform in [0.5,2), bf16 output.
    Entries are N(0,1) rounded to e4m3.  Each M rotates over enough distinct copies of W and X that consecutive
    launches never find their operands in L2."""
    name = "FP8 block-scaled GEMM sweep: X[M,2880] x W[5120,2880]^T, e4m3 operands, fp32 128x128 block scales, bf16 out"
    N, K = 5120, 2880
    MS = (1, 8, 64, 256, 1024, 4096)

    def __init__(self, rank: int, seed=2, ms=None):
        import eidola_b200 as eb
        from eidola_b200 import capi, host
        if ms:
            self.MS = tuple(ms)
        from eidola_b200.capi import DeviceBuffer, c_f32, c_i64, c_u64, c_vp
        self.eb, self.capi, self.host = eb, capi, host
        self.info = eb.device_info(rank_device(rank))
        N, K = self.N, self.K
        kb = (K + 127) // 128
        self.copies = int(1.5 * self.info["l2_bytes"] // (N * K)) + 1
        self.w, self.sw = [], []
        for c in range(self.copies):
            w8, sw = DeviceBuffer(N * K), DeviceBuffer(((N + 127) // 128) * kb * 4)
            capi.call("eb_synth_normal_e4m3", c_vp(w8.ptr), c_i64(N * K), c_u64(seed), c_u64(100 + c), c_u64(0), c_f32(1.0), None)
            capi.call("eb_synth_uniform_f32", c_vp(sw.ptr), c_i64(((N + 127) // 128) * kb), c_u64(seed), c_u64(200 + c),
                      c_u64(0), c_f32(0.5), c_f32(2.0), None)
            self.w.append(w8)
            self.sw.append(sw)
        Mmax = max(self.MS)
        self.x, self.sx, self.y = [], [], []
        self.x_copies = 4
        for c in range(self.x_copies):
            x8, sx = DeviceBuffer(Mmax * K), DeviceBuffer(((Mmax + 127) // 128) * kb * 4)
            capi.call("eb_synth_normal_e4m3", c_vp(x8.ptr), c_i64(Mmax * K), c_u64(seed), c_u64(300 + c), c_u64(0), c_f32(1.0), None)
            capi.call("eb_synth_uniform_f32", c_vp(sx.ptr), c_i64(((Mmax + 127) // 128) * kb), c_u64(seed), c_u64(400 + c),
                      c_u64(0), c_f32(0.5), c_f32(2.0), None)
            self.x.append(x8)
            self.sx.append(sx)
            self.y.append(DeviceBuffer(Mmax * N * 2))
        self.work = DeviceBuffer(max(host.gemm_workspace(M, N, 1) for M in self.MS))
        self.flush = DeviceBuffer(2 << 30)
        capi.call("eb_device_sync")
        self.i = 0

    def launch(self, M: int, stream=None):
        c, xc = self.i % self.copies, self.i % self.x_copies
        self.i += 1
        self.host.gemm_fp8(self.x[xc].ptr, self.sx[xc].ptr, self.w[c].ptr, self.sw[c].ptr, self.y[xc].ptr, M, self.N,
                           self.K, work=self.work, stream=stream)

    def alg_bytes(self, M: int) -> int:
        N, K = self.N, self.K
        kb = (K + 127) // 128
        return N * K + M * K + M * N * 2 + 4 * kb * (((N + 127) // 128) + ((M + 127) // 128))

    def flops(self, M: int) -> float:
        return 2.0 * M * self.N * self.K

    def time_m(self, M: int, reps: int, warm: int) -> float:
        """Average device milliseconds per launch over `reps` back-to-back launches.  The launches are enqueued while a
        long fill kernel still runs, so that the events bracket kernels that are already queued on the device and the
        host's enqueue rate stays out of the figure."""
        c_vp, c_sz = self.capi.c_vp, self.capi.c_sz
        for _ in range(warm):
            self.launch(M)
        t = self.eb.Timer()
        self.capi.call("eb_device_sync")
        for _ in range(2):
            self.capi.call("eb_l2_flush", c_vp(self.flush.ptr), c_sz(self.flush.nbytes), None)
        t.start()
        for _ in range(reps):
            self.launch(M)
        return t.stop() / reps

    def cpu_sample(self, M=64):
        from oracle import binding as orc
        N, K = self.N, self.K
        kb = (K + 127) // 128
        x8 = self.x[0].to_array(np.uint8, (max(self.MS), K))[:M].copy()
        sx = self.sx[0].to_array(np.float32, ((max(self.MS) + 127) // 128, kb))[: (M + 127) // 128].copy()
        w8 = self.w[0].to_array(np.uint8, (N, K))
        sw = self.sw[0].to_array(np.float32, ((N + 127) // 128, kb))
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            out = orc.gemm_fp8_block(x8, sx, w8, sw)
            reps += 1
        dt = time.perf_counter() - t0
        return self.flops(M) * reps / dt / 1e12, dt, reps, out


def run_gemm(args) -> dict:
    rank, world, dist = setup_dist()
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(rank_device(rank)))
    wl = GemmSweep(rank, ms=args.m)
    K, W = args.steps, args.warmup

    def barrier():
        capi.call("eb_device_sync")
        if dist is not None:
            dist.barrier()
            capi.call("eb_device_sync")

    sampler = ClockSampler(rank_device(rank))
    if rank == 0:
        sampler.start()
    for _ in range(W):
        for M in wl.MS:
            wl.launch(M)
    barrier()
    total = eb.Timer()
    total.start()
    for _ in range(K):  # one step = one pass over the sweep
        for M in wl.MS:
            wl.launch(M)
    total_ms = total.stop()
    barrier()
    per_m = {}
    for M in wl.MS:
        ms = wl.time_m(M, reps=20, warm=3)
        per_m[M] = ms
    barrier()
    # end to end: host X in, host Y out, for the largest M
    Mbig = max(wl.MS)
    xb, yb = Mbig * wl.K, Mbig * wl.N * 2
    h_x, h_y = capi.c_vp(), capi.c_vp()
    capi.call("eb_host_alloc", C.byref(h_x), capi.c_sz(xb))
    capi.call("eb_host_alloc", C.byref(h_y), capi.c_sz(yb))
    capi.call("eb_copy_d2h", h_x, capi.c_vp(wl.x[0].ptr), capi.c_sz(xb), None)
    capi.call("eb_device_sync")

    def e2e_step():
        xc = wl.i % wl.x_copies
        capi.call("eb_copy_h2d", capi.c_vp(wl.x[xc].ptr), h_x, capi.c_sz(xb), None)
        wl.launch(Mbig)
        capi.call("eb_copy_d2h", h_y, capi.c_vp(wl.y[xc].ptr), capi.c_sz(yb), None)
        capi.call("eb_device_sync")

    for _ in range(3):
        e2e_step()
    e2e_t = eb.Timer()
    e2e_t.start()
    for _ in range(K):
        e2e_step()
    e2e_ms = e2e_t.stop()
    clocks = sampler.stop() if rank == 0 else None
    status = eb.status_read()
    total_ms, e2e_ms = reduce_max(dist, [total_ms, e2e_ms])
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return {}
    hbm_peak, hbm_kind = measured_peaks()
    fp8 = peak_subrecord(eb, capi)
    t_peak, t_kind = fp8["tflops"], "measured: back-to-back tcgen05.mma.kind::f8f6f4 on shared-memory operands (eb_fp8_mma_peak)"
    sweep = {}
    for M, ms in per_m.items():
        tf = wl.flops(M) / (ms * 1e-3) / 1e12
        gbs = wl.alg_bytes(M) / (ms * 1e-3) / 1e9
        sweep[str(M)] = {"us": ms * 1e3, "tflops": tf, "gbs": gbs, "frac_tensor": tf / t_peak, "frac_hbm": gbs / hbm_peak}
    flops_step = sum(wl.flops(M) for M in wl.MS)
    big = sweep[str(Mbig)]
    out = {
        "metric": "FP8 GEMM TFLOPS vs peak", "value": world * flops_step * K / (total_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
        "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8 e4m3 x e4m3 -> fp32 accumulate, fp32 block scales, bf16 out",
        "data": "synthetic",
        "config": {"workload": wl.name, "M": list(wl.MS), "step": "one launch per M of the sweep",
                   "l2": "%d weight copies (%.0f MB) rotate so no launch finds W in L2" % (wl.copies, wl.copies * wl.N * wl.K / 1e6),
                   "parallelism": ("replicas x%d" % world) if world > 1 else "single GPU"},
        "e2e": {"value": world * wl.flops(Mbig) * K / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "M": Mbig,
                "h2d_bytes_per_step": xb, "d2h_bytes_per_step": yb},
        "gpu_launches": len(wl.MS) * K,
        "sweep": sweep,
        "roofline": {"bound": "tensor", "achieved": big["tflops"], "peak": t_peak, "unit": "TFLOP/s",
                     "frac": big["tflops"] / t_peak, "peak_kind": t_kind, "traffic": None,
                     "kernel": "gemm_fp8 kernel, M=%d" % Mbig, "alg_flops_per_launch": wl.flops(Mbig),
                     "avg_launch_ms": per_m[Mbig], "frac_of_nominal_4500": big["tflops"] / 4500.0,
                     "frac_of_2x_measured_bf16": big["tflops"] / measured_tensor_peak()[0], "fp8_peak": fp8,
                     "small_m_hbm": {"M": min(wl.MS), "achieved_gbs": sweep[str(min(wl.MS))]["gbs"], "peak_gbs": hbm_peak,
                                     "peak_kind": hbm_kind, "frac": sweep[str(min(wl.MS))]["frac_hbm"]}},
        "clocks": clocks, "device_status": status,
    }
    if world == 1 and not args.no_cpu:
        v, dt, reps, cpu_out = wl.cpu_sample(min(64, max(wl.MS)))
        out["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": "M=%d of the sweep, %d repetitions, %.1f s" % (min(64, max(wl.MS)), reps, dt)}
    if dist is not None:
        dist.destroy_process_group()
    return out


def run_reference(args) -> dict:
    """The reference arm: the CPU oracle on all host threads (the reference project has no implementation of this path,
    so the committed CPU restatement is its CPU arm).  Loads nothing of the CUDA library."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return {}
    K = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    cpu = decoder_cpu_sample(reps=max(3, K))
    dt = time.perf_counter() - t0
    v = cpu["value"]
    sample = cpu["sample"] + "; the reference project has no implementation of this path, so this is the committed CPU port"
    return {
        "impl": "reference", "metric": METRIC, "value": v, "unit": "tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": max(3, K), "warmup": 1, "ms_per_step": 1e3 * 256 / v,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8 weights/activations decoded to fp32",
        "data": "synthetic", "config": {"workload": DECODER_NAME, "sample": sample, "wall_s": dt},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cpu["threads"], "kind": "port", "sample": sample,
                         "spread": cpu["spread"]},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decoder", choices=["decoder", "attn", "spec120b", "gemm", "peak"])
    ap.add_argument("--prefill", default="synthetic", choices=["synthetic", "real"],
                    help="decoder: 'real' computes the KV cache with eb_engine_prefill on prompts of U[16,1024] tokens (one eighth of "
                         "the benchmark's range) instead of filling the pages with seeded values")
    ap.add_argument("--no-sub", action="store_true", help="decoder, 1 GPU: skip the attn / gemm_sweep / fp8_peak sub-records")
    ap.add_argument("--no-spec", action="store_true", help="decoder, N > 1 GPUs: skip the 120b-shaped verify sub-record")
    ap.add_argument("--spec-steps", type=int, default=6, help="decoder, N > 1 GPUs: timed steps of the 120b-shaped verify sub-record")
    ap.add_argument("--profile", action="store_true", help="spec120b: time attention/GEMM calls with CUDA events in every step")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--window", type=int, default=0, help="attn: sliding window in tokens (0 = full attention)")
    ap.add_argument("--sigma", type=float, default=1.0, help="attn: sigma of the lognormal context lengths")
    ap.add_argument("--qlen", type=int, default=1, help="attn: query positions per sequence (5 = verify of 4 drafts)")
    ap.add_argument("--m", type=int, nargs="*", default=None, help="gemm: token counts to run instead of the whole sweep")
    ap.add_argument("--seqs", type=int, default=256, help="sequences in the batch (smaller values are for profiler captures)")
    ap.add_argument("--layers", type=int, default=24, help="decoder layers (smaller values are for profiler captures)")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        out = run_reference(args)
    elif args.workload == "attn":
        out = run_attn(args)
    elif args.workload == "spec120b":
        out = run_spec120b(args)
    elif args.workload == "gemm":
        out = run_gemm(args)
    elif args.workload == "peak":
        out = run_peak(args)
    else:
        out = run_decoder(args)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
