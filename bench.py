#!/usr/bin/env python
"""Benchmark of the decode hot path on B200 through the C ABI of libeidola_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line.  Workloads:
  attn   paged sink-attention decode of one layer: 256 ragged sequences, 64 query / 8 KV heads, head_dim 64,
         bf16 KV cache in 16-token pages, context lengths lognormal(median 2048, sigma 1) clipped to [16, 32768],
         per-head sink logits ~ N(0,1), Q/K/V ~ N(0,1), seed 1 (+rank).  One step = one decode token per sequence.
Inputs are synthetic (seeded, generated on the device); the KV working set (~1.5 GB) is an order of magnitude
larger than the L2, so no flush is needed between iterations.

--impl reference times the CPU oracle (the reference project has no implementation of this path) on a bounded
sample of the same workload with all host threads.
"""
from __future__ import annotations

import argparse
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
# dram bytes read+written per launch / algorithmic bytes, from the ncu capture summarised in
# profiles/attn_kernel_paged_sink_decode.md (64-sequence case, scaled by the bytes processed)
NCU_TRAFFIC_RATIO_ATTN = 1.028
S_KV, S_Q, S_SINK = 101, 102, 103


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
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------ attention workload

class AttnWorkload:
    name = "paged sink-attention decode, one layer: 256 ragged seqs, 64q/8kv heads, d64, bf16 KV pages of 16, " \
           "ctx lognormal(median 2048, sigma 1) in [16,32768], full attention"

    def __init__(self, rank: int, n_seqs=256, window=0):
        import eidola_b200 as eb
        from eidola_b200 import capi
        from eidola_b200.capi import DeviceBuffer, c_f32, c_i64, c_u64, c_vp
        from eidola_b200.host import AttnLaunch
        self.eb, self.capi = eb, capi
        self.info = eb.device_info(rank_device(rank))
        seed = 1 + rank
        self.n_kv, self.n_q, self.window = 8, 64, window
        self.ctx = lognormal_lengths(n_seqs, 2048, 1.0, 16, 32768, seed)
        n = n_seqs
        self.q_lens = np.ones(n, np.int32)
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
        self.plan = eb.attn_plan(self.ctx, self.q_lens, PAGE, window, self.info["sm_count"], 0, 1)
        self.launch = AttnLaunch(d_q=self.d_q.ptr, q_stride=self.n_q * HEAD_DIM, d_out=self.d_out.ptr,
                                 out_stride=self.n_q * HEAD_DIM, d_cache=self.d_cache.ptr, num_pages=self.num_pages,
                                 d_block_tables=self.d_bt.ptr, bt_stride=self.bt.shape[1], packed=self.packed,
                                 plan=self.plan, d_sinks=self.d_sinks.ptr, window=window, n_q=self.n_q, n_kv=self.n_kv)
        # pinned host staging for the end-to-end leg
        self.h_q, self.h_out = c_vp(), c_vp()
        capi.call("eb_host_alloc", __import__("ctypes").byref(self.h_q), capi.c_sz(self.q_bytes))
        capi.call("eb_host_alloc", __import__("ctypes").byref(self.h_out), capi.c_sz(self.q_bytes))
        capi.call("eb_copy_d2h", self.h_q, c_vp(self.d_q.ptr), capi.c_sz(self.q_bytes), None)
        capi.call("eb_device_sync")
        self.units_per_step = T  # decode tokens
        visible = np.minimum(self.ctx, window) if window else self.ctx
        # algorithmic bytes of one launch: K and V of every visible token for all 8 KV heads (2 KiB per token),
        # Q in and O out (bf16), and one int32 block-table entry per visible page
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

    e2e_h2d = property(lambda self: self.q_bytes)
    e2e_d2h = property(lambda self: self.q_bytes)

    def config(self) -> dict:
        return {"workload": self.name, "n_seqs": len(self.ctx), "sum_context_tokens": int(self.ctx.sum()),
                "attn_items": self.plan["n_items"], "split_parts": self.plan["n_parts"],
                "l2": "working set %.2f GB >> L2 %.0f MB, no flush" % (self.alg_bytes / 1e9, self.info["l2_bytes"] / 1e6)}

    def cpu_sample(self, n_sample=24):
        """Oracle on every (256/n_sample)-th sequence; returns (tokens, seconds, description)."""
        from oracle import binding as orc
        idx = list(range(0, len(self.ctx), max(1, len(self.ctx) // n_sample)))[:n_sample]
        cache = self.d_cache.to_array(np.uint16, (self.num_pages, 2, self.n_kv, PAGE, HEAD_DIM))
        q = self.d_q.to_array(np.uint16, (self.T, self.n_q * HEAD_DIM))
        sinks = self.d_sinks.to_array(np.float32, self.n_q)
        p = self.packed
        sel = np.array(idx, np.int32)
        q_off = np.arange(len(sel) + 1, dtype=np.int32)
        t0 = time.perf_counter()
        out = orc.attn_paged_sink(q[sel], cache, self.bt, p["slots"][sel], q_off, p["ctx_lens"][sel], sinks,
                                  self.window, self.n_q, self.n_kv)
        dt = time.perf_counter() - t0
        return len(sel), dt, out, sel


def rank_device(rank: int) -> int:
    return int(os.environ.get("LOCAL_RANK", rank))


def run_ours(args) -> dict:
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist  # plumbing only: barrier and max-over-ranks of the timings
        torch.cuda.set_device(rank_device(rank))
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank_device(rank)))
    import eidola_b200 as eb
    from eidola_b200 import capi
    capi.call("eb_device_set", capi.c_i32(rank_device(rank)))
    wl = AttnWorkload(rank, n_seqs=args.seqs)
    K, W = args.steps, args.warmup

    def barrier():
        capi.call("eb_device_sync")
        if dist is not None:
            dist.barrier()
            capi.call("eb_device_sync")

    # ---- device-resident throughput (value) + per-launch durations (roofline)
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
        t.e1_recorded = capi.call("eb_event_record", t.e1, None)
    total_ms = total.stop()
    per_launch = []
    for t in timers:
        ms = capi.c_f32(0)
        capi.call("eb_event_elapsed_ms", t.e0, t.e1, __import__("ctypes").byref(ms))
        per_launch.append(ms.value)
    barrier()
    # ---- end to end through the C ABI with host buffers
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

    if dist is not None:
        import torch
        t = torch.tensor([total_ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, e2e_ms = t.tolist()
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return {}

    peak, peak_kind = measured_peaks()
    avg_launch_ms = sum(per_launch) / len(per_launch)
    achieved = wl.alg_bytes / (avg_launch_ms * 1e-3) / 1e9
    units = wl.units_per_step * world
    out = {
        "metric": "decode tokens/s @256 ragged seqs",
        "value": units * K / (total_ms * 1e-3),
        "unit": "tokens/s",
        "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": total_ms / K,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": dict(wl.config(), parallelism=("replicas x%d (independent sequence sets)" % world) if world > 1 else "single GPU"),
        "e2e": {"value": units * K / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": wl.e2e_h2d,
                "d2h_bytes_per_step": wl.e2e_d2h},
        "gpu_launches": wl.launches_per_step * K,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": peak_kind, "traffic": NCU_TRAFFIC_RATIO_ATTN * wl.alg_bytes, "kernel": "attn_kernel (+ attn_merge_kernel)",
                     "alg_bytes_per_launch": wl.alg_bytes, "avg_launch_ms": avg_launch_ms,
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks,
        "device_status": status,
    }
    # ---- CPU baseline on this box's host cores (rank 0, N=1 only)
    if world == 1 and not args.no_cpu:
        n, dt, cpu_out, sel = wl.cpu_sample()
        gpu_out = wl.d_out.to_array(np.uint16, (wl.T, wl.n_q * HEAD_DIM))[sel]
        g = (gpu_out.astype(np.uint32) << 16).view(np.float32)
        c = (cpu_out.astype(np.uint32) << 16).view(np.float32)
        out["cpu_baseline"] = {"value": n / dt, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port",
                               "sample": "%d of 256 sequences (every %dth), one decode token each, %.1f s" % (n, 256 // n, dt),
                               "max_abs_diff_vs_gpu": float(np.abs(g - c).max())}
    if dist is not None:
        dist.destroy_process_group()
    return out


def run_reference(args) -> dict:
    """The reference arm: the CPU oracle (no reference implementation of this path exists) on all host threads."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return {}
    from oracle import binding as orc
    n_sample = 16
    ctx = lognormal_lengths(256, 2048, 1.0, 16, 32768, 1)
    sel = np.arange(0, 256, 256 // n_sample)[:n_sample]
    ctx_s = ctx[sel]
    pages = ((ctx_s.astype(np.int64) + PAGE - 1) // PAGE)
    num_pages = int(pages.sum())
    bt = np.full((n_sample, int(pages.max())), -1, np.int32)
    perm = np.random.default_rng(1).permutation(num_pages)
    k = 0
    for i, n in enumerate(pages):
        bt[i, :n] = perm[k:k + n]
        k += int(n)
    cache = orc.synth_normal_bf16(1, S_KV, 0, num_pages * 2 * 8 * PAGE * HEAD_DIM).reshape(num_pages, 2, 8, PAGE, HEAD_DIM)
    q = orc.synth_normal_bf16(1, S_Q, 0, n_sample * 64 * HEAD_DIM).reshape(n_sample, 64 * HEAD_DIM)
    sinks = orc.synth_normal_f32(1, S_SINK, 0, 64)
    q_off = np.arange(n_sample + 1, dtype=np.int32)
    slots = np.arange(n_sample, dtype=np.int32)
    K, W = args.steps, args.warmup
    for _ in range(min(W, 1)):
        orc.attn_paged_sink(q, cache, bt, slots, q_off, ctx_s, sinks, 0, 64, 8)
    K = max(1, min(K, 5))
    t0 = time.perf_counter()
    for _ in range(K):
        orc.attn_paged_sink(q, cache, bt, slots, q_off, ctx_s, sinks, 0, 64, 8)
    dt = time.perf_counter() - t0
    v = n_sample * K / dt
    sample = "CPU oracle (port; the reference has no implementation of this path), %d of 256 sequences per step" % n_sample
    return {
        "impl": "reference", "metric": "decode tokens/s @256 ragged seqs", "value": v, "unit": "tokens/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", 1)), "steps": K, "warmup": min(W, 1), "ms_per_step": dt / K * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": AttnWorkload.name, "sample": sample},
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--seqs", type=int, default=256, help="sequences in the batch (smaller values are for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    out = run_reference(args) if args.impl == "reference" else run_ours(args)
    if out:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
