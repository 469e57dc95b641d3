"""Shared builders for the parity tests: seeded ragged batches, paged caches, tolerances."""
from __future__ import annotations

import numpy as np

from oracle import binding as orc

HEAD_DIM = 64
PAGE = 16

# Stream ids of the seeded test tensors (any fixed distinct numbers).
S_KV, S_Q, S_SINK = 101, 102, 103

# Tolerance for bf16 outputs of floating-point kernels whose summation order differs from the oracle's:
# |gpu - oracle| <= ATOL + RTOL * |oracle|, RTOL = one bf16 ulp (2^-7 relative spacing is 2^-8..2^-7).
ATOL = 1e-2
RTOL = 2.0 ** -7
# Attention outputs are convex combinations of N(0,1) values: O(1) for a handful of keys, O(0.05) over thousands.
# The measured worst difference from the oracle is 1e-3..2e-3 (the softmax weights reach the second MMA as a bf16
# head plus remainder), so the absolute part of the bound is 3e-3: a dropped page or a wrong mask on a long
# sequence (errors of 1e-2 and more) fails it.
ATTN_ATOL = 3e-3


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even; infinities and NaN keep their class."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = np.isnan(np.asarray(x, np.float32))
    return np.where(nan, np.uint16(0x7FC0), r).astype(np.uint16)


def assert_close_bf16(got_u16, want_u16, atol=ATOL, rtol=RTOL, what=""):
    g, w = bf16_to_f32(got_u16).astype(np.float64), bf16_to_f32(want_u16).astype(np.float64)
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    err = np.abs(g - w)
    bound = atol + rtol * np.abs(w)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{what}: {bad.sum()} of {bad.size} outside atol={atol} rtol={rtol}; worst at {i}: "
                             f"got {g[i]:.6f} want {w[i]:.6f}")
    return float(err.max())


def lognormal_lengths(n, median, sigma, lo, hi, seed):
    """Context lengths of the paged-attention benchmark: clip(round(exp(N(ln median, sigma))), lo, hi)."""
    rng = np.random.default_rng(seed)
    L = np.rint(np.exp(rng.normal(np.log(median), sigma, size=n)))
    return np.clip(L, lo, hi).astype(np.int32)


def make_cache_host(num_pages, n_kv, seed):
    """[num_pages][2][n_kv][16][64] bf16 ~ N(0,1), element i = eb_normal(seed, S_KV, i)."""
    n = num_pages * 2 * n_kv * PAGE * HEAD_DIM
    return orc.synth_normal_bf16(seed, S_KV, 0, n).reshape(num_pages, 2, n_kv, PAGE, HEAD_DIM)


def make_q_host(T, n_q, seed):
    return orc.synth_normal_bf16(seed, S_Q, 0, T * n_q * HEAD_DIM).reshape(T, n_q * HEAD_DIM)


def make_sinks_host(n_q, seed):
    return orc.synth_normal_f32(seed, S_SINK, 0, n_q)


# ---------------------------------------------------------------------------- GPU-side case builder

class AttnCase:
    """A ragged paged-attention problem resident on the device, built through the C ABI only."""

    def __init__(self, ctx_lens, q_lens, n_kv, seed, sm_count, extra_pages=3, device_synth=False, group=8):
        import eidola_b200 as eb
        from eidola_b200 import capi
        from eidola_b200.capi import DeviceBuffer
        self.eb = eb
        self.n_kv, self.n_q, self.seed, self.sm_count = n_kv, n_kv * group, seed, sm_count
        ctx_lens = np.asarray(ctx_lens, np.int32)
        q_lens = np.asarray(q_lens, np.int32)
        n = len(ctx_lens)
        pages = int(((ctx_lens.astype(np.int64) + PAGE - 1) // PAGE).sum())
        self.num_pages = pages + extra_pages
        self.max_pages = int((ctx_lens.max() + PAGE - 1) // PAGE)
        self.sched = eb.Scheduler(self.num_pages, PAGE, n, self.max_pages, seed)
        slots = [self.sched.admit(int(L)) for L in ctx_lens]
        self.packed = self.sched.pack(slots, q_lens)
        self.bt = self.sched.block_tables()
        T = self.packed["n_tokens"]
        self.T = T
        n_cache = self.num_pages * 2 * n_kv * PAGE * HEAD_DIM
        self.d_cache = DeviceBuffer(n_cache * 2)
        self.d_q = DeviceBuffer(T * self.n_q * HEAD_DIM * 2)
        self.d_sinks = DeviceBuffer(self.n_q * 4)
        if device_synth:
            self.cache = self.q = None
            capi.call("eb_synth_normal_bf16", capi.c_vp(self.d_cache.ptr), capi.c_i64(n_cache), capi.c_u64(seed),
                      capi.c_u64(S_KV), capi.c_u64(0), capi.c_f32(1.0), capi.c_vp(None))
            capi.call("eb_synth_normal_bf16", capi.c_vp(self.d_q.ptr), capi.c_i64(T * self.n_q * HEAD_DIM),
                      capi.c_u64(seed), capi.c_u64(S_Q), capi.c_u64(0), capi.c_f32(1.0), capi.c_vp(None))
            capi.call("eb_synth_normal_f32", capi.c_vp(self.d_sinks.ptr), capi.c_i64(self.n_q), capi.c_u64(seed),
                      capi.c_u64(S_SINK), capi.c_u64(0), capi.c_f32(1.0), capi.c_vp(None))
            capi.call("eb_device_sync")
            self.sinks = make_sinks_host(self.n_q, seed)
        else:
            self.cache = make_cache_host(self.num_pages, n_kv, seed)
            self.q = make_q_host(T, self.n_q, seed)
            self.sinks = make_sinks_host(self.n_q, seed)
            capi.call("eb_copy_h2d", capi.c_vp(self.d_cache.ptr), capi.ptr(self.cache), capi.c_sz(self.cache.nbytes), None)
            capi.call("eb_copy_h2d", capi.c_vp(self.d_q.ptr), capi.ptr(self.q), capi.c_sz(self.q.nbytes), None)
            capi.call("eb_copy_h2d", capi.c_vp(self.d_sinks.ptr), capi.ptr(self.sinks), capi.c_sz(self.sinks.nbytes), None)
            capi.call("eb_device_sync")
        self.d_bt = DeviceBuffer.from_array(self.bt)
        self.d_out = DeviceBuffer(T * self.n_q * HEAD_DIM * 2)

    def host_cache(self):
        if self.cache is None:
            self.cache = self.d_cache.to_array(np.uint16, (self.num_pages, 2, self.n_kv, PAGE, HEAD_DIM))
        return self.cache

    def host_q(self):
        if self.q is None:
            self.q = self.d_q.to_array(np.uint16, (self.T, self.n_q * HEAD_DIM))
        return self.q

    def launch(self, window, chunk_pages=0):
        from eidola_b200.host import AttnLaunch
        eb = self.eb
        plan = eb.attn_plan(self.packed["ctx_lens"], self.packed["q_lens"], PAGE, window, self.sm_count, chunk_pages,
                            8 // self.n_kv)
        return AttnLaunch(d_q=self.d_q.ptr, q_stride=self.n_q * HEAD_DIM, d_out=self.d_out.ptr,
                          out_stride=self.n_q * HEAD_DIM, d_cache=self.d_cache.ptr, num_pages=self.num_pages,
                          d_block_tables=self.d_bt.ptr, bt_stride=self.bt.shape[1], packed=self.packed, plan=plan,
                          d_sinks=self.d_sinks.ptr, window=window, n_q=self.n_q, n_kv=self.n_kv), plan

    def run(self, window, chunk_pages=0):
        from eidola_b200 import capi
        self.d_out.zero()
        launch, plan = self.launch(window, chunk_pages)
        launch.run()
        capi.call("eb_device_sync")
        return self.d_out.to_array(np.uint16, (self.T, self.n_q * HEAD_DIM)), plan

    def oracle(self, window, seqs=None):
        """Oracle output; `seqs` restricts to a subset of sequences (rows of the others are zero)."""
        p = self.packed
        if seqs is None:
            return orc.attn_paged_sink(self.host_q(), self.host_cache(), self.bt, p["slots"], p["q_off"], p["ctx_lens"],
                                       self.sinks, window, self.n_q, self.n_kv)
        out = np.zeros((self.T, self.n_q * HEAD_DIM), np.uint16)
        for i in seqs:
            a, b = int(p["q_off"][i]), int(p["q_off"][i + 1])
            out[a:b] = orc.attn_paged_sink(self.host_q()[a:b], self.host_cache(), self.bt, p["slots"][i:i + 1],
                                           np.array([0, b - a], np.int32), p["ctx_lens"][i:i + 1], self.sinks, window,
                                           self.n_q, self.n_kv)
        return out
