"""GPU parity: seeded generators, KV append and paged sink attention through the C ABI against the CPU oracle."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.helpers import (ATTN_ATOL, HEAD_DIM, PAGE, AttnCase, assert_close_bf16, bf16_to_f32, lognormal_lengths)

pytestmark = pytest.mark.gpu


def test_device_generators_are_bit_exact(gpu):
    from eidola_b200 import capi
    from eidola_b200.capi import DeviceBuffer, c_f32, c_i64, c_u64, c_vp
    n = 1 << 16
    b = DeviceBuffer(n * 4)
    capi.call("eb_synth_normal_f32", c_vp(b.ptr), c_i64(n), c_u64(9), c_u64(4), c_u64(12345), c_f32(0.02), None)
    assert np.array_equal(b.to_array(np.float32, n), orc.synth_normal_f32(9, 4, 12345, n, 0.02))
    capi.call("eb_synth_normal_bf16", c_vp(b.ptr), c_i64(n), c_u64(9), c_u64(5), c_u64(0), c_f32(1.0), None)
    assert np.array_equal(b.to_array(np.uint16, n), orc.synth_normal_bf16(9, 5, 0, n, 1.0))
    capi.call("eb_synth_normal_e4m3", c_vp(b.ptr), c_i64(n), c_u64(9), c_u64(6), c_u64(0), c_f32(100.0), None)
    assert np.array_equal(b.to_array(np.uint8, n), orc.synth_normal_e4m3(9, 6, 0, n, 100.0))
    capi.call("eb_synth_uniform_f32", c_vp(b.ptr), c_i64(n), c_u64(9), c_u64(7), c_u64(0), c_f32(0.5), c_f32(2.0), None)
    assert np.array_equal(b.to_array(np.float32, n), orc.synth_uniform_f32(9, 7, 0, n, 0.5, 2.0))
    rows, cols = 300, 2880
    dc, ds = DeviceBuffer(rows * cols), DeviceBuffer(3 * 23 * 4)
    capi.call("eb_synth_weight_fp8", c_vp(dc.ptr), c_vp(ds.ptr), c_i64(rows + 128), c_i64(cols), c_i64(128),
              c_i64(rows), c_u64(1), c_u64(8), c_f32(0.02), None)
    codes, scales = orc.synth_weight_fp8(1, 8, rows + 128, cols, 128, rows, 0.02)
    assert np.array_equal(ds.to_array(np.float32, (3, 23)), scales)
    assert np.array_equal(dc.to_array(np.uint8, (rows, cols)), codes)


@pytest.mark.parametrize("n_kv", [8, 2])
def test_kv_append_bit_exact(gpu, n_kv):
    import eidola_b200 as eb
    from eidola_b200.capi import DeviceBuffer
    rng = np.random.default_rng(0)
    sched = eb.Scheduler(64, PAGE, 4, 17, seed=0)
    slots = [sched.admit(L) for L in (7, 33, 128, 250)]
    q_lens = [1, 5, 2, 3]
    for s, q in zip(slots, q_lens):
        sched.extend(s, sched.seq_len(s) + q)
    p = sched.pack(slots, q_lens)
    bt = sched.block_tables()
    T = p["n_tokens"]
    stride = (8 * n_kv + 2 * n_kv) * HEAD_DIM  # a fused [q | k | v] row
    qkv = orc.synth_normal_bf16(3, 1, 0, T * stride).reshape(T, stride)
    cache = orc.synth_normal_bf16(3, 2, 0, 64 * 2 * n_kv * PAGE * HEAD_DIM).reshape(64, 2, n_kv, PAGE, HEAD_DIM)
    want = cache.copy()
    k_col, v_col = 8 * n_kv * HEAD_DIM, 9 * n_kv * HEAD_DIM
    orc.kv_append(want, n_kv, HEAD_DIM, PAGE, qkv[:, k_col:], qkv[:, v_col:], stride, bt, p["tok_slot"], p["positions"])
    assert not np.array_equal(want, cache)
    d_cache, d_qkv = DeviceBuffer.from_array(cache), DeviceBuffer.from_array(qkv)
    d_bt, d_slot, d_pos = (DeviceBuffer.from_array(a) for a in (bt, p["tok_slot"], p["positions"]))
    eb.kv_append(d_cache.ptr, 64, n_kv, HEAD_DIM, PAGE, d_qkv.ptr + 2 * k_col, d_qkv.ptr + 2 * v_col, stride, d_bt.ptr,
                 bt.shape[1], d_slot.ptr, d_pos.ptr, T)
    got = d_cache.to_array(np.uint16, cache.shape)
    assert np.array_equal(got, want)
    del rng


CTX_SMALL = [7, 33, 128, 250, 16, 1, 129, 1000, 17, 2049]


@pytest.mark.parametrize("n_kv", [8, 4, 2, 1])
@pytest.mark.parametrize("window", [0, 128])
@pytest.mark.parametrize("q_mode", ["decode", "verify5", "ragged"])
def test_attention_small_matches_oracle(gpu, n_kv, window, q_mode):
    ctx = np.array(CTX_SMALL, np.int32)
    if q_mode == "decode":
        ql = np.ones_like(ctx)
    elif q_mode == "verify5":
        ql = np.minimum(ctx, 5)
    else:
        ql = np.minimum(ctx, np.array([1, 2, 3, 4, 5, 1, 6, 2, 1, 3], np.int32))
    case = AttnCase(ctx, ql, n_kv, seed=1, sm_count=gpu["sm_count"])
    want = case.oracle(window)
    for chunk in (0, 8, 3):
        got, plan = case.run(window, chunk)
        assert_close_bf16(got, want, atol=ATTN_ATOL, what=f"n_kv={n_kv} window={window} {q_mode} chunk={chunk}")
    assert plan["n_items"] > len(ctx) or window  # chunk 3 really split something


@pytest.mark.parametrize("kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("n_kv", [8, 4, 1])
@pytest.mark.parametrize("window", [0, 128, 2048])
def test_attention_verify_kernels_match_oracle(gpu, n_kv, window, kernel, monkeypatch):
    """Verify shapes run on the tcgen05 kernel when the items are long (full layers, windows of 2048 tokens and more)
    and on the mma.sync kernel otherwise; EIDOLA_B200_ATTN_VERIFY=mma keeps everything on the latter.  Both against the
    same oracle at the same tolerance: ragged query lengths, split contexts, windows, fewer KV heads per rank, and plans
    cut the way the entry point's kernel choice asks for."""
    import eidola_b200 as eb
    if kernel == "mma":
        monkeypatch.setenv("EIDOLA_B200_ATTN_VERIFY", "mma")
    else:
        monkeypatch.delenv("EIDOLA_B200_ATTN_VERIFY", raising=False)
    ctx = np.array(CTX_SMALL, np.int32)
    for ql in (np.minimum(ctx, 5), np.minimum(ctx, np.array([1, 2, 3, 4, 5, 1, 6, 2, 1, 3], np.int32))):
        case = AttnCase(ctx, ql, n_kv, seed=2, sm_count=gpu["sm_count"])
        want = case.oracle(window)
        for chunk in (0, 3):
            got, _ = case.run(window, chunk)
            assert_close_bf16(got, want, atol=ATTN_ATOL, what=f"{kernel} n_kv={n_kv} window={window} chunk={chunk}")
        # the plan the engine would make for this launch
        case.sm_count = eb.attn_plan_sm_count(gpu["sm_count"], int(ql.max()), 8 * n_kv, n_kv, window)
        got, _ = case.run(window, 0)
        assert_close_bf16(got, want, atol=ATTN_ATOL, what=f"{kernel} n_kv={n_kv} window={window} planned for its kernel")


def test_attn_plan_sm_count_follows_the_kernel_choice(gpu):
    import eidola_b200 as eb
    sm = gpu["sm_count"]
    assert eb.attn_plan_sm_count(sm, 1, 64, 8, 0) == sm          # decode: one CTA per item
    assert eb.attn_plan_sm_count(sm, 2, 64, 8, 0) == sm          # 16 rows still fit the decode tile
    assert eb.attn_plan_sm_count(sm, 5, 64, 8, 0) == 2 * sm // 8  # verify, full layer: one CTA per (item, KV head), two per SM
    assert eb.attn_plan_sm_count(sm, 5, 16, 2, 0) == sm
    assert eb.attn_plan_sm_count(sm, 5, 8, 1, 0) == 2 * sm
    assert eb.attn_plan_sm_count(sm, 5, 64, 8, 128) == sm        # short window: the mma.sync kernel
    assert eb.attn_plan_sm_count(sm, 5, 64, 8, 4096) == 2 * sm // 8


@pytest.mark.parametrize("n_kv", [2, 8])
@pytest.mark.parametrize("window", [0, 128])
def test_attention_group_of_four(gpu, n_kv, window):
    """8 query heads over 2 KV heads (the tiny decode configuration) and 32 over 8: GQA groups of 4."""
    ctx = np.array(CTX_SMALL, np.int32)
    ql = np.minimum(ctx, np.array([1, 2, 3, 4, 5, 1, 12, 2, 1, 7], np.int32))
    case = AttnCase(ctx, ql, n_kv, seed=3, sm_count=gpu["sm_count"], group=4)
    want = case.oracle(window)
    for chunk in (0, 5):
        got, _ = case.run(window, chunk)
        assert_close_bf16(got, want, atol=ATTN_ATOL, what=f"group 4, n_kv={n_kv} window={window} chunk={chunk}")


def test_attention_benchmark_shape_matches_oracle(gpu):
    """256 ragged sequences, lognormal(median 2048, sigma 1) clipped to [16, 32768], 64 q / 8 kv heads, seed 1."""
    ctx = lognormal_lengths(256, 2048, 1.0, 16, 32768, seed=1)
    case = AttnCase(ctx, np.ones_like(ctx), 8, seed=1, sm_count=gpu["sm_count"], device_synth=True)
    got_full, plan = case.run(0)
    got_win, _ = case.run(128)
    assert plan["n_items"] >= 2 * gpu["sm_count"]
    # the oracle needs ~6e9 multiply-adds for the whole batch; check the longest, the shortest and 22 others
    order = np.argsort(ctx)
    pick = sorted(set([int(order[0]), int(order[-1])] + [int(i) for i in order[5::11]]))
    want_full = case.oracle(0, pick)
    want_win = case.oracle(128, pick)
    rows = np.array(pick)
    assert_close_bf16(got_full[rows], want_full[rows], atol=ATTN_ATOL, what="benchmark shape, full")
    assert_close_bf16(got_win[rows], want_win[rows], atol=ATTN_ATOL, what="benchmark shape, window 128")
    # size-independent properties on all 256 sequences:
    # (1) split-K chunking changes only the summation order
    got_c64, _ = case.run(0, 64)
    assert_close_bf16(got_c64, got_full, atol=ATTN_ATOL, what="chunk 64 vs planned chunk")
    # (2) outputs are convex combinations of V rows scaled by < 1: bounded by max |V|
    assert np.abs(bf16_to_f32(got_full)).max() <= 6.0
    # (3) a windowed layer equals a full layer for every sequence no longer than the window
    short = np.nonzero(ctx <= 128)[0]
    if len(short):
        assert np.array_equal(got_win[short], got_full[short])


def test_attention_is_invariant_to_physical_page_placement(gpu):
    """Same logical K/V at different physical pages gives bit-identical output."""
    from eidola_b200.capi import DeviceBuffer
    ctx = np.array([300, 45, 1100, 16], np.int32)
    case = AttnCase(ctx, [1, 2, 1, 1], 8, seed=5, sm_count=gpu["sm_count"])
    a, _ = case.run(0, 16)
    perm = np.random.default_rng(1).permutation(case.num_pages).astype(np.int32)
    moved = np.empty_like(case.cache)
    moved[perm] = case.cache  # old page p now lives at perm[p]
    bt2 = np.where(case.bt >= 0, perm[np.maximum(case.bt, 0)], -1).astype(np.int32)
    case.d_cache = DeviceBuffer.from_array(moved)
    case.d_bt = DeviceBuffer.from_array(bt2)
    b, _ = case.run(0, 16)
    assert np.array_equal(a, b)


def test_out_of_range_page_is_flagged_not_faulted(gpu):
    import eidola_b200 as eb
    from eidola_b200.capi import DeviceBuffer
    case = AttnCase([40], [1], 8, seed=2, sm_count=gpu["sm_count"])
    bad = case.bt.copy()
    bad[0, 1] = case.num_pages + 7
    case.d_bt = DeviceBuffer.from_array(bad)
    case.run(0)
    assert eb.status_read() & 0x2000
    assert eb.status_read() == 0
