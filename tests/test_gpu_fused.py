"""GPU: the fused epilogue kernels against the oracle's separate steps (rounding points are the same, so integer and
bf16 results are bit-exact except where a row sum of squares is accumulated in another order)."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.helpers import assert_close_bf16

pytestmark = pytest.mark.gpu


def _dev(a):
    from eidola_b200.capi import DeviceBuffer
    return DeviceBuffer.from_array(np.ascontiguousarray(a))


def _call(fn, *args):
    from eidola_b200 import capi
    capi.call(fn, *args)


@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("n_q,n_kv", [(64, 8), (8, 2)])
def test_qkv_rope_append(gpu, splits, n_q, n_kv):
    import eidola_b200 as eb
    from eidola_b200.capi import DeviceBuffer, c_i32, c_vp
    D, PAGE, T = 64, 16, 9
    N = (n_q + 2 * n_kv) * D
    sched = eb.Scheduler(64, PAGE, 4, 17, seed=0)
    slots = [sched.admit(L) for L in (7, 33, 128, 250)]
    q_lens = [1, 5, 2, 1]
    for s, q in zip(slots, q_lens):
        sched.extend(s, sched.seq_len(s) + q)
    p = sched.pack(slots, q_lens)
    bt = sched.block_tables()
    rng = np.random.default_rng(1)
    part = rng.normal(0, 1, size=(splits, T, N)).astype(np.float32)
    acc = np.zeros((T, N), np.float32)
    for s in range(splits):
        acc = acc + part[s]
    qkv = orc.bf16_encode(acc)
    cos, sin = orc.rope_table(300, D, 150000.0)
    want = qkv.copy()
    orc.rope_inplace(want, 0, n_q + n_kv, D, p["positions"], cos, sin)
    cache = orc.synth_normal_bf16(3, 2, 0, 64 * 2 * n_kv * PAGE * D).reshape(64, 2, n_kv, PAGE, D)
    want_cache = cache.copy()
    orc.kv_append(want_cache, n_kv, D, PAGE, want[:, n_q * D:], want[:, (n_q + n_kv) * D:], N, bt, p["tok_slot"], p["positions"])
    d_part, d_qkv, d_cache = _dev(part), _dev(qkv if splits == 1 else np.zeros_like(qkv)), _dev(cache)
    d_pos, d_cos, d_sin, d_bt, d_slot = _dev(p["positions"]), _dev(cos), _dev(sin), _dev(bt), _dev(p["tok_slot"])
    _call("eb_qkv_rope_append", c_vp(d_part.ptr if splits > 1 else None), c_i32(splits), c_vp(d_qkv.ptr), c_i32(T), c_i32(n_q),
          c_i32(n_kv), c_i32(D), c_vp(d_pos.ptr), c_vp(d_cos.ptr), c_vp(d_sin.ptr), c_i32(300), c_vp(d_cache.ptr), c_i32(64),
          c_i32(PAGE), c_vp(d_bt.ptr), c_i32(bt.shape[1]), c_vp(d_slot.ptr), None)
    got = d_qkv.to_array(np.uint16, (T, N))
    assert np.array_equal(got[:, : n_q * D], want[:, : n_q * D])
    assert np.array_equal(d_cache.to_array(np.uint16, cache.shape), want_cache)


@pytest.mark.parametrize("splits", [1, 8])
@pytest.mark.parametrize("H", [2880, 512])
def test_oproj_residual_rmsnorm(gpu, splits, H):
    from eidola_b200.capi import DeviceBuffer, c_f32, c_i32, c_vp
    T = 37
    rng = np.random.default_rng(2)
    part = rng.normal(0, 0.3, size=(splits, T, H)).astype(np.float32)
    acc = np.zeros((T, H), np.float32)
    for s in range(splits):
        acc = acc + part[s]
    o = orc.bf16_encode(acc)
    x0 = orc.synth_normal_bf16(9, 1, 0, T * H).reshape(T, H)
    g = (1.0 + 0.1 * orc.synth_normal_f32(9, 2, 0, H)).astype(np.float32)
    want_x = x0.copy()
    orc.residual_add(want_x, o)
    want_h = orc.rmsnorm(want_x, g, 1e-5)
    d_part, d_o, d_x, d_g, d_h = _dev(part), _dev(o), _dev(x0), _dev(g), DeviceBuffer(T * H * 2)
    _call("eb_oproj_residual_rmsnorm", c_vp(d_part.ptr if splits > 1 else None), c_i32(splits),
          c_vp(d_o.ptr if splits == 1 else None), c_vp(d_x.ptr), c_vp(d_g.ptr), c_i32(T), c_i32(H), c_f32(1e-5), c_vp(d_h.ptr), None)
    assert np.array_equal(d_x.to_array(np.uint16, (T, H)), want_x)
    assert np.array_equal(d_h.to_array(np.uint16, (T, H)), want_h)  # fixed summation order: bit-exact


def test_combine_rmsnorm_and_permute_tiles(gpu):
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer, c_f32, c_i32, c_vp
    T, k, H, E = 200, 4, 2880, 32
    R = T * k
    rng = np.random.default_rng(7)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    want_seg, want_perm = orc.moe_permute(idx, E)
    d_idx = _dev(idx)
    d_seg, d_perm, d_rt = DeviceBuffer((E + 1) * 4), DeviceBuffer(R * 4), DeviceBuffer(R * 4)
    tn = 64
    ws_bytes = host.gemm_workspace(R, H, E)
    d_ws, d_ws2 = DeviceBuffer(ws_bytes), DeviceBuffer(ws_bytes)
    _call("eb_moe_permute_tiles", c_vp(d_idx.ptr), c_i32(T), c_i32(k), c_i32(E), c_vp(d_seg.ptr), c_vp(d_perm.ptr),
          c_vp(d_rt.ptr), c_i32(tn), c_vp(d_ws.ptr), None)
    assert np.array_equal(d_seg.to_array(np.int32, E + 1), want_seg)
    perm = d_perm.to_array(np.int32, (T, k))
    assert np.array_equal(perm, want_perm)
    _call("eb_gemm_group_tiles", c_vp(d_seg.ptr), c_i32(E), c_i32(R), c_i32(tn), c_vp(d_ws2.ptr), None)
    max_tiles = R // tn + E
    words = E + 2 + 2 * max_tiles
    a, b = d_ws.to_array(np.int32, words), d_ws2.to_array(np.int32, words)
    n_tiles = int(a[E + 1])
    assert n_tiles == int(b[E + 1]) == int(np.ceil(np.diff(want_seg) / tn).sum())
    assert np.array_equal(a[: E + 2], b[: E + 2])
    assert np.array_equal(a[E + 2: E + 2 + n_tiles], b[E + 2: E + 2 + n_tiles])
    assert np.array_equal(a[E + 2 + max_tiles: E + 2 + max_tiles + n_tiles], b[E + 2 + max_tiles: E + 2 + max_tiles + n_tiles])
    # combine + residual + rmsnorm
    y = orc.synth_normal_bf16(7, 1, 0, R * H, 0.05).reshape(R, H)
    wts = rng.dirichlet(np.ones(k), size=T).astype(np.float32)
    x0 = orc.synth_normal_bf16(7, 2, 0, T * H).reshape(T, H)
    g = (1.0 + 0.1 * orc.synth_normal_f32(7, 3, 0, H)).astype(np.float32)
    d_y, d_w, d_x, d_x2, d_g, d_h = _dev(y), _dev(wts), _dev(x0), _dev(x0), _dev(g), DeviceBuffer(T * H * 2)
    _call("eb_moe_combine", c_vp(d_y.ptr), c_vp(d_perm.ptr), c_vp(d_w.ptr), c_i32(T), c_i32(k), c_i32(H), c_vp(d_x2.ptr), None)
    want_x = d_x2.to_array(np.uint16, (T, H))  # the unfused kernel is itself checked bit-exactly in test_gpu_moe
    _call("eb_moe_combine_rmsnorm", c_vp(d_y.ptr), c_vp(d_perm.ptr), c_vp(d_w.ptr), c_i32(T), c_i32(k), c_i32(H), c_vp(d_x.ptr),
          c_vp(d_g.ptr), c_f32(1e-5), c_vp(d_h.ptr), None)
    assert np.array_equal(d_x.to_array(np.uint16, (T, H)), want_x)
    assert np.array_equal(d_h.to_array(np.uint16, (T, H)), orc.rmsnorm(want_x, g, 1e-5))  # fixed summation order: bit-exact


def test_argmax_partial_and_merge_equal_whole_row_argmax(gpu):
    """Vocabulary-parallel argmax: candidates of three unequal slices merge to the same token and top1 - top2 margin
    as eb_argmax over the whole row, including ties across slices (lower id wins)."""
    from eidola_b200.capi import DeviceBuffer, c_i32, c_i64, c_vp
    T, V = 37, 5000
    logits = orc.synth_normal_bf16(11, 1, 0, T * V, 2.0).reshape(T, V)
    logits[3, 100] = logits[3, 4000] = 0x4120   # 10.0 twice: a tie between the first and the last slice
    logits[5, :] = 0x3F80                       # a constant row: token 0, margin 0
    d_l = _dev(logits)
    d_tok, d_mg = DeviceBuffer(T * 4), DeviceBuffer(T * 4)
    _call("eb_argmax", c_vp(d_l.ptr), c_i32(T), c_i64(V), c_i64(V), c_vp(d_tok.ptr), c_vp(d_mg.ptr), None)
    want_tok, want_mg = d_tok.to_array(np.int32, T), d_mg.to_array(np.float32, T)
    cuts = [0, 1280, 3968, V]
    cap = 40
    d_cand = DeviceBuffer(3 * cap * 4 * 4)
    for r in range(3):
        v0, v1 = cuts[r], cuts[r + 1]
        _call("eb_argmax_partial", c_vp(d_l.ptr + 2 * v0), c_i32(T), c_i64(v1 - v0), c_i64(V), c_i32(v0),
              c_vp(d_cand.ptr + r * cap * 16), None)
    d_tok2, d_mg2 = DeviceBuffer(T * 4), DeviceBuffer(T * 4)
    _call("eb_argmax_merge", c_vp(d_cand.ptr), c_i32(3), c_i64(cap), c_i32(T), c_vp(d_tok2.ptr), c_vp(d_mg2.ptr), None)
    assert np.array_equal(d_tok2.to_array(np.int32, T), want_tok)
    assert np.array_equal(d_mg2.to_array(np.float32, T), want_mg)
    assert want_tok[3] == 100 and want_mg[3] == 0 and want_tok[5] == 0 and want_mg[5] == 0


def test_argmax_of_rows_without_a_finite_maximum_stays_in_the_vocabulary(gpu):
    """A row of NaN or -inf logits yields token 0 (never an id outside the vocabulary) and raises the status word, in
    the whole-row kernel and in the vocabulary-parallel pair alike; NaNs among finite values are ignored, as in the
    oracle."""
    import eidola_b200 as eb
    from eidola_b200.capi import DeviceBuffer, c_i32, c_i64, c_vp
    T, V = 6, 1000
    logits = orc.synth_normal_bf16(12, 1, 0, T * V, 2.0).reshape(T, V)
    logits[1, :] = 0x7FC0            # NaN everywhere
    logits[2, :] = 0xFF80            # -inf everywhere
    logits[3, 0] = 0x7FC0            # a NaN first, finite values after it
    logits[4, ::2] = 0x7FC0          # NaNs interleaved
    want_tok, _ = orc.argmax(logits)
    assert want_tok[1] == 0 and want_tok[2] == 0 and want_tok[3] != 0
    d_l = _dev(logits)
    d_tok, d_mg = DeviceBuffer(T * 4), DeviceBuffer(T * 4)
    _call("eb_argmax", c_vp(d_l.ptr), c_i32(T), c_i64(V), c_i64(V), c_vp(d_tok.ptr), c_vp(d_mg.ptr), None)
    assert np.array_equal(d_tok.to_array(np.int32, T), want_tok)
    assert eb.status_read() & 0x2000
    cuts = [0, 384, V]
    d_cand = DeviceBuffer(2 * T * 16)
    for r in range(2):
        _call("eb_argmax_partial", c_vp(d_l.ptr + 2 * cuts[r]), c_i32(T), c_i64(cuts[r + 1] - cuts[r]), c_i64(V), c_i32(cuts[r]),
              c_vp(d_cand.ptr + r * T * 16), None)
    d_tok2 = DeviceBuffer(T * 4)
    _call("eb_argmax_merge", c_vp(d_cand.ptr), c_i32(2), c_i64(T), c_i32(T), c_vp(d_tok2.ptr), None, None)
    assert np.array_equal(d_tok2.to_array(np.int32, T), want_tok)
    assert eb.status_read() & 0x2000
    assert eb.status_read() == 0
