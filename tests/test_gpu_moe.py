"""GPU parity of the routing and glue operators against the oracle (bit-exact where the arithmetic is exact)."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.helpers import assert_close_bf16, bf16_to_f32

pytestmark = pytest.mark.gpu


def _dev(a):
    from eidola_b200.capi import DeviceBuffer
    return DeviceBuffer.from_array(np.ascontiguousarray(a))


def _call(fn, *args):
    from eidola_b200 import capi
    capi.call(fn, *args)


# 256 / 37 / 4 / 5 tokens: one token per CTA; 601: two tokens per CTA (odd count); 1000 and 2560: the staged eight-tokens-per-CTA kernel
@pytest.mark.parametrize("T,E,H,k", [(256, 32, 2880, 4), (37, 128, 2880, 4), (4, 8, 512, 2), (5, 256, 512, 8),
                                     (601, 128, 2880, 4), (1000, 32, 2880, 4), (2560, 128, 2880, 4)])
def test_router_indices_and_logits_bit_exact(gpu, T, E, H, k):
    from eidola_b200.capi import DeviceBuffer, c_i32, c_vp
    x = orc.synth_normal_bf16(5, 1, 0, T * H).reshape(T, H)
    wr = orc.synth_normal_bf16(5, 2, 0, E * H, 0.02).reshape(E, H)
    wr[E - 1] = wr[1]  # exact ties: the lower expert must win
    want_idx, want_w, want_l = orc.router_topk(x, wr, k)
    d_x, d_wr = _dev(x), _dev(wr)
    d_idx, d_w, d_l = DeviceBuffer(T * k * 4), DeviceBuffer(T * k * 4), DeviceBuffer(T * E * 4)
    _call("eb_moe_route", c_vp(d_x.ptr), c_vp(d_wr.ptr), c_i32(T), c_i32(E), c_i32(H), c_i32(k), c_vp(d_idx.ptr),
          c_vp(d_w.ptr), c_vp(d_l.ptr), None)
    assert np.array_equal(d_l.to_array(np.float32, (T, E)), want_l)
    assert np.array_equal(d_idx.to_array(np.int32, (T, k)), want_idx)
    assert np.allclose(d_w.to_array(np.float32, (T, k)), want_w, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("T,E,k", [(256, 32, 4), (2560, 128, 4), (3, 8, 2), (1, 4, 4)])
def test_permute_bit_exact(gpu, T, E, k):
    from eidola_b200.capi import DeviceBuffer, c_i32, c_vp
    rng = np.random.default_rng(T)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    want_seg, want_perm = orc.moe_permute(idx, E)
    d_idx = _dev(idx)
    d_seg, d_perm, d_rt = DeviceBuffer((E + 1) * 4), DeviceBuffer(T * k * 4), DeviceBuffer(T * k * 4)
    _call("eb_moe_permute", c_vp(d_idx.ptr), c_i32(T), c_i32(k), c_i32(E), c_vp(d_seg.ptr), c_vp(d_perm.ptr),
          c_vp(d_rt.ptr), None)
    assert np.array_equal(d_seg.to_array(np.int32, E + 1), want_seg)
    perm = d_perm.to_array(np.int32, (T, k))
    assert np.array_equal(perm, want_perm)
    rt = d_rt.to_array(np.int32, T * k)
    assert np.array_equal(rt[perm.reshape(-1)], np.repeat(np.arange(T), k))


def test_moe_pipeline_matches_oracle(gpu):
    """route -> permute -> gather+quantise -> W1 -> silu*up+quantise -> W2 -> combine, against orc_moe_forward."""
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer, c_i32, c_i64, c_vp
    T, E, H, I, k = 200, 8, 768, 640, 4
    R = T * k
    h = orc.synth_normal_bf16(6, 1, 0, T * H).reshape(T, H)
    wr = orc.synth_normal_bf16(6, 2, 0, E * H, 0.02).reshape(E, H)
    w1 = [orc.synth_weight_fp8(6, 10 + e, 2 * I, H, 0, 2 * I, 0.02) for e in range(E)]
    w2 = [orc.synth_weight_fp8(6, 30 + e, H, I, 0, H, 0.02) for e in range(E)]
    w1c, w1s = np.stack([a for a, _ in w1]), np.stack([b for _, b in w1])
    w2c, w2s = np.stack([a for a, _ in w2]), np.stack([b for _, b in w2])
    idx, wts, _ = orc.router_topk(h, wr, k)
    x0 = orc.synth_normal_bf16(6, 3, 0, T * H).reshape(T, H)  # residual stream
    want_moe = orc.moe_forward(h, idx, wts, w1c, w1s, w2c, w2s)
    want_x = x0.copy()
    orc.residual_add(want_x, want_moe)

    d_h, d_wr, d_x = _dev(h), _dev(wr), _dev(x0)
    d_w1c, d_w1s, d_w2c, d_w2s = _dev(w1c), _dev(w1s), _dev(w2c), _dev(w2s)
    d_idx, d_w = DeviceBuffer(R * 4), DeviceBuffer(R * 4)
    d_seg, d_perm, d_rt = DeviceBuffer((E + 1) * 4), DeviceBuffer(R * 4), DeviceBuffer(R * 4)
    kbH, kbI, nblk = (H + 127) // 128, (I + 127) // 128, R // 128 + E
    d_xp8, d_sxp = DeviceBuffer(R * H), DeviceBuffer(nblk * kbH * 4)
    d_gu, d_a8, d_sa, d_y = DeviceBuffer(R * 2 * I * 2), DeviceBuffer(R * I), DeviceBuffer(nblk * kbI * 4), DeviceBuffer(R * H * 2)
    d_ws = DeviceBuffer(host.gemm_workspace(R, 2 * I, E))
    _call("eb_moe_route", c_vp(d_h.ptr), c_vp(d_wr.ptr), c_i32(T), c_i32(E), c_i32(H), c_i32(k), c_vp(d_idx.ptr),
          c_vp(d_w.ptr), None, None)
    assert np.array_equal(d_idx.to_array(np.int32, (T, k)), idx)
    _call("eb_moe_permute", c_vp(d_idx.ptr), c_i32(T), c_i32(k), c_i32(E), c_vp(d_seg.ptr), c_vp(d_perm.ptr),
          c_vp(d_rt.ptr), None)
    _call("eb_quant_gather_block128", c_vp(d_h.ptr), c_i64(H), c_i32(T), c_vp(d_rt.ptr), c_i32(R), c_i32(H),
          c_vp(d_seg.ptr), c_i32(E), c_vp(d_xp8.ptr), c_vp(d_sxp.ptr), None)
    seg, perm = orc.moe_permute(idx, E)
    xp = np.empty((R, H), np.uint16)
    xp[perm.reshape(-1)] = np.repeat(h, k, axis=0)
    want_xp8, want_sxp = orc.quant_act_block128(xp, seg)
    assert np.array_equal(d_xp8.to_array(np.uint8, (R, H)), want_xp8)
    assert np.array_equal(d_sxp.to_array(np.float32, want_sxp.shape), want_sxp)
    host.gemm_fp8(d_xp8.ptr, d_sxp.ptr, d_w1c.ptr, d_w1s.ptr, d_gu.ptr, R, 2 * I, H, n_groups=E, d_seg_off=d_seg.ptr,
                  work=d_ws)
    _call("eb_quant_silu_mul_block128", c_vp(d_gu.ptr), c_i64(2 * I), c_i32(R), c_i32(I), c_vp(d_seg.ptr), c_i32(E),
          c_vp(d_a8.ptr), c_vp(d_sa.ptr), None)
    host.gemm_fp8(d_a8.ptr, d_sa.ptr, d_w2c.ptr, d_w2s.ptr, d_y.ptr, R, H, I, n_groups=E, d_seg_off=d_seg.ptr,
                  work=d_ws)
    _call("eb_moe_combine", c_vp(d_y.ptr), c_vp(d_perm.ptr), c_vp(d_w.ptr), c_i32(T), c_i32(k), c_i32(H), c_vp(d_x.ptr), None)
    got_x = d_x.to_array(np.uint16, (T, H))
    # expert outputs are O(0.01); the residual stream is O(1): compare the stream with the usual bf16 bound and the
    # expert contribution itself with a tight absolute bound
    assert_close_bf16(got_x, want_x, atol=2e-3, rtol=2.0 ** -7, what="moe residual stream")
    contrib = bf16_to_f32(got_x) - bf16_to_f32(x0)
    want_contrib = bf16_to_f32(want_x) - bf16_to_f32(x0)
    assert np.abs(want_contrib).max() > 1e-3
    assert np.abs(contrib - want_contrib).max() <= 1.6e-2  # one bf16 ulp of the O(1) stream either way
    # the expert outputs themselves, against the oracle's stages on the same permuted rows
    gu = orc.gemm_fp8_grouped(want_xp8, want_sxp, seg, w1c, w1s)
    g, u = bf16_to_f32(gu[:, :I]), bf16_to_f32(gu[:, I:])
    act = orc.bf16_encode((g / (np.float32(1.0) + np.exp(-g)) * u).astype(np.float32))
    a8, sa = orc.quant_act_block128(act, seg)
    want_y = orc.gemm_fp8_grouped(a8, sa, seg, w2c, w2s)
    assert_close_bf16(d_gu.to_array(np.uint16, (R, 2 * I)), gu, atol=1e-3, rtol=2.0 ** -7, what="W1 output")
    assert_close_bf16(d_y.to_array(np.uint16, (R, H)), want_y, atol=1e-3, rtol=2.0 ** -7, what="W2 output")


def test_combine_is_bit_exact_given_expert_outputs(gpu):
    from eidola_b200.capi import DeviceBuffer, c_i32, c_vp
    T, k, H, E = 33, 4, 512, 8
    rng = np.random.default_rng(7)
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    _, perm = orc.moe_permute(idx, E)
    y = orc.synth_normal_bf16(7, 1, 0, T * k * H, 0.05).reshape(T * k, H)
    wts = rng.dirichlet(np.ones(k), size=T).astype(np.float32)
    x0 = orc.synth_normal_bf16(7, 2, 0, T * H).reshape(T, H)
    yf = bf16_to_f32(y)
    acc = np.zeros((T, H), np.float32)
    for j in range(k):  # fmaf(w, y, acc) in slot order, emulated in float64 then rounded once per step
        acc = (wts[:, j:j + 1].astype(np.float64) * yf[perm[:, j]].astype(np.float64) + acc.astype(np.float64)).astype(np.float32)
    want = x0.copy()
    orc.residual_add(want, orc.bf16_encode(acc))
    d_x, d_y, d_perm, d_wts = _dev(x0), _dev(y), _dev(perm), _dev(wts)  # keep the buffers alive across the call
    _call("eb_moe_combine", c_vp(d_y.ptr), c_vp(d_perm.ptr), c_vp(d_wts.ptr), c_i32(T), c_i32(k), c_i32(H),
          c_vp(d_x.ptr), None)
    assert np.array_equal(d_x.to_array(np.uint16, (T, H)), want)


def test_glue_kernels(gpu):
    from eidola_b200.capi import DeviceBuffer, c_f32, c_i32, c_i64, c_vp
    T, H = 37, 2880
    x = orc.synth_normal_bf16(8, 1, 0, T * H, 2.0).reshape(T, H)
    g = (1.0 + 0.1 * orc.synth_normal_f32(8, 2, 0, H)).astype(np.float32)
    d_x, d_y, d_g = _dev(x), DeviceBuffer(T * H * 2), _dev(g)
    _call("eb_rmsnorm", c_vp(d_x.ptr), c_vp(d_g.ptr), c_i32(T), c_i32(H), c_f32(1e-5), c_vp(d_y.ptr), None)
    assert np.array_equal(d_y.to_array(np.uint16, (T, H)), orc.rmsnorm(x, g, 1e-5))  # fixed summation order: bit-exact
    # rotary: bit-exact (table from the library's host routine must equal the oracle's)
    import ctypes as C
    max_pos, D = 300, 64
    hc, hs = np.empty((max_pos, D // 2), np.float32), np.empty((max_pos, D // 2), np.float32)
    _call("eb_rope_table", c_i32(max_pos), c_i32(D), C.c_double(150000.0), hc.ctypes.data_as(c_vp), hs.ctypes.data_as(c_vp))
    oc, os_ = orc.rope_table(max_pos, D, 150000.0)
    assert np.array_equal(hc, oc) and np.array_equal(hs, os_)
    qkv = orc.synth_normal_bf16(8, 3, 0, T * 768).reshape(T, 768)
    pos = (np.arange(T) * 7 % max_pos).astype(np.int32)
    want = qkv.copy()
    orc.rope_inplace(want, 0, 10, D, pos, oc, os_)
    d_q, d_pos, d_hc, d_hs = _dev(qkv), _dev(pos), _dev(hc), _dev(hs)
    _call("eb_rope", c_vp(d_q.ptr), c_i64(768), c_i32(10), c_i32(D), c_vp(d_pos.ptr), c_i32(T), c_vp(d_hc.ptr),
          c_vp(d_hs.ptr), c_i32(max_pos), None)
    assert np.array_equal(d_q.to_array(np.uint16, (T, 768)), want)
    # residual add, embedding gather, argmax: exact
    y = orc.synth_normal_bf16(8, 4, 0, T * H).reshape(T, H)
    want = x.copy()
    orc.residual_add(want, y)
    d_x2, d_y2 = _dev(x), _dev(y)
    _call("eb_residual_add", c_vp(d_x2.ptr), c_vp(d_y2.ptr), c_i64(T * H), None)
    assert np.array_equal(d_x2.to_array(np.uint16, (T, H)), want)
    V = 1000
    table = orc.synth_normal_bf16(8, 5, 0, V * H, 0.02).reshape(V, H)
    toks = (np.arange(T) * 131 % V).astype(np.int32)
    d_e, d_table, d_toks = DeviceBuffer(T * H * 2), _dev(table), _dev(toks)
    _call("eb_embed", c_vp(d_table.ptr), c_i32(V), c_i32(H), c_vp(d_toks.ptr), c_i32(T), c_vp(d_e.ptr), None)
    assert np.array_equal(d_e.to_array(np.uint16, (T, H)), orc.embed(table, toks))
    Vb = 201088
    logits = orc.synth_normal_bf16(8, 6, 0, 5 * Vb).reshape(5, Vb)
    logits[1, 777] = logits[1, 200000] = 0x4120  # two equal maxima (10.0): the lower id wins, margin 0
    want_tok, want_m = orc.argmax(logits)
    d_t, d_m, d_lg = DeviceBuffer(5 * 4), DeviceBuffer(5 * 4), _dev(logits)
    _call("eb_argmax", c_vp(d_lg.ptr), c_i32(5), c_i64(Vb), c_i64(Vb), c_vp(d_t.ptr), c_vp(d_m.ptr), None)
    assert np.array_equal(d_t.to_array(np.int32, 5), want_tok) and want_tok[1] == 777
    assert np.array_equal(d_m.to_array(np.float32, 5), want_m) and want_m[1] == 0
