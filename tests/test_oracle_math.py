"""Known-answer checks of the oracle's math against independent float64 numpy (CPU)."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.helpers import HEAD_DIM, PAGE, bf16_to_f32, make_cache_host, make_q_host, make_sinks_host


def _numpy_attention(q, cache, bt, slots, q_off, ctx, sinks, window, n_q, n_kv):
    qf, cf = bf16_to_f32(q).astype(np.float64), bf16_to_f32(cache).astype(np.float64)
    out = np.zeros((q.shape[0], n_q, HEAD_DIM))
    for i, slot in enumerate(slots):
        L, ql = ctx[i], q_off[i + 1] - q_off[i]
        pages = bt[slot, : (L + PAGE - 1) // PAGE]
        K = cf[pages, 0].transpose(1, 0, 2, 3).reshape(n_kv, -1, HEAD_DIM)[:, :L]
        V = cf[pages, 1].transpose(1, 0, 2, 3).reshape(n_kv, -1, HEAD_DIM)[:, :L]
        for j in range(ql):
            p = L - ql + j
            lo = max(0, p - window + 1) if window else 0
            for h in range(n_q):
                s = (K[h // 8, lo:p + 1] @ qf[q_off[i] + j].reshape(n_q, HEAD_DIM)[h]) * 0.125
                m = max(s.max(), sinks[h])
                e = np.exp(s - m)
                out[q_off[i] + j, h] = (e @ V[h // 8, lo:p + 1]) / (e.sum() + np.exp(sinks[h] - m))
    return out.reshape(q.shape[0], -1)


@pytest.mark.parametrize("window", [0, 128, 5])
def test_attention_matches_float64_numpy(window):
    n_kv, n_q = 2, 16
    ctx = np.array([7, 33, 128, 250, 16, 1], np.int32)
    ql = np.array([1, 3, 5, 2, 1, 1], np.int32)
    q_off = np.concatenate([[0], np.cumsum(ql)]).astype(np.int32)
    rng = np.random.default_rng(0)
    n_pages = 40
    perm = rng.permutation(n_pages)
    bt = np.full((6, 16), -1, np.int32)
    k = 0
    for i, L in enumerate(ctx):
        n = (L + PAGE - 1) // PAGE
        bt[i, :n] = perm[k:k + n]
        k += n
    cache = make_cache_host(n_pages, n_kv, 1)
    q = make_q_host(int(ql.sum()), n_q, 1)
    sinks = make_sinks_host(n_q, 1)
    slots = np.arange(6, dtype=np.int32)
    got = orc.attn_paged_sink(q, cache, bt, slots, q_off, ctx, sinks, window, n_q, n_kv)
    want = _numpy_attention(q, cache, bt, slots, q_off, ctx, sinks.astype(np.float64), window, n_q, n_kv)
    err = np.abs(bf16_to_f32(got) - want)
    assert (err <= 1e-5 + 2.0 ** -8 * np.abs(want)).all(), err.max()


def test_sink_only_denominator_analytic():
    """One key, q.k = 0: out = v * 1/(1 + e^sink) when sink >= 0 ... i.e. softmax over {0, sink} without a sink value."""
    n_kv, n_q = 1, 8
    cache = np.zeros((1, 2, n_kv, PAGE, HEAD_DIM), np.uint16)
    cache[0, 1, 0, 0, :] = orc.bf16_encode(np.full(HEAD_DIM, 2.0, np.float32))
    q = np.zeros((1, n_q * HEAD_DIM), np.uint16)
    sinks = np.array([0.0, 1.0, -1.0, 3.0, -30.0, 30.0, 0.5, -0.5], np.float32)
    out = orc.attn_paged_sink(q, cache, np.zeros((1, 1), np.int32), [0], [0, 1], [1], sinks, 0, n_q, n_kv)
    got = bf16_to_f32(out).reshape(n_q, HEAD_DIM)[:, 0]
    want = 2.0 / (1.0 + np.exp(sinks.astype(np.float64)))
    assert np.allclose(got, want, rtol=2.0 ** -8, atol=1e-12)


def test_gemm_power_of_two_scales_is_exact():
    """With power-of-two scales and small integers every partial sum is exact, so the result is the integer GEMM."""
    rng = np.random.default_rng(3)
    M, N, K = 130, 256, 320  # K tail block of 64
    xi = rng.integers(-3, 4, size=(M, K)).astype(np.float32)
    wi = rng.integers(-3, 4, size=(N, K)).astype(np.float32)
    x8, w8 = orc.e4m3_encode(xi), orc.e4m3_encode(wi)
    sx = (2.0 ** rng.integers(-2, 3, size=(2, 3))).astype(np.float32)
    sw = (2.0 ** rng.integers(-2, 3, size=(2, 3))).astype(np.float32)
    y = bf16_to_f32(orc.gemm_fp8_block(x8, sx, w8, sw))
    want = np.zeros((M, N))
    for kb in range(3):
        part = xi[:, kb * 128:(kb + 1) * 128].astype(np.float64) @ wi[:, kb * 128:(kb + 1) * 128].T.astype(np.float64)
        want += part * sx[np.arange(M) // 128, kb][:, None] * sw[np.arange(N) // 128, kb][None, :]
    assert np.array_equal(y, bf16_to_f32(orc.bf16_encode(want.astype(np.float32))))


def test_gemm_grouped_equals_per_group_dense():
    rng = np.random.default_rng(4)
    G, N, K = 3, 128, 256
    seg = [0, 5, 5, 140]
    x = orc.synth_normal_bf16(4, 1, 0, 140 * K).reshape(140, K)
    x8, sx = orc.quant_act_block128(x, seg)
    w8 = np.stack([orc.synth_weight_fp8(4, 10 + g, N, K, 0, N, 0.02)[0] for g in range(G)])
    sw = np.stack([orc.synth_weight_fp8(4, 10 + g, N, K, 0, N, 0.02)[1] for g in range(G)])
    y = orc.gemm_fp8_grouped(x8, sx, seg, w8, sw)
    y0 = orc.gemm_fp8_block(x8[0:5], sx[0:1], w8[0], sw[0])
    y2a = orc.gemm_fp8_block(x8[5:133], sx[1:2], w8[2], sw[2])
    y2b = orc.gemm_fp8_block(x8[133:140], sx[2:3], w8[2], sw[2])
    assert np.array_equal(y[0:5], y0) and np.array_equal(y[5:133], y2a) and np.array_equal(y[133:], y2b)
    # and against float64 on the dequantised operands
    xf = orc.e4m3_decode(x8[5:133]).astype(np.float64)
    wf = orc.e4m3_decode(w8[2]).astype(np.float64)
    want = sum((xf[:, kb * 128:(kb + 1) * 128] @ wf[:, kb * 128:(kb + 1) * 128].T) * float(sx[1, kb]) * float(sw[2][0, kb])
               for kb in range(2))
    assert np.abs(bf16_to_f32(y2a) - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6


def test_router_topk_order_ties_and_weights():
    T, E, H = 9, 32, 320
    x = orc.synth_normal_bf16(5, 1, 0, T * H).reshape(T, H)
    wr = orc.synth_normal_bf16(5, 2, 0, E * H, 0.02).reshape(E, H)
    wr[7] = wr[3]  # an exact tie: the lower index must win
    idx, wts, logits = orc.router_topk(x, wr, 4)
    ref = bf16_to_f32(x).astype(np.float64) @ bf16_to_f32(wr).astype(np.float64).T
    assert np.abs(logits - ref).max() < 1e-4
    assert np.array_equal(logits[:, 3], logits[:, 7])
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-logits[t, e], e))[:4]
        assert idx[t].tolist() == order
        if 3 in order or 7 in order:
            assert 3 in order and (7 not in order or order.index(3) < order.index(7))
        e = np.exp(logits[t, order].astype(np.float64) - logits[t, order[0]])
        assert np.allclose(wts[t], e / e.sum(), rtol=1e-5)
    seg, perm = orc.moe_permute(idx, E)
    flat = sorted(range(T * 4), key=lambda i: (idx.reshape(-1)[i], i))
    assert [int(perm.reshape(-1)[i]) for i in flat] == list(range(T * 4))
    assert seg[0] == 0 and seg[-1] == T * 4 and np.array_equal(np.diff(seg), np.bincount(idx.reshape(-1), minlength=E))


def test_rmsnorm_rope_argmax():
    x = orc.synth_normal_bf16(6, 1, 0, 3 * 512).reshape(3, 512)
    g = np.linspace(0.5, 1.5, 512).astype(np.float32)
    xf = bf16_to_f32(x).astype(np.float64)
    want = xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + 1e-5) * g
    got = bf16_to_f32(orc.rmsnorm(x, g, 1e-5))
    assert np.abs(got - want).max() <= 2.0 ** -8 * np.abs(want).max() + 1e-6
    c, s = orc.rope_table(300, 64, 150000.0)
    assert np.allclose(c[0], 1) and np.allclose(s[0], 0) and np.isclose(c[7, 0], np.cos(7.0)) and np.isclose(
        s[250, 31], np.sin(250 * 150000.0 ** (-62 / 64)))
    y = x.copy()
    pos = np.array([0, 7, 250], np.int32)
    orc.rope_inplace(y, 128, 2, 64, pos, c, s)
    assert np.array_equal(y[:, :128], x[:, :128]) and np.array_equal(y[:, 256:], x[:, 256:]) and np.array_equal(y[0], x[0])
    a, b = xf[1, 128:160], xf[1, 160:192]
    assert np.abs(bf16_to_f32(y[1, 128:160]) - (a * c[7] - b * s[7])).max() < 0.02
    # norm is preserved by a rotation
    assert abs(np.linalg.norm(bf16_to_f32(y[2, 128:192])) - np.linalg.norm(xf[2, 128:192])) < 0.05
    logits = orc.bf16_encode(np.array([[0.5, 2.0, 2.0, -1.0], [3.0, 1.0, 0.0, 2.5]], np.float32))
    tok, margin = orc.argmax(logits)
    assert tok.tolist() == [1, 0] and margin.tolist() == [0.0, 0.5]
    # NaN is never chosen; a row with nothing above -inf yields token 0
    odd = np.array([[0x7FC0, 0x3F80, 0x4000, 0x7FC0], [0x7FC0] * 4, [0xFF80] * 4], np.uint16)
    tok, _ = orc.argmax(odd)
    assert tok.tolist() == [2, 0, 0]


def test_column_bands_quantise_to_the_bands_of_the_whole_matrix():
    """What lets tensor-parallel ranks assemble the O projection's operand from their own heads: scale blocks are 128
    columns wide, so quantising a band of whole blocks alone gives the codes and scales the whole matrix has there, and
    the full-K product on the assembled operand is the single-GPU product bit for bit."""
    rng = np.random.default_rng(21)
    T, K, N, ranks = 200, 1024, 256, 4
    x = orc.bf16_encode(rng.normal(0, 1.5, size=(T, K)).astype(np.float32))
    codes, scales = orc.quant_act_block128(x)
    band = K // ranks
    parts = [orc.quant_act_block128(np.ascontiguousarray(x[:, r * band:(r + 1) * band])) for r in range(ranks)]
    assert np.array_equal(np.concatenate([p[0] for p in parts], axis=1), codes)
    assert np.array_equal(np.concatenate([p[1] for p in parts], axis=1), scales)
    # a token slice (rows 128..199, whole row blocks) of the assembled operand times the whole weight = those rows of Y
    w8, sw = orc.synth_weight_fp8(5, 9, N, K, 0, N, 0.05)
    y = orc.gemm_fp8_block(codes, scales, w8, sw)
    y_slice = orc.gemm_fp8_block(np.ascontiguousarray(codes[128:]), np.ascontiguousarray(scales[1:]), w8, sw)
    assert np.array_equal(y_slice, y[128:])
