"""GPU parity: activation quantiser (bit-exact) and block-scaled FP8 GEMM, dense and grouped, against the oracle."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.helpers import assert_close_bf16, bf16_to_f32

pytestmark = pytest.mark.gpu

# GEMM outputs: the tensor core sums each 128-wide K block in its own order and the scaled blocks are added in
# fp32, so |gpu - oracle| <= ATOL + one bf16 ulp of the oracle value.
G_ATOL, G_RTOL = 1e-2, 2.0 ** -7


def _dev(a):
    from eidola_b200.capi import DeviceBuffer
    return DeviceBuffer.from_array(np.ascontiguousarray(a))


def _sweep_inputs(M, N, K, seed):
    """The GEMM sweep inputs: entries ~ N(0,1) rounded to e4m3, scales uniform in [0.5, 2)."""
    x8 = orc.synth_normal_e4m3(seed, 1, 0, M * K).reshape(M, K)
    w8 = orc.synth_normal_e4m3(seed, 2, 0, N * K).reshape(N, K)
    kb = (K + 127) // 128
    sx = orc.synth_uniform_f32(seed, 3, 0, ((M + 127) // 128) * kb, 0.5, 2.0).reshape(-1, kb)
    sw = orc.synth_uniform_f32(seed, 4, 0, ((N + 127) // 128) * kb, 0.5, 2.0).reshape(-1, kb)
    return x8, sx, w8, sw


@pytest.mark.parametrize("rows,cols", [(1, 2880), (130, 2880), (256, 512), (300, 4096)])
def test_quant_act_dense_bit_exact(gpu, rows, cols):
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    x = orc.synth_normal_bf16(3, 1, 0, rows * cols, 3.0).reshape(rows, cols)
    x[0, :8] = 0
    want_c, want_s = orc.quant_act_block128(x)
    d_x, d_c = _dev(x), DeviceBuffer(rows * cols)
    d_s = DeviceBuffer(want_s.size * 4)
    host.quant_act_block128(d_x.ptr, cols, rows, cols, d_c.ptr, d_s.ptr)
    assert np.array_equal(d_s.to_array(np.float32, want_s.shape), want_s)
    assert np.array_equal(d_c.to_array(np.uint8, (rows, cols)), want_c)


@pytest.mark.parametrize("M", [1, 8, 64, 200, 256])
def test_gemm_dense_small_m_matches_oracle(gpu, M):
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    N, K = 5120, 2880
    x8, sx, w8, sw = _sweep_inputs(M, N, K, seed=2)
    want = orc.gemm_fp8_block(x8, sx, w8, sw)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    d_y = DeviceBuffer(M * N * 2)
    d_work = DeviceBuffer(host.gemm_workspace(M, N, 1))
    for splits, tn in ((1, 0), (0, 0), (4, 0), (1, 128), (1, 16)):
        d_y.zero()
        host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K, work=d_work, splits=splits,
                      tile_tokens=tn)
        got = d_y.to_array(np.uint16, (M, N))
        # outputs are O(100): compare relative to the bf16 grid of the value
        assert_close_bf16(got, want, atol=G_ATOL, rtol=G_RTOL, what=f"M={M} splits={splits} tn={tn}")


def test_gemm_power_of_two_scales_exact(gpu):
    """Small integers and power-of-two scales: every partial sum is exact, the GPU must equal the oracle bit for bit."""
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    rng = np.random.default_rng(3)
    M, N, K = 130, 384, 320
    x8 = orc.e4m3_encode(rng.integers(-3, 4, size=(M, K)).astype(np.float32))
    w8 = orc.e4m3_encode(rng.integers(-3, 4, size=(N, K)).astype(np.float32))
    sx = (2.0 ** rng.integers(-2, 3, size=(2, 3))).astype(np.float32)
    sw = (2.0 ** rng.integers(-2, 3, size=(3, 3))).astype(np.float32)
    want = orc.gemm_fp8_block(x8, sx, w8, sw)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    d_y = DeviceBuffer(M * N * 2)
    for tn in (16, 32, 64, 128):
        d_y.zero()
        host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K, tile_tokens=tn)
        assert np.array_equal(d_y.to_array(np.uint16, (M, N)), want), tn


@pytest.mark.parametrize("M", [1024, 4096])
def test_gemm_dense_large_m_sampled_rows(gpu, M):
    """Large M: the oracle checks three 128-row blocks; a checksum property covers the rest."""
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    N, K = 5120, 2880
    x8, sx, w8, sw = _sweep_inputs(M, N, K, seed=4)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    d_y = DeviceBuffer(M * N * 2)
    host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K)
    got = d_y.to_array(np.uint16, (M, N))
    for blk in (0, M // 256, M // 128 - 1):
        r = slice(blk * 128, blk * 128 + 128)
        want = orc.gemm_fp8_block(x8[r], sx[blk:blk + 1], w8, sw)
        assert_close_bf16(got[r], want, atol=G_ATOL, rtol=G_RTOL, what=f"M={M} block {blk}")
    # linearity in the scales: doubling sx doubles every output exactly (power of two)
    d_sx2 = _dev(sx * 2)
    d_y2 = DeviceBuffer(M * N * 2)
    host.gemm_fp8(d[0].ptr, d_sx2.ptr, d[2].ptr, d[3].ptr, d_y2.ptr, M, N, K)
    assert np.array_equal(bf16_to_f32(d_y2.to_array(np.uint16, (M, N))), 2 * bf16_to_f32(got))


@pytest.mark.parametrize("tn", [0, 16, 64, 128])
def test_gemm_grouped_matches_oracle(gpu, tn):
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    G, N, K = 6, 640, 2880
    seg = np.array([0, 5, 5, 140, 141, 400, 437], np.int32)  # an empty group, a 1-row group, multi-block groups
    R = int(seg[-1])
    x = orc.synth_normal_bf16(5, 1, 0, R * K).reshape(R, K)
    x8, sx = orc.quant_act_block128(x, seg)
    w = [orc.synth_weight_fp8(5, 10 + g, N, K, 0, N, 0.02) for g in range(G)]
    w8, sw = np.stack([a for a, _ in w]), np.stack([b for _, b in w])
    want = orc.gemm_fp8_grouped(x8, sx, seg, w8, sw)
    d_x, d_seg, d_w8, d_sw = _dev(x), _dev(seg), _dev(w8), _dev(sw)
    d_x8, d_sx = DeviceBuffer(R * K), DeviceBuffer((R // 128 + G) * 23 * 4)
    d_y = DeviceBuffer(R * N * 2)
    d_work = DeviceBuffer(host.gemm_workspace(R, N, G))
    host.quant_act_block128(d_x.ptr, K, R, K, d_x8.ptr, d_sx.ptr, d_seg_off=d_seg.ptr, n_groups=G)
    assert np.array_equal(d_x8.to_array(np.uint8, (R, K)), x8)
    assert np.array_equal(d_sx.to_array(np.float32, sx.shape), sx)
    d_y.zero()
    host.gemm_fp8(d_x8.ptr, d_sx.ptr, d_w8.ptr, d_sw.ptr, d_y.ptr, R, N, K, n_groups=G, d_seg_off=d_seg.ptr,
                  work=d_work, tile_tokens=tn)
    got = d_y.to_array(np.uint16, (R, N))
    assert_close_bf16(got, want, atol=1e-3, rtol=G_RTOL, what=f"grouped tn={tn}")


def test_gemm_workspace_too_small_is_refused_or_degrades(gpu):
    """The workspace size travels with the call: explicit K splits that would not fit are refused before any launch,
    automatic splitting falls back to what fits, and a grouped call with too little room for its tile table is refused."""
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer, EbError
    M, N, K = 8, 5120, 2880
    x8, sx, w8, sw = _sweep_inputs(M, N, K, seed=5)
    want = orc.gemm_fp8_block(x8, sx, w8, sw)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    d_y = DeviceBuffer(M * N * 2)
    small = DeviceBuffer(M * N * 4)  # room for one partial plane only
    with pytest.raises(EbError):
        host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K, work=small, splits=4)
    host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K, work=small, splits=0)
    assert_close_bf16(d_y.to_array(np.uint16, (M, N)), want, atol=G_ATOL, rtol=G_RTOL, what="auto splits, small workspace")
    seg = _dev(np.array([0, 3, 8], np.int32))
    w2 = _dev(np.concatenate([w8[:256], w8[256:512]]))
    with pytest.raises(EbError):
        host.gemm_fp8(d[0].ptr, d[1].ptr, w2.ptr, d[3].ptr, d_y.ptr, M, 256, K, n_groups=2, d_seg_off=seg.ptr,
                      work=DeviceBuffer(8))


@pytest.mark.parametrize("M,N,K", [(1024, 5120, 2880), (600, 2880, 512), (513, 200, 4096), (300, 65536, 256)])
def test_gemm_dense_prefill_sized_matches_oracle(gpu, M, N, K):
    """512 tokens and more (256 and more against a very tall weight matrix, the LM-head shape) run on the 128-token x
    256-row kernel: ragged token and weight-row edges included."""
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    x8, sx, w8, sw = _sweep_inputs(M, N, K, seed=6)
    want = orc.gemm_fp8_block(x8, sx, w8, sw)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    d_y = DeviceBuffer(M * N * 2)
    host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K)
    assert_close_bf16(d_y.to_array(np.uint16, (M, N)), want, atol=G_ATOL, rtol=G_RTOL, what=f"M={M} N={N} K={K}")
    # a row pitch that rules out 16-byte stores
    ldy = N + 3
    d_y2 = DeviceBuffer(M * ldy * 2)
    d_y2.zero()
    host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y2.ptr, M, N, K, ldy=ldy)
    got = d_y2.to_array(np.uint16, (M, ldy))
    assert np.array_equal(got[:, :N], d_y.to_array(np.uint16, (M, N)))
    assert not got[:, N:].any()


def test_gemm_prefill_sized_power_of_two_scales_exact(gpu):
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    rng = np.random.default_rng(4)
    M, N, K = 640, 384, 320
    x8 = orc.e4m3_encode(rng.integers(-3, 4, size=(M, K)).astype(np.float32))
    w8 = orc.e4m3_encode(rng.integers(-3, 4, size=(N, K)).astype(np.float32))
    sx = (2.0 ** rng.integers(-2, 3, size=(5, 3))).astype(np.float32)
    sw = (2.0 ** rng.integers(-2, 3, size=(3, 3))).astype(np.float32)
    want = orc.gemm_fp8_block(x8, sx, w8, sw)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    d_y = DeviceBuffer(M * N * 2)
    host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, d_y.ptr, M, N, K)
    assert np.array_equal(d_y.to_array(np.uint16, (M, N)), want)


def test_weight_tiling_layout_bit_exact(gpu):
    """eb_weight_tile_fp8 against a numpy restatement: [groups][N][K] -> [groups][ceil(N/128)][ceil(K/128)][128][128],
    zero padded, ragged N and K."""
    import eidola_b200.host as host
    G, N, K = 3, 200, 2880
    w = np.random.default_rng(7).integers(0, 256, size=(G, N, K)).astype(np.uint8)
    NB, KB = (N + 127) // 128, (K + 127) // 128
    pad = np.zeros((G, NB * 128, KB * 128), np.uint8)
    pad[:, :N, :K] = w
    want = pad.reshape(G, NB, 128, KB, 128).transpose(0, 1, 3, 2, 4)
    d_w = _dev(w)
    tiled = host.weight_tile_fp8(d_w.ptr, G, N, K)
    assert tiled.nbytes == want.size
    assert np.array_equal(tiled.to_array(np.uint8, want.shape), want)


@pytest.mark.parametrize("M,N,K", [(8, 5120, 2880), (256, 2880, 4096), (300, 65536, 256), (1024, 2880, 2880), (513, 200, 4096)])
def test_gemm_dense_tiled_weights_equal_row_major(gpu, M, N, K):
    """The same GEMM on weights stored as 16 KiB tiles: every kernel (decode tiles, split K, persistent, the 128-token x
    256-row kernel, ragged N) must give the row-major result bit for bit -- only the addresses of the loads differ."""
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    x8, sx, w8, sw = _sweep_inputs(M, N, K, seed=8)
    d = [_dev(a) for a in (x8, sx, w8, sw)]
    tiled = host.weight_tile_fp8(d[2].ptr, 1, N, K)
    d_work = DeviceBuffer(host.gemm_workspace(M, N, 1))
    for splits, tn in ((0, 0), (1, 0), (1, 16)) if M <= 512 else ((0, 0),):
        ya, yb = DeviceBuffer(M * N * 2), DeviceBuffer(M * N * 2)
        host.gemm_fp8(d[0].ptr, d[1].ptr, d[2].ptr, d[3].ptr, ya.ptr, M, N, K, work=d_work, splits=splits, tile_tokens=tn)
        host.gemm_fp8(d[0].ptr, d[1].ptr, tiled.ptr, d[3].ptr, yb.ptr, M, N, K, work=d_work, splits=splits, tile_tokens=tn,
                      w_tiled=True)
        assert np.array_equal(ya.to_array(np.uint16, (M, N)), yb.to_array(np.uint16, (M, N))), (splits, tn)


@pytest.mark.parametrize("tn", [0, 64])
def test_gemm_grouped_tiled_weights_equal_row_major(gpu, tn):
    import eidola_b200.host as host
    from eidola_b200.capi import DeviceBuffer
    G, N, K = 6, 2880, 2880  # N = 22.5 blocks: every group's last weight tile is half padding
    seg = np.array([0, 5, 5, 140, 141, 400, 437], np.int32)
    R = int(seg[-1])
    x = orc.synth_normal_bf16(5, 1, 0, R * K).reshape(R, K)
    x8, sx = orc.quant_act_block128(x, seg)
    w = [orc.synth_weight_fp8(5, 10 + g, N, K, 0, N, 0.02) for g in range(G)]
    w8, sw = np.stack([a for a, _ in w]), np.stack([b for _, b in w])
    d_x8, d_sx, d_seg, d_w8, d_sw = _dev(x8), _dev(sx), _dev(seg), _dev(w8), _dev(sw)
    tiled = host.weight_tile_fp8(d_w8.ptr, G, N, K)
    d_work = DeviceBuffer(host.gemm_workspace(R, N, G))
    ya, yb = DeviceBuffer(R * N * 2), DeviceBuffer(R * N * 2)
    host.gemm_fp8(d_x8.ptr, d_sx.ptr, d_w8.ptr, d_sw.ptr, ya.ptr, R, N, K, n_groups=G, d_seg_off=d_seg.ptr, work=d_work, tile_tokens=tn)
    host.gemm_fp8(d_x8.ptr, d_sx.ptr, tiled.ptr, d_sw.ptr, yb.ptr, R, N, K, n_groups=G, d_seg_off=d_seg.ptr, work=d_work, tile_tokens=tn,
                  w_tiled=True)
    got = yb.to_array(np.uint16, (R, N))
    assert np.array_equal(ya.to_array(np.uint16, (R, N)), got)
    assert_close_bf16(got, orc.gemm_fp8_grouped(x8, sx, seg, w8, sw), atol=1e-3, rtol=G_RTOL, what=f"grouped tiled tn={tn}")
