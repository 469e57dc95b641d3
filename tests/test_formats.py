"""Known-answer tests of the number formats and the seeded generators (CPU; oracle side).

The reference project pins integer contracts with small known-answer fixtures
(crates/eidola-common/src/lib.rs:669-707); these follow that style for the formats every kernel shares.
"""
import numpy as np

from oracle import binding as orc


def test_e4m3_all_codes_round_trip():
    codes = np.arange(256, dtype=np.uint8)
    vals = orc.e4m3_decode(codes)
    nan = np.isnan(vals)
    assert list(np.nonzero(nan)[0]) == [0x7F, 0xFF]
    back = orc.e4m3_encode(vals[~nan])
    want = codes[~nan].copy()
    want[want == 0x80] = 0x80  # -0 stays -0
    assert np.array_equal(back, want)


def test_e4m3_known_values():
    x = np.array([0.0, 1.0, -1.0, 448.0, 449.0, 463.9, 464.0, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -9,
                  2.5 * 2.0 ** -9, 0.0625 + 0.00390625, 1.0625, 1.1875, 17.0, 19.0], np.float32)
    want = [0x00, 0x38, 0xB8, 0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE, 0x01, 0x00, 0x02, 0x02,
            # 0.06640625 = 1.0625 * 2^-4 -> tie between 1.0 and 1.125 (x2^-4) -> even mantissa 000
            0x18,
            0x38,  # 1.0625: tie between 1.0 (000) and 1.125 (001) -> even
            0x3A,  # 1.1875: tie between 1.125 (001) and 1.25 (010) -> even = 1.25
            0x58,  # 17 -> tie between 16 (000) and 18 (001) -> 16
            0x5A,  # 19 -> tie between 18 (001) and 20 (010) -> 20
            ]
    assert list(orc.e4m3_encode(x)) == want


def test_e4m3_matches_exhaustive_nearest():
    """Against a brute-force nearest-value search with ties to the even code."""
    codes = np.arange(0, 0x7F, dtype=np.uint8)
    grid = orc.e4m3_decode(codes).astype(np.float64)
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 100, 4000), rng.uniform(-0.02, 0.02, 4000),
                        (grid[:-1] + grid[1:]) / 2]).astype(np.float32)
    got = orc.e4m3_encode(x)
    ax = np.abs(x.astype(np.float64))
    d = np.abs(ax[:, None] - grid[None, :])
    best = d.min(axis=1)
    for i in range(len(x)):
        cands = np.nonzero(d[i] == best[i])[0]
        c = cands[0] if len(cands) == 1 else [k for k in cands if k % 2 == 0][0]
        if ax[i] >= 464:
            c = 0x7E
        want = int(c) | (0x80 if np.signbit(x[i]) else 0)
        assert int(got[i]) == want, (x[i], hex(int(got[i])), hex(want))


def test_bf16_rne():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.3895314e38], np.float32)
    # 1.00390625 = 1 + 2^-8: tie -> even (1.0); 1.01171875 = 1 + 3*2^-8: tie -> 1 + 2^-6
    assert list(orc.bf16_encode(x)) == [0x3F80, 0x3F80, 0x3F82, 0xC020, 0x7F7F]
    assert np.array_equal(orc.bf16_decode(orc.bf16_encode(x[:1])), x[:1])


def test_synth_is_a_pure_function_and_looks_normal():
    a = orc.synth_normal_f32(7, 3, 0, 200000)
    b = orc.synth_normal_f32(7, 3, 100000, 100000)
    assert np.array_equal(a[100000:], b)
    assert abs(a.mean()) < 0.01 and abs(a.std() - 1.0) < 0.01
    assert abs((np.abs(a) > 1.959964).mean() - 0.05) < 0.004
    assert a.max() > 4.0 and a.min() < -4.0
    u = orc.synth_uniform_f32(7, 4, 0, 100000, 0.5, 2.0)
    assert u.min() >= 0.5 and u.max() < 2.0 and abs(u.mean() - 1.25) < 0.01
    assert not np.array_equal(orc.synth_normal_f32(8, 3, 0, 16), a[:16])


def test_weight_quantiser_blocks():
    codes, scales = orc.synth_weight_fp8(1, 9, 200, 192, 0, 200, 0.02)
    assert codes.shape == (200, 192) and scales.shape == (2, 2)
    w = orc.synth_normal_f32(1, 9, 0, 200 * 192, 0.02).reshape(200, 192)
    for br in range(2):
        for bc in range(2):
            blk = w[br * 128:(br + 1) * 128, bc * 128:(bc + 1) * 128]
            assert scales[br, bc] == np.float32(np.abs(blk).max()) / np.float32(448.0)
            deq = orc.e4m3_decode(codes[br * 128:(br + 1) * 128, bc * 128:(bc + 1) * 128]) * scales[br, bc]
            assert np.abs(deq - blk).max() <= np.abs(blk).max() / 16 + 1e-9
    # a band regenerates the same codes as the full tensor
    c2, s2 = orc.synth_weight_fp8(1, 9, 200, 192, 128, 72, 0.02)
    assert np.array_equal(c2, codes[128:]) and np.array_equal(s2, scales[1:])


def test_act_quantiser_segments():
    x = orc.synth_normal_bf16(2, 5, 0, 300 * 256).reshape(300, 256)
    seg = [0, 10, 10, 270, 300]  # blocks: [0,10) | - | [10,138) [138,266) [266,270) | [270,300)
    codes, scales = orc.quant_act_block128(x, seg)
    assert scales.shape == (5, 2)
    xf = orc.bf16_decode(x)
    bounds = [(0, 10), (10, 138), (138, 266), (266, 270), (270, 300)]
    for b, (r0, r1) in enumerate(bounds):
        for bc in range(2):
            blk = xf[r0:r1, bc * 128:(bc + 1) * 128]
            s = np.float32(np.abs(blk).max()) / np.float32(448.0)
            assert scales[b, bc] == s
            assert np.array_equal(codes[r0:r1, bc * 128:(bc + 1) * 128], orc.e4m3_encode(blk / s))
