"""CPU: the sampler's restatement (oracle/sampler.py) -- its random numbers against the library's host function, its
weights against exp(), and the nucleus rule on rows small enough to enumerate by hand."""
import ctypes as C

import numpy as np

from oracle import sampler as smp
from tests.helpers import f32_to_bf16


def _bits(x):
    return f32_to_bf16(np.asarray(x, np.float32))


def test_rand32_is_the_library_function():
    from eidola_b200 import capi
    f = capi.lib().eb_sample_rand32
    f.restype = C.c_uint32
    for seed, ctr in [(0, 0), (1, 0), (0, 1), (12345, 678), (2**64 - 1, 2**40), (0x9E3779B97F4A7C15, 7)]:
        assert int(f(C.c_uint64(seed), C.c_uint64(ctr))) == smp.rand32(seed, ctr)
    draws = np.array([smp.rand32(42, i) for i in range(4096)], np.float64) / 2**32
    assert abs(draws.mean() - 0.5) < 0.02 and abs(np.mean(draws < 0.25) - 0.25) < 0.03


def test_weights_are_the_softmax_numerators():
    rng = np.random.default_rng(0)
    bits = _bits(rng.normal(0, 3, size=5000))
    x = (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    for temp in (0.3, 1.0, 2.0):
        w = smp.weights(bits, smp.scale_of(temp)).astype(np.float64) / 2.0**31
        want = np.exp((x - x.max()) / temp)
        big = want > 1e-3
        assert np.abs(w[big] / want[big] - 1).max() < 2e-6  # the polynomial, the fp32 scale and the truncation together
        assert (np.abs(w[~big] - want[~big]) <= want[~big] * 1e-5 + 2.0**-31).all()  # truncated to a multiple of 2^-31
    assert smp.weights(_bits([-np.inf, -np.inf]), smp.scale_of(1.0)) is None
    w = smp.weights(np.array([0x7FC0, 0x3F80, 0xFF80], np.uint16), smp.scale_of(1.0))  # NaN, 1.0, -inf
    assert w.tolist() == [0, 2**31, 0]


def test_nucleus_rule_on_a_row_one_can_do_by_hand():
    # probabilities 1/2, 1/4, 1/8, 1/8 at temperature 1 (logits in units of ln 2)
    bits = _bits(np.array([0.0, -1.0, -2.0, -2.0]) * np.log(2.0))
    sc = smp.scale_of(1.0)
    w = smp.weights(bits, sc)
    assert abs(int(w[1]) / int(w[0]) - 0.5) < 1e-2  # bf16 logits: ln 2 is not exact
    for top_p, n_in in [(0.0, 1), (0.4, 1), (0.6, 2), (0.8, 4), (1.0, 4)]:  # the tie at the threshold comes in whole
        thr, M, _, k = smp.nucleus(bits, sc, smp.top_p_q24(top_p))
        assert int((k >= thr).sum()) == n_in, (top_p, thr)
    # the draw walks the nucleus in id order
    thr, M, w, k = smp.nucleus(bits, sc, smp.top_p_q24(1.0))
    edges = np.cumsum([int(v) for v in w])
    for r32 in (0, 2**31, 2**32 - 1, int(edges[0] / M * 2**32) + 8, int(edges[1] / M * 2**32) + 8):
        want = (M * r32) >> 32
        assert smp.sample_row(bits, sc, smp.top_p_q24(1.0), r32, 0) == int(np.searchsorted(edges, want, side="right"))
    assert smp.sample_row(bits, np.float32(0), 0, 123, 3) == 3  # a greedy row is left alone
    assert smp.sample_row(bits, sc, smp.top_p_q24(0.0), 2**32 - 1, 3) == 0  # top_p 0: the most probable token


def test_draws_follow_the_distribution():
    rng = np.random.default_rng(1)
    bits = _bits(rng.normal(0, 1.5, size=50))
    sc = smp.scale_of(0.8)
    thr, M, w, k = smp.nucleus(bits, sc, smp.top_p_q24(0.9))
    p = np.where(k >= thr, w, 0).astype(np.float64)
    p /= p.sum()
    n = 20000
    counts = np.bincount([smp.draw((thr, M, w, k), smp.rand32(7, i)) for i in range(n)], minlength=50)
    assert (counts[p == 0] == 0).all()
    live = p > 0
    chi2 = (((counts[live] - n * p[live]) ** 2) / (n * p[live])).sum()
    assert chi2 < 2.0 * live.sum() + 20, (chi2, live.sum())


def test_the_restatement_reproduces_its_committed_vectors():
    """tests/golden/sampler.npz (made by tests/golden/make_sampler_golden.py): inputs, thresholds, masses and tokens."""
    from pathlib import Path
    g = np.load(Path(__file__).with_name("golden") / "sampler.npz")
    T = g["bits"].shape[0]
    got = smp.sample(g["bits"], g["scales"], g["q24"], g["r32"], np.full(T, -1, np.int32))
    assert np.array_equal(got, g["tokens"])
    for t in range(T):
        thr, mass, _, _ = smp.nucleus(g["bits"][t], g["scales"][t], int(g["q24"][t]))
        assert thr == int(g["threshold_key"][t]) and mass == int(g["nucleus_mass"][t])
    assert g["tokens"][0] == 77  # the dominant token of row 0
