"""GPU: the temperature / top-p sampler (eb_sample_top_p, eb_engine_seq_sampling) against its CPU restatement, bit for
bit: the token is integer arithmetic on weights both sides compute with the same rounded fp32 operations."""
import numpy as np
import pytest

from oracle import sampler as smp
from tests.decoder_cases import tiny_config
from tests.helpers import bf16_to_f32, f32_to_bf16

pytestmark = pytest.mark.gpu


def _run(bits, ld, scales, q24s, r32s, greedy):
    from eidola_b200 import capi
    from eidola_b200.capi import DeviceBuffer, c_i32, c_i64, c_vp
    T, V = bits.shape
    padded = np.zeros((T, ld), np.uint16)
    padded[:, :V] = bits
    padded[:, V:] = 0x7F80  # +inf beyond the row: must never be read
    d_l = DeviceBuffer.from_array(padded)
    d_s, d_q, d_r = (DeviceBuffer.from_array(np.asarray(a, dt)) for a, dt in ((scales, np.float32), (q24s, np.uint32), (r32s, np.uint32)))
    d_t = DeviceBuffer.from_array(np.asarray(greedy, np.int32))
    capi.call("eb_sample_top_p", c_vp(d_l.ptr), c_i32(T), c_i64(V), c_i64(ld), c_vp(d_s.ptr), c_vp(d_q.ptr), c_vp(d_r.ptr), c_vp(d_t.ptr), None)
    return d_t.to_array(np.int32, (T,))


@pytest.mark.parametrize("V,ld", [(201088, 201088), (4096, 4096), (1000, 1003), (37, 40)])
def test_sampler_matches_its_restatement_bit_for_bit(gpu, V, ld):
    import eidola_b200 as eb
    rng = np.random.default_rng(V)
    T = 24
    x = rng.normal(0, 2.5, size=(T, V)).astype(np.float32)
    x[1, ::7] = -np.inf
    x[2, 5] = np.nan
    x[3] = -np.inf               # nothing to weigh: the row is left alone
    x[4, 3] = np.inf             # an infinite logit: left to the greedy token
    x[5] = 1.25                  # one value everywhere: the nucleus is the whole row whatever top_p says
    bits = f32_to_bf16(x)
    temps = rng.choice([0.05, 0.3, 0.7, 1.0, 1.5, 4.0], size=T)
    scales = np.array([smp.scale_of(t) for t in temps], np.float32)
    scales[6] = 0.0              # a greedy row
    q24s = np.array([smp.top_p_q24(p) for p in rng.choice([0.0, 0.1, 0.5, 0.9, 0.95, 1.0], size=T)], np.uint32)
    r32s = np.array([smp.rand32(V, t) for t in range(T)], np.uint32)
    r32s[7], r32s[8] = 0, 2**32 - 1
    greedy = np.arange(T, dtype=np.int32) % V
    want = smp.sample(bits, scales, q24s, r32s, greedy)
    got = _run(bits, ld, scales, q24s, r32s, greedy)
    assert np.array_equal(got, want), (np.flatnonzero(got != want), got, want)
    assert got[3] == greedy[3] and got[4] == greedy[4] and got[6] == greedy[6]
    assert int(eb.status_read()) == 0


def test_draws_from_the_kernel_follow_the_softmax(gpu):
    rng = np.random.default_rng(5)
    V, T = 64, 4096
    row = f32_to_bf16(rng.normal(0, 1.5, size=V).astype(np.float32))
    bits = np.tile(row, (T, 1))
    sc = smp.scale_of(0.9)
    got = _run(bits, V, np.full(T, sc, np.float32), np.full(T, smp.top_p_q24(0.92), np.uint32),
               np.array([smp.rand32(99, t) for t in range(T)], np.uint32), np.zeros(T, np.int32))
    thr, M, w, k = smp.nucleus(row, sc, smp.top_p_q24(0.92))
    p = np.where(k >= thr, w, 0).astype(np.float64)
    p /= p.sum()
    counts = np.bincount(got, minlength=V)
    assert (counts[p == 0] == 0).all()  # nothing outside the nucleus is ever drawn
    live = p > 0
    chi2 = (((counts[live] - T * p[live]) ** 2) / (T * p[live])).sum()
    assert chi2 < 2.0 * live.sum() + 20, (chi2, int(live.sum()))
    x = bf16_to_f32(row).astype(np.float64)
    soft = np.exp((x - x.max()) / 0.9)
    soft = np.where(live, soft, 0) / soft[live].sum()
    assert np.abs(p - soft).max() < 1e-5  # the integer weights are the softmax


def test_engine_sampling_is_seeded_per_sequence_and_leaves_greedy_rows_alone(gpu):
    """Three sequences decode together: one greedy, two with a temperature.  The greedy one gets the tokens it gets alone;
    the sampled ones reproduce with the same seed, whatever shares their steps, and are what the restatement draws from
    the step's logits."""
    import eidola_b200 as eb
    cfg = tiny_config()

    def run(sampling, who=(0, 1, 2), steps=6):
        eng = eb.Engine(cfg)
        eng.kv_fill_synth()
        ctx = [40, 70, 9]
        slots = {i: eng.admit(ctx[i]) for i in who}
        for i, (t, p, seed) in sampling.items():
            if i in slots:
                eng.sampling(slots[i], t, p, seed)
        toks = {i: 17 + i for i in who}
        out = {i: [] for i in who}
        checked = 0
        for _ in range(steps):
            order = list(who)
            nxt, _ = eng.step([slots[i] for i in order], [1] * len(order), [toks[i] for i in order])
            logits = eng.read_logits()
            for row, i in enumerate(order):
                if i in sampling:  # the restatement on this row's logits
                    t, p, seed = sampling[i]
                    pos = eng.seq_len(slots[i])  # the position of the token just drawn
                    want = smp.sample_row(logits[row], smp.scale_of(t), smp.top_p_q24(p), smp.rand32(seed, pos), -1)
                    assert int(nxt[row]) == want, (i, int(nxt[row]), want)
                    checked += 1
                else:
                    assert int(nxt[row]) == int(bf16_to_f32(logits[row]).argmax())
                toks[i] = int(nxt[row])
                out[i].append(int(nxt[row]))
        return out, checked

    plan = {1: (0.8, 0.95, 1234), 2: (1.5, 1.0, 77)}
    a, n_checked = run(plan)
    assert n_checked == 12
    greedy_alone, _ = run({}, who=(0,))
    # (the greedy sequence shares 128-row activation scale blocks with the others, whose tokens differ between the runs:
    # its logits move by rounding noise, its tokens only where the margin is small; the first step has identical inputs)
    assert a[0][0] == greedy_alone[0][0]
    b, _ = run(plan)
    assert a == b  # same seeds, same tokens
    c, _ = run({1: (0.8, 0.95, 4321), 2: (1.5, 1.0, 77)})
    assert c[1] != a[1]  # another seed, another continuation
    eng = eb.Engine(cfg)
    s = eng.admit(5)
    with pytest.raises(eb.EbError):
        eng.sampling(s, 1e-9, 1.0, 0)
    with pytest.raises(eb.EbError):
        eng.sampling(s + 1, 1.0, 1.0, 0)  # not a live slot
    eng.sampling(s, 0.0)  # back to greedy is always fine


def test_the_kernel_reproduces_the_committed_vectors(gpu):
    from pathlib import Path
    g = np.load(Path(__file__).with_name("golden") / "sampler.npz")
    T, V = g["bits"].shape
    got = _run(g["bits"], V, g["scales"], g["q24"], g["r32"], np.full(T, -1, np.int32))
    assert np.array_equal(got, g["tokens"])
