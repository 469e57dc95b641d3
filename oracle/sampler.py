"""CPU restatement of the temperature / top-p sampler (test infrastructure: only tests, the smoke check and the CPU legs
of the benchmark may use it; the product path is eidola_b200/csrc/sample.cu).

Parity unpinned: the reference holds no sampler (its server forwards `temperature` and `top_p`,
crates/eidola-server/src/types.rs:24-30, to a remote engine), so there is no golden vector of the reference's to check
this against.  It restates the published nucleus-sampling rule (keep the smallest set of most probable tokens whose
mass reaches top_p, renormalise, draw) in the integer form the CUDA kernel documents, so that the two agree bit for bit:

    W_v   = trunc(2^31 * 2^t),  t = (x_v - max x) * scale  (fp32, each operation rounded; 2^t by the degree-8 Taylor
            polynomial of 2^f in Horner form on the fraction f of t; t < -32 and NaN logits weigh nothing)
    thr   = the largest bf16 value whose tail mass sum{W_v : x_v >= thr} reaches max(1, (sum W * top_p_q24) >> 24)
    token = first v in id order whose running mass over {x_v >= thr} exceeds (tail mass * rand32) >> 32
"""
import numpy as np

_COEF = [np.float32(c) for c in (1.3215486790e-6, 1.5252733804e-5, 1.5403530393e-4, 1.3333558146e-3, 9.6181291076e-3,
                                 5.5504108665e-2, 2.4022650696e-1, 6.9314718056e-1, 1.0)]  # ln2^k / k!, k = 8 .. 0
_MASK64 = (1 << 64) - 1


def rand32(seed: int, counter: int) -> int:
    """splitmix64 of (seed, counter), upper half: eb_sample_rand32."""
    z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return z >> 32


def scale_of(temperature: float) -> np.float32:
    """log2(e) / temperature as the fp32 the kernel is given."""
    return np.float32(np.float32(1.4426950408889634) / np.float32(temperature))


def top_p_q24(top_p: float) -> int:
    return int(min(max(float(top_p), 0.0), 1.0) * (1 << 24))


def keys(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> keys ascending in the value."""
    b = bits.astype(np.uint32)
    return np.where(b & 0x8000, (~b) & 0xFFFF, b | 0x8000).astype(np.uint32)


def weights(bits: np.ndarray, scale) -> np.ndarray:
    """W_v as uint64 for one row of bf16 bit patterns (uint16); None when the row has no finite maximum."""
    b = bits.astype(np.uint32)
    nan = (b & 0x7FFF) > 0x7F80
    x = (b << 16).view(np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        finite_or_inf = np.where(nan, np.float32(-np.inf), x)
        mx = np.float32(finite_or_inf.max())
        if not (mx > -np.inf) or mx == np.inf:
            return None
        t = (x - mx).astype(np.float32) * np.float32(scale)
        t = t.astype(np.float32)
        ok = (t >= np.float32(-32.0)) & ~nan
        tt = np.where(ok, t, np.float32(0.0)).astype(np.float32)
        n = np.floor(tt).astype(np.float32)
        f = (tt - n).astype(np.float32)
        p = np.full(f.shape, _COEF[0], np.float32)
        for c in _COEF[1:]:
            p = (p * f).astype(np.float32)
            p = (p + c).astype(np.float32)
        w = np.ldexp(p.astype(np.float64), n.astype(np.int64) + 31)  # exact: p has 24 bits
    return np.where(ok, np.floor(w), 0.0).astype(np.uint64)


def nucleus(bits: np.ndarray, scale, q24: int):
    """(threshold key, nucleus mass, weights) of one row, or None."""
    w = weights(bits, scale)
    if w is None:
        return None
    k = keys(bits)
    mass = np.zeros(65536, dtype=object)
    per_key = np.bincount(k, weights=None, minlength=65536)  # counts; mass per key = count * weight of that key
    first = np.full(65536, -1, np.int64)
    order = np.argsort(k, kind="stable")
    ks = k[order]
    starts = np.flatnonzero(np.r_[True, ks[1:] != ks[:-1]])
    for s in starts:
        first[ks[s]] = order[s]
    Z = 0
    for key in np.flatnonzero(per_key):
        m = int(per_key[key]) * int(w[first[key]])
        mass[key] = m
        Z += m
    target = Z if q24 >= (1 << 24) else (Z * q24) >> 24
    target = max(1, target)
    cum = 0
    thr = 0
    for key in np.flatnonzero(per_key)[::-1]:
        cum += mass[key]
        thr = int(key)
        if cum >= target:
            break
    return thr, cum, w, k


def sample_row(bits: np.ndarray, scale, q24: int, r32: int, greedy_token: int) -> int:
    """The token eb_sample_top_p writes for one row (greedy_token where it leaves the row alone)."""
    if not (np.float32(scale) > 0):
        return greedy_token
    nu = nucleus(np.asarray(bits, np.uint16), scale, q24)
    if nu is None:
        return greedy_token
    return draw(nu, r32)


def draw(nu, r32: int) -> int:
    """The token for one 32-bit random number, given nucleus()'s result for the row."""
    thr, M, w, k = nu
    want = (M * r32) >> 32
    inc = np.where(k >= thr, w, np.uint64(0)).astype(np.uint64)
    run = np.cumsum(inc, dtype=np.uint64)  # M < 2^49: no wrap
    return int(np.searchsorted(run, np.uint64(want), side="right"))


def sample(logits_bits: np.ndarray, scales, q24s, r32s, greedy) -> np.ndarray:
    """All rows: logits_bits [T][V] uint16."""
    return np.array([sample_row(logits_bits[t], scales[t], int(q24s[t]), int(r32s[t]), int(greedy[t]))
                     for t in range(logits_bits.shape[0])], np.int32)
