"""Generate tests/golden/sampler.npz from the sampler's CPU restatement (run from the repository root):

    python tests/golden/make_sampler_golden.py

The reference project holds no sampler and so no golden vectors for one; these pin the restatement itself (and, through
tests/test_gpu_sampler.py, the kernel): a later change that alters a weight, a threshold or a drawn token of these rows
fails tests/test_sampler_oracle.py.
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle import sampler as smp  # noqa: E402
from tests.helpers import f32_to_bf16  # noqa: E402


def rows():
    rng = np.random.default_rng(20261125)
    T, V = 32, 1536
    x = rng.normal(0, 3.0, size=(T, V)).astype(np.float32)
    x[0] += np.where(np.arange(V) == 77, 25.0, 0.0)   # one dominant token
    x[1, ::5] = -np.inf
    x[2, 9] = np.nan
    x[3] = 0.5                                          # every token alike
    bits = f32_to_bf16(x)
    temps = rng.choice([0.1, 0.5, 0.8, 1.0, 1.3, 2.0], size=T)
    top_ps = rng.choice([0.0, 0.2, 0.5, 0.9, 0.99, 1.0], size=T)
    scales = np.array([smp.scale_of(t) for t in temps], np.float32)
    q24 = np.array([smp.top_p_q24(p) for p in top_ps], np.uint32)
    r32 = np.array([smp.rand32(7, t) for t in range(T)], np.uint32)
    return bits, scales, q24, r32


def main():
    bits, scales, q24, r32 = rows()
    T = bits.shape[0]
    tokens = smp.sample(bits, scales, q24, r32, np.full(T, -1, np.int32))
    thr = np.zeros(T, np.int64)
    mass = np.zeros(T, np.uint64)
    for t in range(T):
        nu = smp.nucleus(bits[t], scales[t], int(q24[t]))
        thr[t], mass[t] = nu[0], nu[1]
    out = Path(__file__).with_name("sampler.npz")
    np.savez_compressed(out, bits=bits, scales=scales, q24=q24, r32=r32, tokens=tokens, threshold_key=thr, nucleus_mass=mass)
    print("wrote", out, out.stat().st_size, "bytes; tokens", tokens.tolist())


if __name__ == "__main__":
    main()
