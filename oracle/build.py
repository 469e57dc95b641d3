"""Build the CPU oracle (test infrastructure) into oracle/liboracle.so with g++.

There is no reference implementation of this path to compile (the reference project
delegates inference to a third-party process), so there is no oracle/_ref here.
Everything is compiled with -ffp-contract=off: a*b+c rounds twice unless the source says
fmaf(), so the arithmetic does not depend on the compiler's contraction choices and matches
the device intrinsics operation for operation.  -march=x86-64-v3 (AVX2+FMA) keeps the library runnable on a
host other than the one that built it.
"""
from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"
COMMON = ["-O3", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-fPIC", "-std=c++17", "-Wall"]


def build(force: bool = False) -> Path:
    srcs = {"synth.cpp": [], "oracle.cpp": [], "model.cpp": []}
    deps = [HERE / s for s in srcs if (HERE / s).exists()] + sorted((HERE.parent / "include").glob("*.h"))
    if not force and LIB_PATH.exists() and all(d.stat().st_mtime <= LIB_PATH.stat().st_mtime for d in deps):
        return LIB_PATH
    objs = []
    for s, extra in srcs.items():
        if not (HERE / s).exists():
            continue
        obj = HERE / (s + ".o")
        cmd = ["g++", *COMMON, *extra, "-c", str(HERE / s), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed on {s}:\n{r.stderr}")
        objs.append(str(obj))
    r = subprocess.run(["g++", "-shared", "-fopenmp", "-o", str(LIB_PATH), *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"oracle link failed:\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
