"""CPU: the GGUF reader the checkpoint loader uses (eb_gguf_read_f32, host only) on every tensor type it reads --
F32, F16, BF16 and the block formats Q4_0, Q8_0, MXFP4 -- at ranges that start and end inside blocks."""
import ctypes as C

import numpy as np
import pytest

from tests.gguf_writer import GGML_BF16, GGML_F16, GGML_F32, GGML_MXFP4, GGML_Q4_0, GGML_Q8_0, Blocked, write_gguf


def _read(path, name, e0, n):
    from eidola_b200 import capi
    out = np.empty(max(n, 1), np.float32)
    typ, total = C.c_int32(0), C.c_int64(0)
    capi.call("eb_gguf_read_f32", str(path).encode(), name.encode(), C.c_int64(e0), C.c_int64(n), capi.ptr(out), C.byref(typ), C.byref(total))
    return out[:n], int(typ.value), int(total.value)


def test_every_tensor_type_reads_back_what_was_written(tmp_path):
    from eidola_b200.capi import EbError
    rng = np.random.default_rng(2)
    a = rng.normal(0, 0.7, size=(6, 96)).astype(np.float32)
    a[2, 32:64] = 0.0          # a block of zeros
    a[3, 5] = 40.0             # one large element decides its block's scale
    tensors = {"f32": a, "f16": a.astype(np.float16), "bf16": (a.view(np.uint32) >> 16).astype(np.uint16),
               "q8": Blocked("q8_0", a), "q4": Blocked("q4_0", a), "mx": Blocked("mxfp4", a),
               "mx3d": Blocked("mxfp4", rng.normal(0, 2.0, size=(3, 4, 64)).astype(np.float32))}
    path = tmp_path / "types.gguf"
    write_gguf(path, tensors)
    want = {"f32": (a, GGML_F32), "f16": (a.astype(np.float16).astype(np.float32), GGML_F16),
            "bf16": (((a.view(np.uint32) >> 16) << 16).view(np.float32), GGML_BF16),
            "q8": (tensors["q8"].values, GGML_Q8_0), "q4": (tensors["q4"].values, GGML_Q4_0),
            "mx": (tensors["mx"].values, GGML_MXFP4), "mx3d": (tensors["mx3d"].values, GGML_MXFP4)}
    for name, (vals, typ) in want.items():
        flat = vals.reshape(-1)
        for e0, n in [(0, flat.size), (0, 1), (31, 2), (33, 95), (flat.size - 7, 7), (100, 0)]:
            got, t, total = _read(path, name, e0, n)
            assert t == typ and total == flat.size
            assert np.array_equal(got, flat[e0:e0 + n]), (name, e0, n)
    # the block formats are what their definitions say, not only what the writer wrote: spot values by hand
    q8 = tensors["q8"]
    d = np.frombuffer(q8.raw[:2], np.float16)[0].astype(np.float32)
    assert _read(path, "q8", 0, 1)[0][0] == d * np.frombuffer(q8.raw[2:3], np.int8)[0]
    mx = tensors["mx"]
    e, b = mx.raw[0], mx.raw[1]
    table = [0, 0.5, 1, 1.5, 2, 3, 4, 6]
    v0 = (-1 if b & 8 else 1) * table[b & 7] * 2.0 ** (e - 127)
    v16 = (-1 if (b >> 4) & 8 else 1) * table[(b >> 4) & 7] * 2.0 ** (e - 127)
    got = _read(path, "mx", 0, 32)[0]
    assert got[0] == np.float32(v0) and got[16] == np.float32(v16)
    # quantisation noise of the formats themselves, as a sanity check of the writer
    assert np.abs(tensors["q8"].values - a).max() <= np.abs(a).max() / 127
    assert np.abs(tensors["mx"].values - a)[a != 40.0].max() <= 0.26 * np.abs(a).max()
    with pytest.raises(EbError):
        _read(path, "nope", 0, 1)
    with pytest.raises(EbError):
        _read(path, "q8", 570, 10)  # past the end
