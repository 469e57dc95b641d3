"""A minimal GGUF (version 3) writer for the loader tests: little endian, F32 / F16 / BF16 tensors and the block formats
Q4_0, Q8_0 and MXFP4 (pass `Blocked(kind, float32 array)`), 32-byte alignment.

Layout per the container's published specification: magic, version, tensor count, metadata count, metadata entries,
tensor table (name, number of dimensions, extents innermost first, type, offset from the start of the data section),
padding, data."""
from __future__ import annotations

import struct

import numpy as np

GGML_F32, GGML_F16, GGML_BF16 = 0, 1, 30
GGML_Q4_0, GGML_Q8_0, GGML_MXFP4 = 2, 8, 39
ALIGN = 32
E2M1 = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


class Blocked:
    """A float32 array stored in a block format: 32 consecutive elements of a row share a scale.  `raw` is the bytes
    of the file, `values` what a reader must get back (fp32, the array's shape).

      q8_0  : fp16 d = absmax / 127, int8 round(x / d)
      q4_0  : fp16 d = (the element of largest magnitude) / -8, 4-bit codes min(15, int(x / d + 8.5)); element i in the
              low nibble of byte i, element i + 16 in the high nibble
      mxfp4 : one byte e (scale 2^(e - 127), the smallest power of two with absmax / scale <= 6), 4-bit codes sign | index
              of the nearest of 0, 0.5, 1, 1.5, 2, 3, 4, 6; nibbles as in q4_0
    """

    def __init__(self, kind: str, a: np.ndarray):
        a = np.ascontiguousarray(a, np.float32)
        assert a.shape[-1] % 32 == 0
        self.kind, self.shape = kind, a.shape
        self.ggml_type = {"q4_0": GGML_Q4_0, "q8_0": GGML_Q8_0, "mxfp4": GGML_MXFP4}[kind]
        x = a.reshape(-1, 32)
        nb = x.shape[0]
        if kind == "q8_0":
            d = (np.abs(x).max(axis=1) / 127.0).astype(np.float16)
            df = d.astype(np.float32)
            q = np.where(df[:, None] > 0, np.rint(x / np.where(df > 0, df, 1)[:, None]), 0).clip(-127, 127).astype(np.int8)
            raw = np.empty((nb, 34), np.uint8)
            raw[:, :2] = d.view(np.uint8).reshape(nb, 2)
            raw[:, 2:] = q.view(np.uint8)
            vals = df[:, None] * q.astype(np.float32)
        elif kind == "q4_0":
            i = np.abs(x).argmax(axis=1)
            d = (x[np.arange(nb), i] / -8.0).astype(np.float16)
            df = d.astype(np.float32)
            q = np.where(df[:, None] != 0, np.floor(x / np.where(df != 0, df, 1)[:, None] + 8.5), 8).clip(0, 15).astype(np.uint8)
            raw = np.empty((nb, 18), np.uint8)
            raw[:, :2] = d.view(np.uint8).reshape(nb, 2)
            raw[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
            vals = df[:, None] * (q.astype(np.float32) - 8.0)
        else:
            amax = np.abs(x).max(axis=1)
            e = np.where(amax > 0, np.ceil(np.log2(np.where(amax > 0, amax, 1) / 6.0)), -127).astype(np.int32).clip(-127, 127)
            scale = np.ldexp(np.float32(1), e).astype(np.float32)
            idx = np.abs(np.abs(x / scale[:, None])[:, :, None] - E2M1[None, None, :]).argmin(axis=2).astype(np.uint8)
            q = idx | ((x < 0).astype(np.uint8) << 3)
            raw = np.empty((nb, 17), np.uint8)
            raw[:, 0] = (e + 127).astype(np.uint8)
            raw[:, 1:] = q[:, :16] | (q[:, 16:] << 4)
            vals = scale[:, None] * np.where(q & 8, -E2M1[q & 7], E2M1[q & 7])
        self.raw = raw.tobytes()
        self.values = vals.astype(np.float32).reshape(a.shape)


def _string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> numpy array (float32 -> F32, float16 -> F16, uint16 -> BF16 bit patterns) or Blocked, C order."""
    md = {"general.architecture": "eidola-b200-decoder", "general.alignment": np.uint32(ALIGN)}
    md.update(metadata or {})
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(md))
    for k, v in md.items():
        head += _string(k)
        if isinstance(v, str):
            head += struct.pack("<I", 8) + _string(v)
        elif isinstance(v, np.uint32):
            head += struct.pack("<II", 4, int(v))
        elif isinstance(v, (float, np.float32)):
            head += struct.pack("<If", 6, float(v))
        elif isinstance(v, list) and all(isinstance(x, str) for x in v):     # array of strings
            head += struct.pack("<IIQ", 9, 8, len(v)) + b"".join(_string(x) for x in v)
        elif isinstance(v, list):                                            # array of int32
            head += struct.pack("<IIQ", 9, 5, len(v)) + struct.pack("<%di" % len(v), *[int(x) for x in v])
        else:
            raise TypeError(k)
    table, blobs, off = b"", [], 0
    for name, a in tensors.items():
        if isinstance(a, Blocked):
            typ, shape, raw = a.ggml_type, a.shape, a.raw
        else:
            a = np.ascontiguousarray(a)
            typ = {np.dtype(np.float32): GGML_F32, np.dtype(np.float16): GGML_F16, np.dtype(np.uint16): GGML_BF16}[a.dtype]
            shape, raw = a.shape, a.tobytes()
        table += _string(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in reversed(shape))
        table += struct.pack("<IQ", typ, off)
        pad = (-len(raw)) % ALIGN
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    body = head + table
    body += b"\0" * ((-len(body)) % ALIGN)
    with open(path, "wb") as f:
        f.write(body)
        for b in blobs:
            f.write(b)
