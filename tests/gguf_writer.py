"""A minimal GGUF (version 3) writer for the loader tests: little endian, F32 / BF16 tensors, 32-byte alignment.

Layout per the container's published specification: magic, version, tensor count, metadata count, metadata entries,
tensor table (name, number of dimensions, extents innermost first, type, offset from the start of the data section),
padding, data."""
from __future__ import annotations

import struct

import numpy as np

GGML_F32, GGML_F16, GGML_BF16 = 0, 1, 30
ALIGN = 32


def _string(s: str) -> bytes:
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def write_gguf(path, tensors: dict, metadata: dict | None = None) -> None:
    """tensors: name -> numpy array (float32 -> F32, float16 -> F16, uint16 -> BF16 bit patterns), C order."""
    md = {"general.architecture": "eidola-b200-decoder", "general.alignment": np.uint32(ALIGN)}
    md.update(metadata or {})
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(md))
    for k, v in md.items():
        head += _string(k)
        if isinstance(v, str):
            head += struct.pack("<I", 8) + _string(v)
        elif isinstance(v, np.uint32):
            head += struct.pack("<II", 4, int(v))
        else:
            raise TypeError(k)
    table, blobs, off = b"", [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a)
        typ = {np.dtype(np.float32): GGML_F32, np.dtype(np.float16): GGML_F16, np.dtype(np.uint16): GGML_BF16}[a.dtype]
        table += _string(name) + struct.pack("<I", a.ndim) + b"".join(struct.pack("<Q", d) for d in reversed(a.shape))
        table += struct.pack("<IQ", typ, off)
        raw = a.tobytes()
        pad = (-len(raw)) % ALIGN
        blobs.append(raw + b"\0" * pad)
        off += len(raw) + pad
    body = head + table
    body += b"\0" * ((-len(body)) % ALIGN)
    with open(path, "wb") as f:
        f.write(body)
        for b in blobs:
            f.write(b)
