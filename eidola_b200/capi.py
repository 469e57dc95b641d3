"""ctypes binding of libeidola_b200.so -- the same C ABI a Rust host would bind with `extern "C"`.

Nothing here computes: every call goes to the CUDA library.  If the library has not been built
the import fails loudly; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import numpy as np

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "lib" / "libeidola_b200.so"
HEADER = PKG.parent / "include" / "eidola_b200.h"

c_i32, c_i64, c_u64, c_f32, c_vp, c_sz = C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_void_p, C.c_size_t
P = C.POINTER


class EbError(RuntimeError):
    def __init__(self, fn: str, code: int, msg: str):
        super().__init__(f"{fn} -> {code}: {msg}")
        self.code = code


class AttnItem(C.Structure):
    _fields_ = [("seq", c_i32), ("page_begin", c_i32), ("page_end", c_i32), ("part", c_i32)]


class AttnArgs(C.Structure):
    _fields_ = [
        ("d_q", c_vp), ("q_stride", c_i64), ("d_out", c_vp), ("out_stride", c_i64),
        ("d_cache", c_vp), ("num_pages", c_i32),
        ("d_block_tables", c_vp), ("bt_stride", c_i32),
        ("d_seq_slots", c_vp), ("d_q_off", c_vp), ("d_ctx_lens", c_vp),
        ("n_seqs", c_i32), ("max_q_len", c_i32),
        ("d_sinks", c_vp), ("window", c_i32),
        ("n_q", c_i32), ("n_kv", c_i32), ("head_dim", c_i32), ("page_size", c_i32),
        ("scale", c_f32),
        ("d_items", c_vp), ("n_items", c_i32),
        ("d_seq_part", c_vp), ("n_parts", c_i32),
        ("d_part_acc", c_vp), ("d_part_ml", c_vp),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("d_x8", c_vp), ("d_sx", c_vp), ("d_w8", c_vp), ("d_sw", c_vp), ("d_y", c_vp), ("ldy", c_i64),
        ("rows", c_i32), ("N", c_i32), ("K", c_i32), ("n_groups", c_i32),
        ("d_seg_off", c_vp), ("d_work", c_vp), ("tile_tokens", c_i32), ("splits", c_i32), ("tiles_ready", c_i32),
        ("work_bytes", c_sz), ("w_tiled", c_i32),
    ]


class Config(C.Structure):
    """eb_config."""
    _fields_ = [
        ("n_layers", c_i32), ("hidden", c_i32), ("n_q_heads", c_i32), ("n_kv_heads", c_i32), ("head_dim", c_i32),
        ("window", c_i32),
        ("n_experts", c_i32), ("top_k", c_i32), ("inter", c_i32), ("vocab", c_i32),
        ("page_size", c_i32), ("num_pages", c_i32), ("max_seqs", c_i32), ("max_pages_per_seq", c_i32),
        ("max_tokens", c_i32), ("max_q_len", c_i32),
        ("rope_theta", c_f32), ("rms_eps", c_f32), ("init_std", c_f32),
        ("seed", c_u64),
        ("debug", c_i32),
        ("window_ring", c_i32),
    ]


def make_config(**kw) -> "Config":
    """eb_config with the defaults of the benchmark family (head_dim 64, page 16, window 128, top-4, std 0.02)."""
    d = dict(head_dim=64, window=128, top_k=4, page_size=16, max_q_len=1, rope_theta=150000.0, rms_eps=1e-5,
             init_std=0.02, seed=0, debug=0, window_ring=0)
    d.update(kw)
    c = Config()
    for k, v in d.items():
        setattr(c, k, v)
    return c


def declared_symbols(header: Path = HEADER) -> list[str]:
    """Every function the public header declares."""
    text = header.read_text()
    return sorted(set(re.findall(r"^\s*int32_t\s+(eb_\w+)\s*\(", text, flags=re.M)))


def load_library(path: Path = LIB_PATH) -> C.CDLL:
    if not path.exists():
        raise ImportError(
            f"{path} is missing: build it with `python -m eidola_b200.build` (nvcc, sm_100a). "
            "There is no CPU fallback.")
    return C.CDLL(str(path))


_lib = load_library()


def lib() -> C.CDLL:
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(512)
    _lib.eb_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(fn: str, rc: int) -> None:
    if rc != 0:
        raise EbError(fn, rc, last_error())


def call(fn: str, *args) -> None:
    """Call an entry point and raise EbError on a non-zero status."""
    f = getattr(_lib, fn)
    f.restype = c_i32
    check(fn, f(*args))


def call_rc(fn: str, *args) -> int:
    f = getattr(_lib, fn)
    f.restype = c_i32
    return int(f(*args))


def ptr(a: np.ndarray):
    return a.ctypes.data_as(c_vp)


class DeviceBuffer:
    """A caller-owned device allocation (eb_malloc / eb_free)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        p = c_vp()
        call("eb_malloc", C.byref(p), c_sz(max(self.nbytes, 1)))
        self.ptr = p.value

    @classmethod
    def from_array(cls, a: np.ndarray, stream=None) -> "DeviceBuffer":
        a = np.ascontiguousarray(a)
        b = cls(a.nbytes)
        if a.nbytes:
            call("eb_copy_h2d", c_vp(b.ptr), ptr(a), c_sz(a.nbytes), c_vp(stream))
            call("eb_stream_sync", c_vp(stream))
        return b

    def to_array(self, dtype, shape, stream=None) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        assert out.nbytes <= self.nbytes, (out.nbytes, self.nbytes)
        if out.nbytes:
            call("eb_copy_d2h", ptr(out), c_vp(self.ptr), c_sz(out.nbytes), c_vp(stream))
            call("eb_stream_sync", c_vp(stream))
        return out

    def zero(self, stream=None) -> None:
        call("eb_memset", c_vp(self.ptr), c_i32(0), c_sz(self.nbytes), c_vp(stream))

    def free(self) -> None:
        if self.ptr:
            call("eb_free", c_vp(self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def device_count() -> int:
    n = c_i32(0)
    rc = call_rc("eb_device_count", C.byref(n))
    return int(n.value) if rc == 0 else 0


def device_info(device: int = 0) -> dict:
    sm, l2, hbm, maj, mnr = c_i32(), c_i64(), c_i64(), c_i32(), c_i32()
    call("eb_device_info", c_i32(device), C.byref(sm), C.byref(l2), C.byref(hbm), C.byref(maj), C.byref(mnr))
    return {"sm_count": sm.value, "l2_bytes": l2.value, "hbm_bytes": hbm.value, "cc": (maj.value, mnr.value)}


def mem_info() -> tuple[int, int]:
    """(free, total) bytes of the current device."""
    f, t = c_i64(0), c_i64(0)
    call("eb_device_mem_info", C.byref(f), C.byref(t))
    return int(f.value), int(t.value)


def static_status_read() -> int:
    """Status word built into the library for eb_attn_paged_sink_static calls that passed none; reading clears it."""
    s = c_i32(0)
    call("eb_attn_static_status_read", C.byref(s))
    return int(s.value)


def status_read() -> int:
    s = c_i32(0)
    call("eb_status_read", C.byref(s))
    return int(s.value)


class Timer:
    """CUDA-event timer on a given stream (eb_event_*)."""

    def __init__(self, stream=None):
        self.stream = stream
        self.e0, self.e1 = c_vp(), c_vp()
        call("eb_event_create", C.byref(self.e0))
        call("eb_event_create", C.byref(self.e1))

    def start(self):
        call("eb_event_record", self.e0, c_vp(self.stream))

    def stop(self) -> float:
        call("eb_event_record", self.e1, c_vp(self.stream))
        ms = c_f32(0)
        call("eb_event_elapsed_ms", self.e0, self.e1, C.byref(ms))
        return float(ms.value)
