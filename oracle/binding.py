"""ctypes binding of oracle/liboracle.so (TEST INFRASTRUCTURE: the CPU checker, never the product path).

numpy conventions: bf16 tensors are uint16 arrays of bit patterns, e4m3 tensors are uint8 arrays.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "liboracle.so"

c_i32, c_i64, c_u64, c_f32, c_f64, c_vp = C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_double, C.c_void_p


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        from . import build as _b  # type: ignore
        _b.build()
    return C.CDLL(str(LIB_PATH))


_lib = _load()


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(c_vp)


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.int32))


def _void(name, *args):
    f = getattr(_lib, name)
    f.restype = None
    f(*args)


def set_threads(n: int) -> int:
    """Use n OpenMP threads (0 = leave as is); returns the number in effect."""
    _lib.orc_set_threads.restype = C.c_int
    return int(_lib.orc_set_threads(C.c_int(n)))


def set_threads_pinned(n: int) -> int:
    """Use n OpenMP threads and pin each worker (not the calling thread) to one allowed CPU; returns the number in effect."""
    _lib.orc_set_threads_pinned.restype = C.c_int
    return int(_lib.orc_set_threads_pinned(C.c_int(n)))


# ---- formats / synthetic tensors

def synth_normal_f32(seed, stream, idx0, n, scale=1.0) -> np.ndarray:
    out = np.empty(n, np.float32)
    _void("orc_synth_normal_f32", c_u64(seed), c_u64(stream), c_u64(idx0), c_i64(n), c_f32(scale), _p(out))
    return out


def synth_normal_bf16(seed, stream, idx0, n, scale=1.0) -> np.ndarray:
    out = np.empty(n, np.uint16)
    _void("orc_synth_normal_bf16", c_u64(seed), c_u64(stream), c_u64(idx0), c_i64(n), c_f32(scale), _p(out))
    return out


def synth_normal_e4m3(seed, stream, idx0, n, scale=1.0) -> np.ndarray:
    out = np.empty(n, np.uint8)
    _void("orc_synth_normal_e4m3", c_u64(seed), c_u64(stream), c_u64(idx0), c_i64(n), c_f32(scale), _p(out))
    return out


def synth_uniform_f32(seed, stream, idx0, n, lo, hi) -> np.ndarray:
    out = np.empty(n, np.float32)
    _void("orc_synth_uniform_f32", c_u64(seed), c_u64(stream), c_u64(idx0), c_i64(n), c_f32(lo), c_f32(hi), _p(out))
    return out


def synth_weight_fp8(seed, stream, rows_total, cols, row0, nrows, std):
    codes = np.empty((nrows, cols), np.uint8)
    scales = np.empty(((nrows + 127) // 128, (cols + 127) // 128), np.float32)
    _void("orc_synth_weight_fp8", c_u64(seed), c_u64(stream), c_i64(rows_total), c_i64(cols), c_i64(row0),
          c_i64(nrows), c_f32(std), _p(codes), _p(scales))
    return codes, scales


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    q = np.empty(x.shape, np.uint8)
    _void("orc_e4m3_encode", _p(x), _p(q), c_i64(x.size))
    return q


def e4m3_decode(q: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, np.uint8)
    x = np.empty(q.shape, np.float32)
    _void("orc_e4m3_decode", _p(q), _p(x), c_i64(q.size))
    return x


def bf16_encode(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    h = np.empty(x.shape, np.uint16)
    _void("orc_bf16_encode", _p(x), _p(h), c_i64(x.size))
    return h


def bf16_decode(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16)
    return (h.astype(np.uint32) << 16).view(np.float32)


def quant_act_block128(x_bf16: np.ndarray, seg_off=None):
    x = np.ascontiguousarray(x_bf16, np.uint16)
    rows, cols = x.shape
    seg = _i32([0, rows] if seg_off is None else seg_off)
    lens = np.diff(seg)
    n_blk = int(((lens + 127) // 128).sum())
    codes = np.empty((rows, cols), np.uint8)
    scales = np.empty((max(n_blk, 1), (cols + 127) // 128), np.float32)
    _void("orc_quant_act_block128", _p(x), c_i64(cols), _p(seg), c_i32(len(seg) - 1), _p(codes), _p(scales))
    return codes, scales[:n_blk]


# ---- GEMM

def gemm_fp8_block(x8, sx, w8, sw) -> np.ndarray:
    M, K = x8.shape
    N = w8.shape[0]
    y = np.empty((M, N), np.uint16)
    _void("orc_gemm_fp8_block", _p(np.ascontiguousarray(x8)), _p(np.ascontiguousarray(sx, np.float32)),
          _p(np.ascontiguousarray(w8)), _p(np.ascontiguousarray(sw, np.float32)), c_i64(M), c_i64(N), c_i64(K), _p(y))
    return y


def gemm_fp8_grouped(x8, sx, seg_off, w8, sw) -> np.ndarray:
    R, K = x8.shape
    G, N = w8.shape[0], w8.shape[1]
    y = np.zeros((R, N), np.uint16)
    seg = _i32(seg_off)
    _void("orc_gemm_fp8_grouped", _p(np.ascontiguousarray(x8)), _p(np.ascontiguousarray(sx, np.float32)), _p(seg),
          c_i32(G), _p(np.ascontiguousarray(w8)), _p(np.ascontiguousarray(sw, np.float32)), c_i64(N), c_i64(K), _p(y))
    return y


# ---- KV cache / attention

def kv_append(cache, n_kv, head_dim, page_size, k_new, v_new, row_stride, block_tables, tok_slot, positions) -> None:
    bt = _i32(block_tables)
    _void("orc_kv_append", _p(cache), c_i32(n_kv), c_i32(head_dim), c_i32(page_size), k_new.ctypes.data_as(c_vp),
          v_new.ctypes.data_as(c_vp), c_i64(row_stride), _p(bt), c_i32(bt.shape[1]), _p(_i32(tok_slot)),
          _p(_i32(positions)), c_i32(len(positions)))


def attn_paged_sink(q, cache, block_tables, seq_slots, q_off, ctx_lens, sinks, window, n_q, n_kv, head_dim=64,
                    page_size=16, scale=0.125) -> np.ndarray:
    """q: [T][n_q*head_dim] uint16 (contiguous).  Returns out of the same shape."""
    q = np.ascontiguousarray(q, np.uint16)
    T = q.shape[0]
    out = np.zeros((T, n_q * head_dim), np.uint16)
    bt = _i32(block_tables)
    _void("orc_attn_paged_sink", _p(q), c_i64(n_q * head_dim), _p(cache), _p(bt), c_i32(bt.shape[1]),
          _p(_i32(seq_slots)), _p(_i32(q_off)), _p(_i32(ctx_lens)), c_i32(len(ctx_lens)),
          _p(np.ascontiguousarray(sinks, np.float32)), c_i32(window), c_i32(n_q), c_i32(n_kv), c_i32(head_dim),
          c_i32(page_size), c_f32(scale), _p(out), c_i64(n_q * head_dim))
    return out


# ---- glue

def rmsnorm(x, g, eps) -> np.ndarray:
    x = np.ascontiguousarray(x, np.uint16)
    T, H = x.shape
    y = np.empty_like(x)
    _void("orc_rmsnorm", _p(x), _p(np.ascontiguousarray(g, np.float32)), c_i64(T), c_i64(H), c_f32(eps), _p(y))
    return y


def rope_table(max_pos, head_dim, theta):
    c = np.empty((max_pos, head_dim // 2), np.float32)
    s = np.empty((max_pos, head_dim // 2), np.float32)
    _void("orc_rope_table", c_i32(max_pos), c_i32(head_dim), c_f64(theta), _p(c), _p(s))
    return c, s


def rope_inplace(x, col0, n_heads, head_dim, positions, cos_t, sin_t) -> None:
    """Rotate heads stored at columns [col0, col0 + n_heads*head_dim) of the row-major uint16 matrix x."""
    assert x.flags["C_CONTIGUOUS"] and x.dtype == np.uint16
    base = x.ctypes.data + 2 * col0
    _void("orc_rope", c_vp(base), c_i64(x.shape[1]), c_i32(n_heads), c_i32(head_dim), _p(_i32(positions)),
          c_i32(x.shape[0]), _p(cos_t), _p(sin_t))


def residual_add(x, y) -> None:
    _void("orc_residual_add", _p(x), _p(np.ascontiguousarray(y)), c_i64(x.size))


def embed(table, tokens) -> np.ndarray:
    tokens = _i32(tokens)
    H = table.shape[1]
    x = np.empty((len(tokens), H), np.uint16)
    _void("orc_embed", _p(table), c_i64(H), _p(tokens), c_i32(len(tokens)), _p(x))
    return x


# ---- MoE

def router_topk(x, wr, top_k):
    x = np.ascontiguousarray(x, np.uint16)
    wr = np.ascontiguousarray(wr, np.uint16)
    T, H = x.shape
    E = wr.shape[0]
    idx = np.empty((T, top_k), np.int32)
    wts = np.empty((T, top_k), np.float32)
    logits = np.empty((T, E), np.float32)
    _void("orc_router_topk", _p(x), _p(wr), c_i32(T), c_i32(E), c_i32(H), c_i32(top_k), _p(idx), _p(wts), _p(logits))
    return idx, wts, logits


def moe_permute(idx, E):
    idx = _i32(idx)
    T, k = idx.shape
    seg = np.empty(E + 1, np.int32)
    perm = np.empty((T, k), np.int32)
    _void("orc_moe_permute", _p(idx), c_i32(T), c_i32(k), c_i32(E), _p(seg), _p(perm))
    return seg, perm


def moe_forward(h, idx, wts, w1, s1, w2, s2) -> np.ndarray:
    h = np.ascontiguousarray(h, np.uint16)
    T, H = h.shape
    E, I2, _ = w1.shape
    out = np.empty((T, H), np.uint16)
    _void("orc_moe_forward", _p(h), c_i32(T), c_i32(H), c_i32(I2 // 2), c_i32(E), c_i32(idx.shape[1]), _p(_i32(idx)),
          _p(np.ascontiguousarray(wts, np.float32)), _p(w1), _p(s1), _p(w2), _p(s2), _p(out))
    return out


def argmax(logits):
    logits = np.ascontiguousarray(logits, np.uint16)
    T, V = logits.shape
    tok = np.empty(T, np.int32)
    margin = np.empty(T, np.float32)
    _void("orc_argmax", _p(logits), c_i32(T), c_i64(V), _p(tok), _p(margin))
    return tok, margin


# ---- whole decoder

class Config(C.Structure):
    """eb_config as include/eidola_b200.h declares it, mirrored here so that the CPU checker (and a benchmark arm that
    runs nothing but the checker) needs no part of the CUDA library's binding."""
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


def make_config(**kw) -> Config:
    """The benchmark family's defaults (head_dim 64, page 16, window 128, top-4, std 0.02), as the engine's binding has them."""
    d = dict(head_dim=64, window=128, top_k=4, page_size=16, max_q_len=1, rope_theta=150000.0, rms_eps=1e-5,
             init_std=0.02, seed=0, debug=0, window_ring=0)
    d.update(kw)
    c = Config()
    for k, v in d.items():
        setattr(c, k, v)
    return c


class Model:
    """orc_model_*: the CPU decoder.  `cfg` is the ctypes eb_config the engine is created with."""

    def __init__(self, cfg):
        self.cfg = cfg
        _lib.orc_model_create.restype = c_vp
        self._h = c_vp(_lib.orc_model_create(C.byref(cfg)))

    def close(self):
        if self._h:
            _void("orc_model_destroy", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def kv_fill_synth(self):
        _void("orc_model_kv_fill_synth", self._h)

    def last(self, which: str) -> np.ndarray:
        """Intermediate of the last layer the last step ran: "qkv" (rotated q | k | v rows), "attn" (attention output) or
        "o" (O projection output); a copy, [T][width] bf16 bits."""
        idx = {"qkv": 0, "attn": 1, "o": 2}[which]
        p = C.POINTER(C.c_uint16)()
        _lib.orc_model_last.restype = C.c_int64
        n = int(_lib.orc_model_last(self._h, C.c_int32(idx), C.byref(p)))
        c = self.cfg
        width = {"qkv": (c.n_q_heads + 2 * c.n_kv_heads) * c.head_dim, "attn": c.n_q_heads * c.head_dim, "o": c.hidden}[which]
        return np.ctypeslib.as_array(p, shape=(n // width, width)).copy()

    def embed_table(self) -> np.ndarray:
        """A writable view of the embedding table [vocab][hidden] (uint16 bf16 bits)."""
        _lib.orc_model_embed.restype = C.POINTER(C.c_uint16)
        p = _lib.orc_model_embed(self._h)
        return np.ctypeslib.as_array(p, shape=(self.cfg.vocab, self.cfg.hidden))

    def step(self, packed, tokens, block_tables, n_layers_run=None, want_logits=True, want_debug=False):
        """packed: the dict eb_sched_pack produces.  Returns a dict of outputs."""
        c = self.cfg
        T, n = int(packed["n_tokens"]), len(packed["slots"])
        bt = _i32(block_tables)
        nl = c.n_layers if n_layers_run is None else n_layers_run
        out = {"next": np.empty(T, np.int32), "margin": np.empty(T, np.float32)}
        logits = np.empty((T, c.vocab), np.uint16) if want_logits else None
        ridx = np.zeros((c.n_layers, T, c.top_k), np.int32) if want_debug else None
        rlog = np.zeros((c.n_layers, T, c.n_experts), np.float32) if want_debug else None
        hid = np.zeros((c.n_layers + 1, T, c.hidden), np.uint16) if want_debug else None
        opt = lambda a: _p(a) if a is not None else c_vp(None)  # noqa: E731
        _void("orc_model_step", self._h, c_i32(T), c_i32(n), _p(_i32(tokens)), _p(_i32(packed["tok_slot"])),
              _p(_i32(packed["positions"])), _p(_i32(packed["slots"])), _p(_i32(packed["q_off"])),
              _p(_i32(packed["ctx_lens"])), _p(bt), c_i32(bt.shape[1]), c_i32(nl), _p(out["next"]), _p(out["margin"]),
              opt(logits), opt(ridx), opt(rlog), opt(hid))
        out.update(logits=logits, route_idx=ridx, route_logits=rlog, hidden=hid)
        return out
