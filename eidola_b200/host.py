"""Typed wrappers over the C ABI: one Python function per entry point, arguments in the header's order."""
from __future__ import annotations

import ctypes as C

import numpy as np

from .capi import (AttnArgs, AttnItem, Config, GemmArgs, DeviceBuffer, call, c_f32, c_i32, c_i64, c_sz, c_u64, c_vp, lib, ptr)

I32 = np.int32


def _i32(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=I32))


class Scheduler:
    """eb_sched_*: page pool + block tables + ragged packing (host only)."""

    def __init__(self, num_pages: int, page_size: int, max_seqs: int, max_pages_per_seq: int, seed: int):
        self._h = c_vp()
        call("eb_sched_create", c_i32(num_pages), c_i32(page_size), c_i32(max_seqs), c_i32(max_pages_per_seq),
             c_u64(seed), C.byref(self._h))
        self.num_pages, self.page_size, self.max_seqs, self.max_pages = num_pages, page_size, max_seqs, max_pages_per_seq

    def close(self):
        if self._h:
            call("eb_sched_destroy", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def admit(self, context_len: int) -> int:
        slot = c_i32(-1)
        call("eb_sched_admit", self._h, c_i32(context_len), C.byref(slot))
        return int(slot.value)

    def extend(self, slot: int, new_len: int) -> None:
        call("eb_sched_extend", self._h, c_i32(slot), c_i32(new_len))

    def truncate(self, slot: int, new_len: int) -> None:
        call("eb_sched_truncate", self._h, c_i32(slot), c_i32(new_len))

    def release(self, slot: int) -> None:
        call("eb_sched_release", self._h, c_i32(slot))

    def free_pages(self) -> int:
        n = c_i32(0)
        call("eb_sched_free_pages", self._h, C.byref(n))
        return int(n.value)

    def seq_len(self, slot: int) -> int:
        n = c_i32(0)
        call("eb_sched_seq_len", self._h, c_i32(slot), C.byref(n))
        return int(n.value)

    def block_tables(self) -> np.ndarray:
        """A copy of the [max_seqs][max_pages_per_seq] table."""
        p = C.POINTER(c_i32)()
        stride = c_i32(0)
        call("eb_sched_block_tables", self._h, C.byref(p), C.byref(stride))
        return np.ctypeslib.as_array(p, shape=(self.max_seqs, int(stride.value))).copy()

    def pack(self, slots, q_lens) -> dict:
        slots, q_lens = _i32(slots), _i32(q_lens)
        n = len(slots)
        cap = int(q_lens.sum()) if n else 0
        q_off = np.zeros(n + 1, I32)
        ctx = np.zeros(n, I32)
        tok_seq, tok_slot, pos = np.zeros(cap, I32), np.zeros(cap, I32), np.zeros(cap, I32)
        nt = c_i32(0)
        call("eb_sched_pack", self._h, ptr(slots), ptr(q_lens), c_i32(n), ptr(q_off), ptr(ctx), ptr(tok_seq),
             ptr(tok_slot), ptr(pos), C.byref(nt))
        assert nt.value == cap
        return {"slots": slots, "q_lens": q_lens, "q_off": q_off, "ctx_lens": ctx, "tok_seq": tok_seq,
                "tok_slot": tok_slot, "positions": pos, "n_tokens": cap}


def attn_plan_sm_count(sm_count: int, max_q_len: int, n_q: int, n_kv: int, window: int) -> int:
    """The sm_count to plan with so that the automatic chunk size suits the kernel the launch will run."""
    lib().eb_attn_plan_sm_count.restype = C.c_int32
    return int(lib().eb_attn_plan_sm_count(c_i32(sm_count), c_i32(max_q_len), c_i32(n_q), c_i32(n_kv), c_i32(window)))


def attn_plan(ctx_lens, q_lens, page_size: int, window: int, sm_count: int, chunk_pages: int = 0,
              parts_per_item: int = 1) -> dict:
    ctx_lens, q_lens = _i32(ctx_lens), _i32(q_lens)
    n = len(ctx_lens)
    cap = int(((ctx_lens.astype(np.int64) + page_size - 1) // page_size).sum()) + n + 1
    items = (AttnItem * cap)()
    n_items, n_parts = c_i32(0), c_i32(0)
    seq_part = np.zeros(n + 1, I32)
    call("eb_attn_plan", ptr(ctx_lens), ptr(q_lens), c_i32(n), c_i32(page_size), c_i32(window), c_i32(sm_count),
         c_i32(chunk_pages), c_i32(parts_per_item), items, c_i32(cap), C.byref(n_items), ptr(seq_part),
         C.byref(n_parts))
    arr = np.frombuffer(items, dtype=I32).reshape(cap, 4)[: n_items.value].copy()
    return {"items": arr, "seq_part": seq_part, "n_items": int(n_items.value), "n_parts": int(n_parts.value)}


def kv_append(d_cache, num_pages, n_kv, head_dim, page_size, d_k_new, d_v_new, row_stride, d_block_tables, bt_stride,
              d_tok_slot, d_positions, n_tokens, stream=None) -> None:
    call("eb_kv_append", c_vp(d_cache), c_i32(num_pages), c_i32(n_kv), c_i32(head_dim), c_i32(page_size),
         c_vp(d_k_new), c_vp(d_v_new), c_i64(row_stride), c_vp(d_block_tables), c_i32(bt_stride), c_vp(d_tok_slot),
         c_vp(d_positions), c_i32(n_tokens), c_vp(stream))


def attn_workspace(n_parts, max_q_len, n_q, head_dim) -> tuple[int, int]:
    a, m = c_sz(0), c_sz(0)
    call("eb_attn_workspace", c_i32(n_parts), c_i32(max_q_len), c_i32(n_q), c_i32(head_dim), C.byref(a), C.byref(m))
    return int(a.value), int(m.value)


def attn_paged_sink(args: AttnArgs, stream=None) -> None:
    call("eb_attn_paged_sink", C.byref(args), c_vp(stream))


def attn_paged_sink_static(args: AttnArgs, d_status=None, stream=None) -> None:
    """The variant that allocates nothing: split-K scratch lives in arrays built into the library."""
    call("eb_attn_paged_sink_static", C.byref(args), c_vp(d_status), c_vp(stream))


class AttnLaunch:
    """Device-resident arguments of one attention launch, built from a packed step and a plan."""

    def __init__(self, *, d_q, q_stride, d_out, out_stride, d_cache, num_pages, d_block_tables, bt_stride, packed,
                 plan, d_sinks, window, n_q, n_kv, head_dim=64, page_size=16, scale=0.125):
        self.max_q_len = int(packed["q_lens"].max()) if len(packed["q_lens"]) else 1
        self.bufs = {
            "seq_slots": DeviceBuffer.from_array(_i32(packed["slots"])),
            "q_off": DeviceBuffer.from_array(_i32(packed["q_off"])),
            "ctx_lens": DeviceBuffer.from_array(_i32(packed["ctx_lens"])),
            "items": DeviceBuffer.from_array(_i32(plan["items"])),
            "seq_part": DeviceBuffer.from_array(_i32(plan["seq_part"])),
        }
        acc_b, ml_b = attn_workspace(plan["n_parts"], self.max_q_len, n_q, head_dim)
        self.bufs["acc"] = DeviceBuffer(acc_b)
        self.bufs["ml"] = DeviceBuffer(ml_b)
        a = AttnArgs()
        a.d_q, a.q_stride, a.d_out, a.out_stride = d_q, q_stride, d_out, out_stride
        a.d_cache, a.num_pages = d_cache, num_pages
        a.d_block_tables, a.bt_stride = d_block_tables, bt_stride
        a.d_seq_slots, a.d_q_off, a.d_ctx_lens = (self.bufs[k].ptr for k in ("seq_slots", "q_off", "ctx_lens"))
        a.n_seqs, a.max_q_len = len(packed["slots"]), self.max_q_len
        a.d_sinks, a.window = d_sinks, window
        a.n_q, a.n_kv, a.head_dim, a.page_size, a.scale = n_q, n_kv, head_dim, page_size, scale
        a.d_items, a.n_items = self.bufs["items"].ptr, plan["n_items"]
        a.d_seq_part, a.n_parts = self.bufs["seq_part"].ptr, plan["n_parts"]
        a.d_part_acc, a.d_part_ml = self.bufs["acc"].ptr, self.bufs["ml"].ptr
        self.args = a

    def run(self, stream=None) -> None:
        attn_paged_sink(self.args, stream)


def quant_act_block128(d_x, ldx, rows, cols, d_codes, d_scales, d_seg_off=None, n_groups=1, stream=None) -> None:
    call("eb_quant_act_block128", c_vp(d_x), c_i64(ldx), c_i32(rows), c_i32(cols), c_vp(d_seg_off), c_i32(n_groups),
         c_vp(d_codes), c_vp(d_scales), c_vp(stream))


def gemm_workspace(rows, N, n_groups) -> int:
    b = c_sz(0)
    call("eb_gemm_workspace", c_i32(rows), c_i32(N), c_i32(n_groups), C.byref(b))
    return int(b.value)


def gemm_fp8(d_x8, d_sx, d_w8, d_sw, d_y, rows, N, K, *, ldy=None, n_groups=1, d_seg_off=None, work=None,
             tile_tokens=0, splits=0, stream=None, w_tiled=False) -> None:
    """eb_gemm_fp8_block (n_groups == 1, no segments) or eb_gemm_fp8_grouped.  `work` is the DeviceBuffer lent as
    workspace (its size travels with the call, the library refuses what would not fit)."""
    d_work, work_bytes = (work.ptr, work.nbytes) if work is not None else (None, 0)
    a = GemmArgs()
    a.d_x8, a.d_sx, a.d_w8, a.d_sw, a.d_y = d_x8, d_sx, d_w8, d_sw, d_y
    a.ldy = N if ldy is None else ldy
    a.rows, a.N, a.K, a.n_groups = rows, N, K, n_groups
    a.d_seg_off, a.d_work, a.tile_tokens, a.splits = d_seg_off, d_work, tile_tokens, splits
    a.work_bytes = work_bytes
    a.w_tiled = 1 if w_tiled else 0
    call("eb_gemm_fp8_grouped" if d_seg_off is not None else "eb_gemm_fp8_block", C.byref(a), c_vp(stream))


def weight_tile_fp8(d_w8, n_groups, N, K, stream=None) -> DeviceBuffer:
    """eb_weight_tile_fp8: a new device buffer holding the 16 KiB-tile layout of row-major e4m3 weights."""
    b = c_sz(0)
    call("eb_weight_tiled_bytes", c_i32(n_groups), c_i32(N), c_i32(K), C.byref(b))
    out = DeviceBuffer(int(b.value))
    call("eb_weight_tile_fp8", c_vp(d_w8), c_i32(n_groups), c_i32(N), c_i32(K), c_vp(out.ptr), c_vp(stream))
    return out


class Comm:
    """eb_comm_*: the NCCL communicator of a tensor-/expert-parallel engine (one process per GPU)."""

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        call("eb_comm_unique_id", buf)
        return buf.raw

    def __init__(self, unique_id: bytes, rank: int, size: int):
        assert len(unique_id) == 128
        self._h = c_vp()
        self.rank, self.size = rank, size
        call("eb_comm_create", C.c_char_p(unique_id), c_i32(rank), c_i32(size), C.byref(self._h))

    def allreduce_f32(self, d_buf, count, stream=None) -> None:
        call("eb_comm_allreduce_f32", self._h, c_vp(d_buf), c_i64(count), c_vp(stream))

    def allgather(self, bufs, bytes_per_rank, stream=None) -> None:
        """In place, 1..3 buffers: rank r's slice of buffer i sits at offset r * bytes_per_rank[i]."""
        n = len(bufs)
        ptrs = (C.c_void_p * n)(*[int(b) for b in bufs])
        sizes = (C.c_int64 * n)(*[int(b) for b in bytes_per_rank])
        call("eb_comm_allgather", self._h, c_i32(n), ptrs, sizes, c_vp(stream))

    def reduce_scatter_f32(self, d_buf, count_per_rank, stream=None) -> None:
        call("eb_comm_reduce_scatter_f32", self._h, c_vp(d_buf), c_i64(count_per_rank), c_vp(stream))

    def async_error(self) -> int:
        """0 while the communicator is healthy (ncclCommGetAsyncError)."""
        e = c_i32(0)
        call("eb_comm_async_error", self._h, C.byref(e))
        return int(e.value)

    def abort(self) -> None:
        """Tear the communicator down without waiting for its peers (after a lost rank or a missed deadline)."""
        if self._h:
            call("eb_comm_abort", self._h)

    def close(self):
        if self._h:
            call("eb_comm_destroy", self._h)
            self._h = None


class PeerLost(RuntimeError):
    """A rank of the tensor-parallel group left or stopped answering; the communicator has been aborted."""

    def __init__(self, msg: str, ranks):
        super().__init__(msg)
        self.ranks = list(ranks)


class StepGuard:
    """Host-side liveness check of a tensor-parallel group, run BETWEEN steps, before the next launch.

    No kernel of this library waits on another rank outside a collective, and a collective whose peer never joins
    would block the stream.  So failure detection stays on the host, in the reference's style: its engine supervisor
    polls a child with a deadline and turns silence into an error (crates/eidola-app-core/src/local_models.rs:
    2020-2064, 2066-2099), and its tests script the failing peer (tests/chat_harness/mod.rs:100-108).  Every rank
    announces the step it is about to launch in a key-value store (anything with set(key, value) and get(key), e.g.
    torch.distributed.TCPStore); a rank that shuts down says so with leave().  wait_peers(step) returns once every
    peer has announced `step`; if a peer has left, or the deadline passes, it aborts the communicator (so that no
    collective of the next step can block) and raises PeerLost.  A rank leaves only between steps, with none of its
    kernels or collectives in flight.
    """

    def __init__(self, store, rank: int, world: int, comm=None, deadline_s: float = 5.0, poll_s: float = 0.005,
                 clock=None, sleep=None):
        import time
        self.store, self.rank, self.world, self.comm = store, rank, world, comm
        self.deadline_s, self.poll_s = deadline_s, poll_s
        self.clock = clock or time.monotonic
        self.sleep = sleep or time.sleep
        self.aborted = False

    def _get(self, key: str):
        try:
            if hasattr(self.store, "check") and not self.store.check([key]):
                return None
            v = self.store.get(key)
        except (KeyError, RuntimeError):
            return None
        return v.decode() if isinstance(v, (bytes, bytearray)) else v

    def announce(self, step: int) -> None:
        self.store.set(f"eb/step/{self.rank}", str(int(step)))

    def leave(self) -> None:
        self.store.set(f"eb/left/{self.rank}", "1")

    def _abort(self, msg: str, ranks):
        if self.comm is not None and not self.aborted:
            self.comm.abort()
        self.aborted = True
        raise PeerLost(msg, ranks)

    def wait_peers(self, step: int) -> None:
        t0 = self.clock()
        peers = [r for r in range(self.world) if r != self.rank]
        while True:
            behind = []
            for r in peers:
                v = self._get(f"eb/step/{r}")
                if v is None or int(v) < step:
                    behind.append(r)
            if not behind:
                return  # a peer that leaves after announcing this step is caught before the next one
            left = [r for r in behind if self._get(f"eb/left/{r}") is not None]
            if left:
                self._abort(f"rank(s) {left} left the group before step {step}", left)
            if self.comm is not None and self.comm.async_error() != 0:
                self._abort(f"communicator reports an asynchronous error before step {step}", behind)
            if self.clock() - t0 > self.deadline_s:
                self._abort(f"rank(s) {behind} did not announce step {step} within {self.deadline_s} s", behind)
            self.sleep(self.poll_s)


class Engine:
    """eb_engine_*: weights, KV pages, scheduler and the decode step."""

    def __init__(self, cfg: Config, tp_rank: int = 0, tp_size: int = 1, comm: "Comm | None" = None):
        self.cfg = cfg
        self._h = c_vp()
        self._comm = comm  # keep the communicator alive as long as the engine
        if tp_size == 1:
            call("eb_engine_create", C.byref(cfg), C.byref(self._h))
        else:
            call("eb_engine_create_tp", C.byref(cfg), c_i32(tp_rank), c_i32(tp_size), comm._h, C.byref(self._h))
        self._last_T = 0

    def close(self):
        if self._h:
            call("eb_engine_destroy", self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def memory(self) -> dict:
        w, k, x = c_i64(0), c_i64(0), c_i64(0)
        call("eb_engine_memory", self._h, C.byref(w), C.byref(k), C.byref(x))
        return {"weights": w.value, "kv": k.value, "work": x.value}

    def load_gguf(self, path: str) -> None:
        call("eb_engine_load_gguf", self._h, C.c_char_p(str(path).encode()))

    def kv_fill_synth(self) -> None:
        call("eb_engine_kv_fill_synth", self._h)

    def admit(self, context_len: int) -> int:
        slot = c_i32(-1)
        call("eb_engine_seq_admit", self._h, c_i32(context_len), C.byref(slot))
        return int(slot.value)

    def admit_evicting(self, context_len: int):
        """eb_engine_seq_admit_evicting: (slot, slots evicted to make room)."""
        cap = int(self.cfg.max_seqs)
        slot, n = c_i32(-1), c_i32(0)
        ev = (C.c_int32 * cap)()
        call("eb_engine_seq_admit_evicting", self._h, c_i32(context_len), C.byref(slot), ev, c_i32(cap), C.byref(n))
        return int(slot.value), [int(ev[i]) for i in range(n.value)]

    def pin(self, slot: int, pinned: bool = True) -> None:
        call("eb_engine_seq_pin", self._h, c_i32(slot), c_i32(1 if pinned else 0))

    def release(self, slot: int) -> None:
        call("eb_engine_seq_release", self._h, c_i32(slot))

    def truncate(self, slot: int, new_len: int) -> None:
        call("eb_engine_seq_truncate", self._h, c_i32(slot), c_i32(new_len))

    def truncate_many(self, slots, new_lens) -> None:
        slots, new_lens = _i32(slots), _i32(new_lens)
        call("eb_engine_seq_truncate_many", self._h, ptr(slots), ptr(new_lens), c_i32(len(slots)))

    def seq_len(self, slot: int) -> int:
        n = c_i32(0)
        call("eb_engine_seq_len", self._h, c_i32(slot), C.byref(n))
        return int(n.value)

    def block_tables(self) -> np.ndarray:
        sp = c_vp()
        call("eb_engine_sched", self._h, C.byref(sp))
        p = C.POINTER(c_i32)()
        stride = c_i32(0)
        call("eb_sched_block_tables", sp, C.byref(p), C.byref(stride))
        return np.ctypeslib.as_array(p, shape=(self.cfg.max_seqs, int(stride.value))).copy()

    def step(self, slots, q_lens, tokens):
        """Returns (next_tokens[T], margins[T])."""
        slots, q_lens, tokens = _i32(slots), _i32(q_lens), _i32(tokens)
        T = int(q_lens.sum())
        assert len(tokens) == T
        nxt, mg = np.empty(T, I32), np.empty(T, np.float32)
        call("eb_engine_step", self._h, ptr(slots), ptr(q_lens), c_i32(len(slots)), ptr(tokens), ptr(nxt), ptr(mg))
        self._last_T = T
        return nxt, mg

    def prefill(self, slots, prompts):
        """eb_engine_prefill: `prompts` is a list of token-id arrays.  Returns (first generated token per sequence, its
        margin, steps run, summed device milliseconds)."""
        slots = _i32(slots)
        lens = _i32([len(p) for p in prompts])
        flat = _i32(np.concatenate([np.asarray(p, I32) for p in prompts]))
        nxt, mg = np.empty(len(slots), I32), np.empty(len(slots), np.float32)
        steps, ms = c_i32(0), c_f32(0)
        call("eb_engine_prefill", self._h, ptr(slots), ptr(lens), c_i32(len(slots)), ptr(flat), ptr(nxt), ptr(mg), C.byref(steps),
             C.byref(ms))
        self._last_T = 0
        return nxt, mg, int(steps.value), float(ms.value)

    def sampling(self, slot: int, temperature: float, top_p: float = 1.0, seed: int = 0) -> None:
        """eb_engine_seq_sampling: temperature > 0 draws this sequence's tokens (nucleus top_p, counter-based random
        numbers from `seed`); temperature <= 0 returns it to greedy decoding."""
        call("eb_engine_seq_sampling", self._h, c_i32(slot), c_f32(temperature), c_f32(top_p), C.c_uint64(seed))

    def free_pages(self) -> int:
        """Pages of the pool that no sequence holds."""
        sp, n = c_vp(), c_i32(0)
        call("eb_engine_sched", self._h, C.byref(sp))
        call("eb_sched_free_pages", sp, C.byref(n))
        return int(n.value)

    def chunk_tokens(self) -> int:
        """Most new tokens one sequence may bring to a step (eb_engine_chunk_tokens)."""
        n = c_i32(0)
        call("eb_engine_chunk_tokens", self._h, C.byref(n))
        return int(n.value)

    def step_launch(self, slots, q_lens, tokens) -> None:
        slots, q_lens, tokens = _i32(slots), _i32(q_lens), _i32(tokens)
        self._last_T = int(q_lens.sum())
        call("eb_engine_step_launch", self._h, ptr(slots), ptr(q_lens), c_i32(len(slots)), ptr(tokens))

    def step_wait(self):
        nxt, mg = np.empty(self._last_T, I32), np.empty(self._last_T, np.float32)
        call("eb_engine_step_wait", self._h, ptr(nxt), ptr(mg))
        return nxt, mg

    def last_step_stats(self) -> tuple[float, int]:
        ms, n = c_f32(0), c_i32(0)
        call("eb_engine_last_step_stats", self._h, C.byref(ms), C.byref(n))
        return float(ms.value), int(n.value)

    def read_logits(self) -> np.ndarray:
        out = np.empty((self._last_T, self.cfg.vocab), np.uint16)
        call("eb_engine_read_logits", self._h, ptr(out), c_i64(out.nbytes))
        return out

    def read_routing(self, layer: int) -> np.ndarray:
        out = np.empty((self._last_T, self.cfg.top_k), I32)
        call("eb_engine_read_routing", self._h, c_i32(layer), ptr(out), c_i64(out.nbytes))
        return out

    def read_hidden(self, layer: int) -> np.ndarray:
        out = np.empty((self._last_T, self.cfg.hidden), np.uint16)
        call("eb_engine_read_hidden", self._h, c_i32(layer), ptr(out), c_i64(out.nbytes))
        return out

    def read_last(self, which: str, width: int) -> np.ndarray:
        """debug = 1: "qkv" (projection rows, q heads rotated) or "attn" (attention output) of the last layer."""
        out = np.empty((self._last_T, width), np.uint16)
        call("eb_engine_debug_read_last", self._h, c_i32({"qkv": 0, "attn": 1}[which]), ptr(out), c_i64(out.nbytes))
        return out

    def force_hidden(self, layer: int, x=None) -> None:
        if x is None:
            call("eb_engine_debug_force_hidden", self._h, c_i32(layer), c_vp(None), c_i32(0))
        else:
            x = np.ascontiguousarray(x, np.uint16)
            call("eb_engine_debug_force_hidden", self._h, c_i32(layer), ptr(x), c_i32(x.shape[0]))

    def last_step_copies(self) -> tuple[int, int]:
        """(host -> device, device -> host) bytes the last step copied."""
        a, b = c_i64(0), c_i64(0)
        call("eb_engine_last_step_copies", self._h, C.byref(a), C.byref(b))
        return int(a.value), int(b.value)

    def profile(self, on: bool) -> None:
        call("eb_engine_profile", self._h, c_i32(1 if on else 0))

    def last_step_breakdown(self) -> dict:
        ms = (c_f32 * 8)()
        call("eb_engine_last_step_breakdown", self._h, ms)
        return dict(zip(("attn_full", "attn_window", "dense_gemm", "expert_gemm", "lm_head", "collectives", "router",
                         "quantisers"), [float(v) for v in ms]))

    def stream(self):
        st = c_vp()
        call("eb_engine_stream", self._h, C.byref(st))
        return st.value
