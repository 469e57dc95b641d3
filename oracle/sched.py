"""Pure-Python restatement of the page scheduler and the split-K attention plan (TEST INFRASTRUCTURE).

Block tables, packing arrays and plans are integer work: the CUDA library's host scheduler must match this
bit for bit.  The reference project has no page scheduler; its nearest analogue is the whole-engine admission
planner, crates/eidola-app-core/src/local_models.rs:441-485 and :653-701 (plan and reserve atomically, refuse
without side effects).  Parity unpinned: no reference test asserts a block table.
"""
from __future__ import annotations

M64 = (1 << 64) - 1


def mix64(z: int) -> int:
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & M64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & M64
    z ^= z >> 31
    return z


def eb_hash(seed: int, stream: int, idx: int) -> int:
    z = mix64((seed + 0x9E3779B97F4A7C15) & M64)
    z = mix64(z ^ ((stream * 0xD1B54A32D192ED03 + 0x8CB92BA72F3D8DD7) & M64))
    z = mix64(z ^ ((idx * 0x9E3779B97F4A7C15 + 0x2545F4914F6CDD1D) & M64))
    return z


def plan_evictions(required, budget, entries):
    """The reference's pure eviction planner (crates/eidola-app-core/src/local_models.rs:653-701), restated: `entries` is a
    list of (key, footprint, last_used, pinned, in_flight) in registry order.  Returns the keys to evict, least recently
    used first and only as many as needed, [] when the request already fits, or a string starting with "budget" /
    "held" when it cannot fit (nothing is evicted then)."""
    if required > budget:
        return "budget"
    free = max(0, budget - sum(e[1] for e in entries))
    if free >= required:
        return []
    cand = sorted((e for e in entries if not e[3] and not e[4]), key=lambda e: e[2])
    out = []
    for e in cand:
        if free >= required:
            break
        free += e[1]
        out.append(e[0])
    return out if free >= required else "held"


class Sched:
    def __init__(self, num_pages, page_size, max_seqs, max_pages, seed):
        self.page_size, self.max_seqs, self.max_pages = page_size, max_seqs, max_pages
        fl = list(range(num_pages))
        for i in range(num_pages - 1, 0, -1):
            j = eb_hash(seed, 0x5EED, i) % (i + 1)
            fl[i], fl[j] = fl[j], fl[i]
        self.free = fl
        self.tables = [[-1] * max_pages for _ in range(max_seqs)]
        self.len = [-1] * max_seqs

    def _pages(self, n):
        return (n + self.page_size - 1) // self.page_size

    def admit(self, n):
        need = self._pages(n)
        if need > self.max_pages or need > len(self.free):
            return None
        slot = next((i for i in range(self.max_seqs) if self.len[i] < 0), None)
        if slot is None:
            return None
        for p in range(need):
            self.tables[slot][p] = self.free.pop()
        self.len[slot] = n
        return slot

    def extend(self, slot, n):
        have, need = self._pages(self.len[slot]), self._pages(n)
        if need > self.max_pages or need - have > len(self.free):
            return False
        for p in range(have, need):
            self.tables[slot][p] = self.free.pop()
        self.len[slot] = n
        return True

    def truncate(self, slot, n):
        have, need = self._pages(self.len[slot]), self._pages(n)
        for p in range(have - 1, need - 1, -1):
            self.free.append(self.tables[slot][p])
            self.tables[slot][p] = -1
        self.len[slot] = n

    def release(self, slot):
        self.truncate(slot, 0)
        self.len[slot] = -1

    def pack(self, slots, q_lens):
        q_off, ctx, tok_seq, tok_slot, pos = [], [], [], [], []
        t = 0
        for i, (s, ql) in enumerate(zip(slots, q_lens)):
            L = self.len[s]
            q_off.append(t)
            ctx.append(L)
            for j in range(ql):
                tok_seq.append(i)
                tok_slot.append(s)
                pos.append(L - ql + j)
                t += 1
        q_off.append(t)
        return {"q_off": q_off, "ctx_lens": ctx, "tok_seq": tok_seq, "tok_slot": tok_slot, "positions": pos}


def attn_plan(ctx_lens, q_lens, page_size, window, sm_count, chunk_pages=0, parts_per_item=1):
    rng = []
    total = 0
    for L, ql in zip(ctx_lens, q_lens):
        t_lo = max(0, L - ql - window + 1) if window > 0 else 0
        pb, pe = t_lo // page_size, (L + page_size - 1) // page_size
        rng.append((pb, pe))
        total += pe - pb
    chunk = chunk_pages
    if chunk == 0:
        target = 4 * sm_count
        chunk = min(512, max(8, (total + target - 1) // target))
        max_np = max((pe - pb for pb, pe in rng), default=0)
        if len(rng) >= sm_count and max_np <= 2 * chunk:  # short ranges that already fill the SMs stay whole
            chunk = max(chunk, min(512, max_np))
    items, seq_part, parts = [], [], 0
    for i, (pb, pe) in enumerate(rng):
        np_ = pe - pb
        k = (np_ + chunk - 1) // chunk
        seq_part.append(parts)
        base, rem = divmod(np_, k)
        p = pb
        for c in range(k):
            sz = base + (1 if c < rem else 0)
            items.append((i, p, p + sz, parts))
            p += sz
            parts += parts_per_item
    seq_part.append(parts)
    items.sort(key=lambda it: -(it[2] - it[1]))  # stable
    return {"items": items, "seq_part": seq_part, "n_parts": parts}
