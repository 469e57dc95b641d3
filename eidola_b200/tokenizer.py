"""Tokenizer and chat template from the metadata of a GGUF checkpoint, for the engine process (eidola_b200.server).

The reference's client starts its engine with `--jinja` (crates/eidola-app-core/src/local_models.rs:1612-1626): the
engine is expected to turn `messages` into a prompt with the chat template stored in the model file and to tokenise it
with the vocabulary stored there.  The reference itself contains neither step (they live inside the third-party engine);
this module restates the two published schemes the files of the reference's model catalogue use:

* byte-level BPE ("gpt2" tokenizer model): text is split by a pre-tokenisation pattern, every piece is mapped byte by
  byte to printable code points, and adjacent symbols are merged in the order of the file's merge list;
* the chat template is a Jinja program over `messages`, `add_generation_prompt`, `bos_token` and `eos_token`.

Metadata keys read: tokenizer.ggml.model, .pre, .tokens, .merges, .token_type (3 = control: matched verbatim in the
text), .bos_token_id, .eos_token_id, tokenizer.chat_template.  Nothing here was checked against a file from elsewhere
(there is no network where this was written): the tests build their own vocabulary, merges and template.
"""
from __future__ import annotations

import struct
from functools import lru_cache

_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


def read_gguf_metadata(path, keys_prefix: tuple[str, ...] = ("tokenizer.", "general."), tensor_shapes: dict | None = None) -> dict:
    """The metadata entries of a GGUF file whose keys start with one of `keys_prefix` (arrays as Python lists).  When
    `tensor_shapes` is a dict it receives name -> extents (outermost first) of every tensor of the file."""
    out = {}
    with open(path, "rb") as f:
        if f.read(4) != b"GGUF":
            raise ValueError("%s is not a GGUF file" % path)
        version, = struct.unpack("<I", f.read(4))
        if version not in (2, 3):
            raise ValueError("GGUF version %d (2 and 3 are read)" % version)
        n_tensors, n_kv = struct.unpack("<QQ", f.read(16))

        def string():
            n, = struct.unpack("<Q", f.read(8))
            return f.read(n).decode("utf-8", errors="replace")

        def value(t, keep):
            if t in _SCALAR:
                fmt = _SCALAR[t]
                return struct.unpack(fmt, f.read(struct.calcsize(fmt)))[0]
            if t == 8:
                return string()
            if t == 9:
                et, n = struct.unpack("<IQ", f.read(12))
                if et in _SCALAR and not keep:  # skip large numeric arrays nobody asked for in one seek
                    f.seek(n * struct.calcsize(_SCALAR[et]), 1)
                    return None
                return [value(et, keep) for _ in range(n)]
            raise ValueError("GGUF metadata value type %d" % t)

        for _ in range(n_kv):
            key = string()
            t, = struct.unpack("<I", f.read(4))
            keep = key.startswith(keys_prefix)
            v = value(t, keep)
            if keep:
                out[key] = v
        if tensor_shapes is not None:
            for _ in range(n_tensors):
                name = string()
                nd, = struct.unpack("<I", f.read(4))
                ne = struct.unpack("<%dQ" % nd, f.read(8 * nd))
                f.read(12)  # type, offset
                tensor_shapes[name] = tuple(reversed(ne))
    return out


@lru_cache(maxsize=1)
def _byte_to_char() -> dict:
    """The byte <-> printable code point table of byte-level BPE: printable Latin-1 bytes stand for themselves, the
    other 68 bytes take the code points from 256 upwards in order."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    return table


# Pre-tokenisation patterns by tokenizer.ggml.pre.  "gpt2": contractions, letters, digits, other, white space.  "gpt-4o":
# the 200k-vocabulary scheme (case-aware words with optional contraction suffix, digit runs of up to three).
_PATTERNS = {
    "gpt2": r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+",
    "gpt-4o": (r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?"
               r"|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?"
               r"|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+"),
}


class BpeTokenizer:
    """Byte-level BPE over a GGUF vocabulary.  encode(text) -> ids, decode(ids) -> text; control tokens (token_type 3)
    that occur verbatim in the text become their own id and are never merged with their surroundings."""

    def __init__(self, tokens, merges, token_type=None, pre="gpt2", bos_id=None, eos_id=None, chat_template=None):
        import regex
        self.tokens = list(tokens)
        self.id_of = {t: i for i, t in enumerate(self.tokens)}
        self.rank = {}
        for r, m in enumerate(merges):
            a, _, b = m.partition(" ")
            self.rank[(a, b)] = r
        self.pattern = regex.compile(_PATTERNS.get(pre, _PATTERNS["gpt2"]))
        self.control = [t for t, k in zip(self.tokens, token_type or []) if k == 3 and t]
        self.control_re = regex.compile("|".join(regex.escape(t) for t in sorted(self.control, key=len, reverse=True))) if self.control else None
        self.control_ids = {self.id_of[t] for t in self.control}
        self.b2c = _byte_to_char()
        self.c2b = {c: b for b, c in self.b2c.items()}
        self.bos_id, self.eos_id = bos_id, eos_id
        self.eos = eos_id if eos_id is not None else -1
        self.chat_template = chat_template
        self._cache = {}

    @classmethod
    def from_gguf(cls, path):
        """None when the file carries no byte-level BPE vocabulary."""
        md = read_gguf_metadata(path)
        if md.get("tokenizer.ggml.model") != "gpt2" or not md.get("tokenizer.ggml.tokens"):
            return None
        return cls(md["tokenizer.ggml.tokens"], md.get("tokenizer.ggml.merges") or [], md.get("tokenizer.ggml.token_type"),
                   md.get("tokenizer.ggml.pre") or "gpt2", md.get("tokenizer.ggml.bos_token_id"), md.get("tokenizer.ggml.eos_token_id"),
                   md.get("tokenizer.chat_template"))

    def _bpe(self, piece: str) -> list[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        sym = [self.b2c[b] for b in piece.encode("utf-8")]
        while len(sym) > 1:
            best, at = None, -1
            for i in range(len(sym) - 1):
                r = self.rank.get((sym[i], sym[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            a, b = sym[at], sym[at + 1]
            merged, i = [], 0
            while i < len(sym):  # every occurrence of the pair, left to right
                if i + 1 < len(sym) and sym[i] == a and sym[i + 1] == b:
                    merged.append(a + b)
                    i += 2
                else:
                    merged.append(sym[i])
                    i += 1
            sym = merged
        ids = []
        for s in sym:
            i = self.id_of.get(s)
            if i is None:  # a symbol the vocabulary lacks: fall back to its bytes' own tokens
                ids += [self.id_of[c] for c in s if c in self.id_of]
            else:
                ids.append(i)
        if len(self._cache) < 65536:
            self._cache[piece] = ids
        return ids

    def encode(self, text: str) -> list[int]:
        out: list[int] = []
        pos = 0
        spans = list(self.control_re.finditer(text)) if self.control_re else []
        for m in spans + [None]:
            chunk = text[pos:m.start()] if m else text[pos:]
            for piece in self.pattern.findall(chunk):
                out += self._bpe(piece)
            if m:
                out.append(self.id_of[m.group()])
                pos = m.end()
        return out

    def token_bytes(self, i: int, skip_control: bool = True) -> bytes:
        """The bytes one id stands for (a token may end in the middle of a UTF-8 sequence: join bytes, then decode)."""
        if not (0 <= i < len(self.tokens)):
            return b"?"
        if i in self.control_ids:
            return b"" if skip_control else self.tokens[i].encode("utf-8")
        buf = bytearray()
        for c in self.tokens[i]:
            b = self.c2b.get(c)
            buf += bytes([b]) if b is not None else c.encode("utf-8")
        return bytes(buf)

    def decode(self, ids, skip_control: bool = True) -> str:
        return b"".join(self.token_bytes(i, skip_control) for i in ids).decode("utf-8", errors="replace")

    def template(self, messages, tools=None, tool_choice=None) -> list[int]:
        """`messages` -> prompt ids: the file's chat template when it has one (it also sees `tools` and `tool_choice`, as
        the request carries them), a plain role header otherwise."""
        norm = []
        for m in messages:
            content = m.get("content") or ""
            if isinstance(content, list):  # OpenAI content parts: keep the text parts
                content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
            norm.append(dict(m, role=m.get("role", "user"), content=content))  # (tool_calls, name, ... stay for the template)
        if self.chat_template:
            import jinja2
            env = jinja2.Environment(trim_blocks=True, lstrip_blocks=True, undefined=jinja2.ChainableUndefined)
            env.globals["raise_exception"] = _raise
            tok = lambda i: self.tokens[i] if i is not None and 0 <= i < len(self.tokens) else ""  # noqa: E731
            text = env.from_string(self.chat_template).render(messages=norm, add_generation_prompt=True, tools=tools,
                                                              tool_choice=tool_choice, bos_token=tok(self.bos_id),
                                                              eos_token=tok(self.eos_id))
        else:
            text = "".join("<|%s|>\n%s\n" % (m["role"], m["content"]) for m in norm) + "<|assistant|>\n"
        ids = self.encode(text)
        return ids or self.encode(" ")


def _raise(msg):
    raise ValueError(msg)


def shape_from_gguf(path) -> dict:
    """The decoder's dimensions as a GGUF file's `<architecture>.*` metadata states them, under the names of eb_config
    (only the keys the file has).  Keys read: block_count, embedding_length, attention.head_count, .head_count_kv,
    .key_length (head dimension), .sliding_window, expert_count, expert_used_count, expert_feed_forward_length (else
    feed_forward_length), rope.freq_base, attention.layer_norm_rms_epsilon; the vocabulary size is the number of rows of
    token_embd.weight."""
    general = read_gguf_metadata(path, ("general.",))
    arch = general.get("general.architecture")
    if not arch:
        return {}
    shapes: dict = {}
    md = read_gguf_metadata(path, (arch + ".",), shapes)
    names = {"block_count": "n_layers", "embedding_length": "hidden", "attention.head_count": "n_q_heads",
             "attention.head_count_kv": "n_kv_heads", "attention.key_length": "head_dim", "attention.sliding_window": "window",
             "expert_count": "n_experts", "expert_used_count": "top_k", "rope.freq_base": "rope_theta",
             "attention.layer_norm_rms_epsilon": "rms_eps"}
    out = {}
    for key, name in names.items():
        v = md.get("%s.%s" % (arch, key))
        if v is not None and not isinstance(v, list):
            out[name] = float(v) if name in ("rope_theta", "rms_eps") else int(v)
    inter = md.get(arch + ".expert_feed_forward_length", md.get(arch + ".feed_forward_length"))
    if inter is not None and not isinstance(inter, list):
        out["inter"] = int(inter)
    if out and "token_embd.weight" in shapes:
        out["vocab"] = int(shapes["token_embd.weight"][0])
    return out

