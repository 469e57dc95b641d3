"""CPU: the byte-level BPE tokenizer and chat template read from GGUF metadata (eidola_b200/tokenizer.py).  The vocabulary
and merge list are trained here on a few sentences, so every expectation can be checked by hand or by round trip."""
import collections

import numpy as np

from eidola_b200.tokenizer import BpeTokenizer, _byte_to_char, read_gguf_metadata
from tests.gguf_writer import write_gguf

CORPUS = ("the quick brown fox jumps over the lazy dog. the dog sleeps; the fox thinks. "
          "hello hello world, hello there! numbers 12345 and 678. naïve café über straße 東京 \n\n new line")
CONTROL = ["<|start|>", "<|end|>", "<|message|>", "<|eot|>"]
TEMPLATE = ("{{ bos_token }}{% for m in messages %}<|start|>{{ m['role'] }}<|message|>{{ m['content'] }}<|end|>{% endfor %}"
            "{% if add_generation_prompt %}<|start|>assistant<|message|>{% endif %}")


def _train(n_merges=120):
    """A toy trainer: repeatedly merge the most frequent adjacent pair of the corpus' pre-tokens (ties: first seen)."""
    import regex
    from eidola_b200.tokenizer import _PATTERNS
    b2c = _byte_to_char()
    words = [[b2c[b] for b in w.encode()] for w in regex.findall(_PATTERNS["gpt2"], CORPUS)]
    merges = []
    for _ in range(n_merges):
        pairs = collections.Counter()
        for w in words:
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += 1
        if not pairs or pairs.most_common(1)[0][1] < 2:
            break
        (a, b), _ = pairs.most_common(1)[0]
        merges.append(f"{a} {b}")
        for w in words:
            i = 0
            while i + 1 < len(w):
                if w[i] == a and w[i + 1] == b:
                    w[i:i + 2] = [a + b]
                else:
                    i += 1
    tokens = [b2c[b] for b in range(256)] + [m.replace(" ", "") for m in merges] + CONTROL
    types = [1] * (256 + len(merges)) + [3] * len(CONTROL)
    return tokens, merges, types


def _tok():
    tokens, merges, types = _train()
    return BpeTokenizer(tokens, merges, types, "gpt2", bos_id=tokens.index("<|start|>"), eos_id=tokens.index("<|eot|>"), chat_template=TEMPLATE)


def test_round_trip_and_merges():
    t = _tok()
    rng = np.random.default_rng(0)
    texts = [CORPUS, "", " ", "a", "hello", "the the the", "tab\there\r\n", "emoji 🙂 and 東京タワー", "'s 't I'm we'll",
             "".join(chr(int(c)) for c in rng.integers(32, 0x2FF, size=200))]
    for s in texts:
        ids = t.encode(s)
        assert t.decode(ids) == s
        assert all(0 <= i < len(t.tokens) for i in ids)
    # merges apply in the order of the list: the corpus' commonest words are single tokens, unseen words are not
    assert len(t.encode(" the")) == 1 and len(t.encode(" hello")) == 1
    assert len(t.encode(" zyxwv")) > 1
    # a word the corpus only has with a leading space is merged as far as the shared pairs go, no further
    ids = t.encode("hello")
    assert "".join(t.tokens[i] for i in ids) == "hello" and 1 < len(ids) < 5
    assert len(t.encode(CORPUS)) < len(CORPUS.encode()) * 0.75  # it compresses what it was trained on (pairs seen twice)


def test_control_tokens_are_atomic_and_skipped_on_decode():
    t = _tok()
    ids = t.encode("<|start|>user<|message|>hi<|end|>")
    names = [t.tokens[i] for i in ids]
    assert names[0] == "<|start|>" and "<|message|>" in names and names[-1] == "<|end|>"
    assert t.decode(ids) == "userhi" and t.decode(ids, skip_control=False) == "<|start|>user<|message|>hi<|end|>"
    assert t.encode("<|start") != [t.id_of["<|start|>"]]  # only the whole spelling is the control token
    # a token that ends inside a UTF-8 sequence: bytes join across tokens
    parts = [t.token_bytes(i) for i in t.encode("é東")]
    assert b"".join(parts).decode() == "é東" and len(parts) > 2


def test_chat_template_and_gguf_metadata(tmp_path):
    tokens, merges, types = _train()
    path = tmp_path / "tok.gguf"
    write_gguf(path, {"x": np.zeros((2, 32), np.float32)},
               {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "gpt2", "tokenizer.ggml.tokens": tokens,
                "tokenizer.ggml.merges": merges, "tokenizer.ggml.token_type": types,
                "tokenizer.ggml.bos_token_id": np.uint32(tokens.index("<|start|>")),
                "tokenizer.ggml.eos_token_id": np.uint32(tokens.index("<|eot|>")), "tokenizer.chat_template": TEMPLATE})
    md = read_gguf_metadata(path)
    assert md["tokenizer.ggml.tokens"] == tokens and md["tokenizer.ggml.merges"] == merges and md["tokenizer.ggml.token_type"] == types
    t = BpeTokenizer.from_gguf(path)
    assert t is not None and t.eos == tokens.index("<|eot|>")
    ids = t.template([{"role": "system", "content": "be brief"}, {"role": "user", "content": [{"type": "text", "text": "hello fox"}]}])
    text = t.decode(ids, skip_control=False)
    assert text == ("<|start|><|start|>system<|message|>be brief<|end|><|start|>user<|message|>hello fox<|end|>"
                    "<|start|>assistant<|message|>")
    assert ids.count(t.id_of["<|message|>"]) == 3
    # a file without a vocabulary: no tokenizer (the server falls back to bytes)
    write_gguf(tmp_path / "plain.gguf", {"x": np.zeros((2, 32), np.float32)})
    assert BpeTokenizer.from_gguf(tmp_path / "plain.gguf") is None
    # the engine's own reader still finds the tensors behind array-valued metadata
    import ctypes as C
    from eidola_b200 import capi
    out = np.empty(64, np.float32)
    capi.call("eb_gguf_read_f32", str(path).encode(), b"x", C.c_int64(0), C.c_int64(64), capi.ptr(out), None, None)
    assert not out.any()


def test_the_200k_scheme_splits_digits_in_threes_and_keeps_case_runs():
    import regex
    from eidola_b200.tokenizer import _PATTERNS
    p = regex.compile(_PATTERNS["gpt-4o"])
    assert p.findall("abc 1234567 XyZ don't") == ["abc", " ", "123", "456", "7", " Xy", "Z", " don't"]
    assert "".join(p.findall(CORPUS)) == CORPUS  # the pattern covers every character


def test_engine_dimensions_come_from_the_files_architecture_metadata(tmp_path):
    from eidola_b200.tokenizer import shape_from_gguf
    tokens, merges, types = _train()
    md = {"general.architecture": "gpt-oss", "gpt-oss.block_count": np.uint32(24), "gpt-oss.embedding_length": np.uint32(2880),
          "gpt-oss.attention.head_count": np.uint32(64), "gpt-oss.attention.head_count_kv": np.uint32(8),
          "gpt-oss.attention.key_length": np.uint32(64), "gpt-oss.attention.sliding_window": np.uint32(128),
          "gpt-oss.expert_count": np.uint32(32), "gpt-oss.expert_used_count": np.uint32(4),
          "gpt-oss.expert_feed_forward_length": np.uint32(2880), "gpt-oss.feed_forward_length": np.uint32(9999),
          "gpt-oss.rope.freq_base": 150000.0, "gpt-oss.attention.layer_norm_rms_epsilon": 1e-5,
          "tokenizer.ggml.model": "gpt2", "tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges, "tokenizer.ggml.token_type": types}
    path = tmp_path / "arch.gguf"
    write_gguf(path, {"x": np.zeros((2, 32), np.float32), "token_embd.weight": np.zeros((500, 32), np.float32)}, md)
    got = shape_from_gguf(path)
    assert got == {"n_layers": 24, "hidden": 2880, "n_q_heads": 64, "n_kv_heads": 8, "head_dim": 64, "window": 128, "n_experts": 32,
                   "top_k": 4, "inter": 2880, "rope_theta": 150000.0, "rms_eps": got["rms_eps"], "vocab": 500}
    assert abs(got["rms_eps"] - 1e-5) < 1e-9
    # a file that states nothing keeps the caller's defaults
    write_gguf(tmp_path / "bare.gguf", {"x": np.zeros((2, 32), np.float32)})
    assert shape_from_gguf(tmp_path / "bare.gguf") == {}
