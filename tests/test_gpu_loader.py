"""GPU: a GGUF checkpoint loaded into the engine.

The seeded weights are defined as fp32 values (eb_normal * std) that the engine quantises; writing exactly those values
to a GGUF file and loading it must therefore reproduce the seeded engine bit for bit -- block scales, e4m3 codes, tile
layout, bf16 embeddings and router, fp32 sinks -- which a decode step's logits show.  A second file with one tensor
changed shows that the file, not the seed, decides."""
import numpy as np
import pytest

from oracle import binding as orc
from tests.decoder_cases import TINY_CONTEXTS, tiny_config
from tests.gguf_writer import Blocked, write_gguf

pytestmark = pytest.mark.gpu


def _sid(layer, kind, expert=0):
    return ((layer + 1) << 20) | (kind << 12) | expert


def _seeded_tensors(cfg):
    """The fp32 values the engine's random init is defined by (stream ids as the engine numbers its tensors)."""
    H, I, E, D = cfg.hidden, cfg.inter, cfg.n_experts, cfg.head_dim
    nqkv, hqd = (cfg.n_q_heads + 2 * cfg.n_kv_heads) * D, cfg.n_q_heads * D
    std, seed = cfg.init_std, cfg.seed
    f = lambda stream, n, scale=std: orc.synth_normal_f32(seed, stream, 0, n, scale)  # noqa: E731
    t = {"token_embd.weight": f(_sid(-1, 1), cfg.vocab * H).reshape(cfg.vocab, H),
         "output.weight": f(_sid(-1, 2), cfg.vocab * H).reshape(cfg.vocab, H),
         "output_norm.weight": np.ones(H, np.float32)}
    for l in range(cfg.n_layers):
        t[f"blk.{l}.attn_qkv.weight"] = f(_sid(l, 1), nqkv * H).reshape(nqkv, H)
        t[f"blk.{l}.attn_output.weight"] = f(_sid(l, 2), H * hqd).reshape(H, hqd)
        t[f"blk.{l}.ffn_gate_inp.weight"] = f(_sid(l, 3), E * H).reshape(E, H)
        t[f"blk.{l}.ffn_gate_up_exps.weight"] = np.stack([f(_sid(l, 4, e), 2 * I * H).reshape(2 * I, H) for e in range(E)])
        t[f"blk.{l}.ffn_down_exps.weight"] = np.stack([f(_sid(l, 5, e), H * I).reshape(H, I) for e in range(E)])
        t[f"blk.{l}.attn_sinks.weight"] = f(_sid(l, 6), cfg.n_q_heads, 1.0)
        t[f"blk.{l}.attn_norm.weight"] = np.ones(H, np.float32)
        t[f"blk.{l}.ffn_norm.weight"] = np.ones(H, np.float32)
    return t


def _step(eng, cfg):
    eng.kv_fill_synth()
    slots = [eng.admit(L) for L in TINY_CONTEXTS]
    nxt, mg = eng.step(slots, [1, 5, 2, 3], np.arange(11, dtype=np.int32) * 37 % cfg.vocab)
    return nxt, eng.read_logits()


def test_gguf_checkpoint_reproduces_the_seeded_engine(gpu, tmp_path):
    import eidola_b200 as eb
    cfg = tiny_config()
    tensors = _seeded_tensors(cfg)
    path = tmp_path / "tiny.gguf"
    write_gguf(path, tensors)
    want_next, want_logits = _step(eb.Engine(cfg), cfg)
    cfg2 = tiny_config(seed=12345)  # another seed: everything the step uses must come from the file
    cfg2.seed = 12345
    eng = eb.Engine(cfg2)
    eng.load_gguf(path)
    # the KV stand-in is seeded too: fill it from the first engine's seed by re-creating with that seed
    cfg3 = tiny_config()
    eng3 = eb.Engine(cfg3)
    eng3.load_gguf(path)
    got_next, got_logits = _step(eng3, cfg3)
    assert np.array_equal(got_logits, want_logits) and np.array_equal(got_next, want_next)
    # a BF16 copy of the embeddings and an F16-free file: embeddings are stored as bf16 anyway, so nothing changes
    t2 = dict(tensors)
    t2["token_embd.weight"] = orc.bf16_encode(tensors["token_embd.weight"])
    path2 = tmp_path / "tiny_bf16_embd.gguf"
    write_gguf(path2, t2)
    eng4 = eb.Engine(tiny_config())
    eng4.load_gguf(path2)
    _, logits4 = _step(eng4, cfg)
    assert np.array_equal(logits4, want_logits)
    # the file decides: a zero LM head gives zero logits
    t3 = dict(tensors)
    t3["output.weight"] = np.zeros_like(tensors["output.weight"])
    path3 = tmp_path / "tiny_zero_head.gguf"
    write_gguf(path3, t3)
    eng.load_gguf(path3)
    _, logits0 = _step(eng, cfg2)
    assert not logits0.any()
    # a missing tensor and a wrong shape are refused by name
    t4 = {k: v for k, v in tensors.items() if k != "blk.1.ffn_down_exps.weight"}
    path4 = tmp_path / "tiny_missing.gguf"
    write_gguf(path4, t4)
    with pytest.raises(eb.EbError) as err:
        eb.Engine(tiny_config()).load_gguf(path4)
    assert "blk.1.ffn_down_exps.weight" in str(err.value)
    with pytest.raises(eb.EbError):
        eb.Engine(tiny_config(hidden=1024)).load_gguf(path)
    assert eb.status_read() == 0


def test_block_quantised_checkpoint_loads_as_its_dequantised_values(gpu, tmp_path):
    """Checkpoints as they are distributed keep their linear layers in block formats (8-bit attention and head, 4-bit
    microscaling experts): loading such a file must be loading the fp32 values its blocks stand for."""
    import eidola_b200 as eb
    cfg = tiny_config()
    tensors = _seeded_tensors(cfg)
    blocked, plain = dict(tensors), dict(tensors)
    kinds = {"attn_qkv.weight": "q8_0", "attn_output.weight": "q4_0", "ffn_gate_up_exps.weight": "mxfp4", "ffn_down_exps.weight": "mxfp4"}
    for l in range(cfg.n_layers):
        for suffix, kind in kinds.items():
            b = Blocked(kind, tensors[f"blk.{l}.{suffix}"])
            blocked[f"blk.{l}.{suffix}"], plain[f"blk.{l}.{suffix}"] = b, b.values
    b = Blocked("q8_0", tensors["output.weight"])
    blocked["output.weight"], plain["output.weight"] = b, b.values
    write_gguf(tmp_path / "blocked.gguf", blocked)
    write_gguf(tmp_path / "plain.gguf", plain)
    out = []
    for name in ("blocked.gguf", "plain.gguf"):
        eng = eb.Engine(tiny_config())
        eng.load_gguf(tmp_path / name)
        out.append(_step(eng, cfg))
    assert np.array_equal(out[0][1], out[1][1]) and np.array_equal(out[0][0], out[1][0])
    _, unquantised = _step(eb.Engine(cfg), cfg)
    assert not np.array_equal(out[0][1], unquantised)  # (the 4-bit experts are a different model, as they should be)
    assert eb.status_read() == 0
