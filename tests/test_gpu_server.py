"""GPU: the engine process started the way the reference's client starts its engine -- the `llama-server` argv of
crates/eidola-app-core/src/local_models.rs:1612-1626, stdin/stdout closed, stderr piped -- polled on /health like
local_models.rs:2020-2064 and spoken to over /v1/chat/completions.  Weights: a GGUF checkpoint of the tiny decoder."""
import json
import os
import socket
import subprocess
import sys
import time
import urllib.request
from pathlib import Path

import numpy as np
import pytest

from tests.decoder_cases import tiny_config
from tests.gguf_writer import write_gguf
from tests.test_gpu_loader import _seeded_tensors

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("with_tokenizer,extra_argv", [(False, []), (True, []), (False, ["--spec-lookup", "4"])],
                         ids=["byte_tokens", "file_tokenizer", "lookup_drafts"])
def test_engine_process_honours_the_llama_server_contract(gpu, tmp_path, with_tokenizer, extra_argv):
    cfg = tiny_config()
    model = tmp_path / "tiny.gguf"
    metadata = None
    if with_tokenizer:  # the file's own vocabulary, merges and chat template (tests/test_tokenizer.py trains them)
        from tests.test_tokenizer import TEMPLATE, _train
        tokens, merges, types = _train()
        metadata = {"tokenizer.ggml.model": "gpt2", "tokenizer.ggml.pre": "gpt2", "tokenizer.ggml.tokens": tokens,
                    "tokenizer.ggml.merges": merges, "tokenizer.ggml.token_type": types,
                    "tokenizer.ggml.bos_token_id": np.uint32(tokens.index("<|start|>")),
                    "tokenizer.ggml.eos_token_id": np.uint32(tokens.index("<|eot|>")), "tokenizer.chat_template": TEMPLATE}
    write_gguf(model, _seeded_tensors(cfg), metadata)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    argv = [sys.executable, "-m", "eidola_b200.server", "-m", str(model), "--host", "127.0.0.1", "--port", str(port), "--alias",
            "tiny@local", "-c", "256", "-ngl", "999", "--jinja", "--no-webui", "--shape", "tiny", "--seqs", "4"] + extra_argv
    child = subprocess.Popen(argv, cwd=str(ROOT), stdin=subprocess.DEVNULL, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE,
                             env=dict(os.environ, PYTHONPATH=str(ROOT)))
    url = "http://127.0.0.1:%d" % port
    try:
        deadline = time.time() + 120          # the client allows 300 s and polls every 250 ms
        ready = False
        while time.time() < deadline and child.poll() is None:
            try:
                ready = urllib.request.urlopen(url + "/health", timeout=2).status == 200
            except Exception:
                ready = False
            if ready:
                break
            time.sleep(0.25)
        assert ready, "engine never became healthy: " + (child.stderr.read().decode()[-2000:] if child.poll() is not None else "still loading")
        body = {"model": "tiny@local", "messages": [{"role": "user", "content": "Hello"}], "max_completion_tokens": 12,
                "stream": True, "stream_options": {"include_usage": True}}
        req = urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
        t0 = time.perf_counter()
        raw = urllib.request.urlopen(req, timeout=60).read().decode()
        dt = time.perf_counter() - t0
        chunks, usage, done = 0, None, False
        for event in raw.split("\n\n"):
            for line in event.splitlines():
                if line.startswith("data:"):
                    p = line[5:].lstrip()
                    if p == "[DONE]":
                        done = True
                    else:
                        j = json.loads(p)
                        usage = j.get("usage") or usage
                        chunks += bool(j.get("choices") and "content" in j["choices"][0]["delta"] and j["choices"][0]["delta"]["content"] != "")
        assert done and usage and usage["completion_tokens"] >= 1 and usage["prompt_tokens"] > 10
        # greedy decoding of fixed weights: the same request gives the same reply
        blocking = dict(body, stream=False)
        blocking.pop("stream_options")
        a = json.load(urllib.request.urlopen(urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(blocking).encode()), timeout=60))
        b = json.load(urllib.request.urlopen(urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(blocking).encode()), timeout=60))
        assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"] and a["usage"] == b["usage"]
        # a request with a temperature is drawn on the device: repeatable with its seed, and not the greedy reply
        # (ids above 255 all print as '?' with the byte tokenizer: `return_token_ids` shows what was drawn)
        def ask(extra):
            rq = urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(dict(blocking, return_token_ids=True, **extra)).encode())
            return json.load(urllib.request.urlopen(rq, timeout=60))["choices"][0]["token_ids"]
        g = ask({})
        s1 = ask({"temperature": 1.5, "top_p": 0.95, "seed": 11})
        s2 = ask({"temperature": 1.5, "top_p": 0.95, "seed": 11})
        s3 = ask({"temperature": 1.5, "top_p": 0.95, "seed": 12})
        assert s1 == s2 and len(s1) >= 1
        assert s1 != g or s3 != g, (g, s1, s3)  # 4096-way draws at temperature 1.5: both equal to greedy would be no sampling
        # the next turn of the conversation finds the first turn's pages: only the new tokens are prefilled
        turn2 = dict(blocking, messages=body["messages"] + [{"role": "assistant", "content": a["choices"][0]["message"]["content"]},
                                                            {"role": "user", "content": "And then?"}])
        t2 = json.load(urllib.request.urlopen(urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(turn2).encode()), timeout=60))
        assert t2["usage"]["prompt_tokens_details"]["cached_tokens"] >= 16 and t2["usage"]["completion_tokens"] >= 1
        assert t2["usage"]["prompt_tokens"] > a["usage"]["prompt_tokens"]
        print(f"engine process: healthy, streamed {chunks} content chunks and usage {usage} in {dt * 1e3:.1f} ms; "
              f"second turn: {t2['usage']['prompt_tokens_details']['cached_tokens']} of {t2['usage']['prompt_tokens']} prompt tokens from the cache")
    finally:
        child.kill()                            # the client ends its engine with SIGKILL (kill_on_drop)
        child.wait(timeout=30)


def test_chat_backend_over_the_real_engine(gpu):
    """The `ChatBackend` mirror in front of an in-process engine: blocking and streamed replies agree, usage ends the
    stream, a sampled request is repeatable, and the second turn of the conversation is served from the first one's pages."""
    import eidola_b200 as eb
    from eidola_b200.backend import EidolaB200Backend, ServerError
    from eidola_b200.server import EngineAdapter, EngineLoop
    cfg = tiny_config(max_seqs=4, max_pages_per_seq=24, num_pages=96, max_tokens=128, max_q_len=5)
    loop = EngineLoop(EngineAdapter(eb.Engine(cfg), cfg), context_tokens=256)
    loop.start()
    be = EidolaB200Backend(loop, "tiny@local")
    try:
        req = {"model": "tiny@local", "messages": [{"role": "user", "content": "Hello there, engine"}], "max_completion_tokens": 10}
        a = be.send(req)
        assert a.meta.usage["completion_tokens"] >= 1 and a.meta.usage["prompt_tokens"] > 16
        rx = be.send_stream(dict(req, stream=True))
        events = []
        while True:
            ev = rx.get(timeout=60)
            events.append(ev)
            if isinstance(ev, ServerError) or ev.kind == "done":
                break
        assert events[-1].kind == "done" and events[-1].meta.usage["completion_tokens"] == a.meta.usage["completion_tokens"]
        streamed = "".join(e.chunk["choices"][0]["delta"].get("content", "") for e in events if e.kind == "chunk")
        assert streamed == a.response["choices"][0]["message"]["content"]
        assert events[-1].meta.usage.get("prompt_tokens_details", {}).get("cached_tokens", 0) >= 16  # the first call's pages
        s1 = be.send(dict(req, temperature=1.2, top_p=0.9))
        assert s1.meta.usage["completion_tokens"] >= 1
        with pytest.raises(ServerError):
            be.send(dict(req, n=2))  # not a field of the reference's request type
        assert int(eb.status_read()) == 0
    finally:
        loop.stop.set()
