"""An engine process that honours the `llama-server` contract of the reference's client.

The reference's client starts its local engine as a child process

    <engine> -m <model.gguf> --host 127.0.0.1 --port P --alias <model id> -c 8192 -ngl 999 --jinja --no-webui

(crates/eidola-app-core/src/local_models.rs:1612-1626), waits for `GET /health` to answer 200 within 300 s
(local_models.rs:2020-2064), then posts `{model, messages, max_completion_tokens, [stream, stream_options]}` to
`/v1/chat/completions` (crates/eidola-common/src/lib.rs:116-139) and reads either one JSON body or server-sent events
whose `data:` lines carry `choices[0].delta.content`, a final `usage` object and `[DONE]`
(crates/eidola-app-core/src/lib.rs:7232-7340).  This module is that process for libeidola_b200:

    python -m eidola_b200.server -m model.gguf --host 127.0.0.1 --port 8080 --alias gpt-oss-20b -c 8192 -ngl 999 --jinja --no-webui

One engine thread owns the engine handle (one thread per handle, as the reference's supervisor owns its child,
local_models.rs:1633-1638) and runs continuous batching: requests that arrive are admitted (idle sequences are evicted,
least recently used first, when the page pool is full), their prompts are prefilled together, and every iteration
decodes one token for every live sequence.  HTTP threads only enqueue requests and drain per-request token queues.

The reference contains no tokenizer, chat template or sampler (they live inside the third-party engine).  Here: a GGUF
file that carries a byte-level BPE vocabulary (tokenizer.ggml.*) and a chat template is served with them
(eidola_b200/tokenizer.py); a file without gets the identity on UTF-8 bytes (ids 0..255) with a plain `<|role|>` template.  Decoding is greedy unless
the request carries `temperature` > 0 (then `top_p` and `seed` apply: eb_engine_seq_sampling, drawn on the device).  With
the random-init weights the replies are noise -- the process contract, the batching and the timings are what is real.
"""
from __future__ import annotations

import argparse
import codecs
import json
import queue
import sys
import threading
import time
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

import numpy as np


class ByteTokenizer:
    """Token id = UTF-8 byte.  Ids at or above 256 (a model with a larger vocabulary produces them) print as '?'."""
    eos = 0

    @staticmethod
    def encode(text: str) -> list[int]:
        return list(text.encode("utf-8"))

    @staticmethod
    def template(messages) -> list[int]:
        out: list[int] = []
        for m in messages:
            content = m.get("content") or ""
            if isinstance(content, list):  # OpenAI content parts: keep the text parts
                content = "".join(p.get("text", "") for p in content if isinstance(p, dict))
            out += ByteTokenizer.encode("<|%s|>\n%s\n" % (m.get("role", "user"), content))
        out += ByteTokenizer.encode("<|assistant|>\n")
        return [b if b != 0 else 32 for b in out] or [32]

    @staticmethod
    def token_bytes(i: int) -> bytes:
        return bytes([i if 0 < i < 256 else 63])

    @staticmethod
    def decode(ids) -> str:
        return bytes((i if 0 < i < 256 else 63) for i in ids).decode("utf-8", errors="replace")


class Request:
    def __init__(self, prompt_ids, max_tokens, temperature=0.0, top_p=1.0, seed=0, stop=()):
        self.prompt_ids, self.max_tokens = prompt_ids, max_tokens
        self.temperature, self.top_p, self.seed = temperature, top_p, seed  # temperature 0: greedy
        self.stop = [s.encode("utf-8") for s in stop if s]  # generation ends before the first of these appears in the text
        self.text = bytearray()   # bytes generated so far
        self.sent = 0             # how many of them have left as ("bytes", ...) events
        self.finish = "length"
        self.cancelled = False    # set by the HTTP thread when the client has gone away: the loop ends the sequence
        self.history = []         # the tokens whose K and V are in the sequence's pages
        self.ngram = {}           # (a, b) -> index of the token that followed the last occurrence of "a b" (draft lookup)
        self.indexed = 0          # history tokens the index covers
        self.cached_tokens = 0    # how many of the prompt's tokens were found in an idle sequence's pages
        # ("token", id) and ("bytes", text bytes) ... ("done", usage) | ("error", message)
        self.out: "queue.Queue[tuple[str, object]]" = queue.Queue()
        self.slot = None
        self.generated = 0
        self.t_arrive = time.perf_counter()


def make_request(tokenizer, body: dict) -> Request:
    """A request body (the fields of the reference server's ChatCompletionRequest, crates/eidola-server/src/types.rs:10-66,
    plus `seed` and `max_tokens`) -> Request; ValueError with the message for a 400 otherwise."""
    messages = body.get("messages")
    if not (isinstance(messages, list) and messages):
        raise ValueError("body must be JSON with a non-empty `messages` array")
    max_tokens = int(body.get("max_completion_tokens") or body.get("max_tokens") or 256)
    # `temperature` (0..2) and `top_p`: absent or 0 is greedy.  `seed` makes a sampled reply repeatable.
    try:
        temperature = float(body.get("temperature") or 0.0)
        top_p = float(body["top_p"]) if body.get("top_p") is not None else 1.0
        seed = int(body["seed"]) & (2**64 - 1) if body.get("seed") is not None else int(time.time_ns()) & (2**64 - 1)
        assert 0.0 <= temperature <= 2.0 and 0.0 <= top_p <= 1.0
    except Exception:
        raise ValueError("`temperature` must lie in [0, 2], `top_p` in [0, 1], `seed` be an integer") from None
    stop = body.get("stop")  # a string or up to 4 of them
    stop = [stop] if isinstance(stop, str) else (stop or [])
    if not (isinstance(stop, list) and len(stop) <= 4 and all(isinstance(x, str) for x in stop)):
        raise ValueError("`stop` must be a string or up to 4 strings")
    try:
        # `tools` / `tool_choice` are for the model's chat template to spell out; nothing here executes a tool
        if body.get("tools") and getattr(tokenizer, "chat_template", None):
            prompt_ids = tokenizer.template(messages, tools=body["tools"], tool_choice=body.get("tool_choice"))
        else:
            prompt_ids = tokenizer.template(messages)
    except Exception as e:  # a chat template may refuse a conversation (roles out of order, ...)
        raise ValueError("chat template: %s" % e) from None
    return Request(prompt_ids, max(1, max_tokens), temperature, top_p, seed, stop)


class EngineLoop(threading.Thread):
    """The thread that owns the engine.  `engine` needs admit_evicting(context_len) -> (slot, evicted), prefill(slots,
    prompts) -> (first_tokens, ...), step(slots, q_lens, tokens) -> (next, margins), release(slot), and max_seqs /
    context_tokens attributes: eidola_b200.host.Engine behind a thin adapter, or a scripted fake in the CPU tests."""

    def __init__(self, engine, context_tokens: int, tokenizer=ByteTokenizer):
        super().__init__(daemon=True)
        self.engine, self.context_tokens = engine, context_tokens
        self.tokenizer = tokenizer  # template(messages) -> ids, token_bytes(id), decode(ids), eos
        self.inbox: "queue.Queue[Request]" = queue.Queue()
        self.live: dict[int, Request] = {}
        self.last: dict[int, int] = {}
        self.ready = threading.Event()
        self.stop = threading.Event()
        self.stats = {"steps": 0, "prefill_tokens": 0, "generated": 0, "evicted": 0, "prefix_hits": 0, "prefix_tokens": 0}
        # Finished sequences stay in the page pool, unpinned, with the tokens their pages hold: a chat client sends the
        # whole conversation again with every turn, and the next turn then prefills only what is new.  The engine evicts
        # them, least recently used first, when it needs their pages (eb_engine_seq_admit_evicting).
        self.idle: dict[int, list[int]] = {}
        self.min_prefix = 16      # shorter common prefixes are not worth a sequence of their own
        # Draft tokens without a draft model: when the last two tokens occurred before in the sequence, the tokens that
        # followed them then are proposed now and verified in the same step (q_len = 1 + drafts: the verify kernels); the
        # accepted ones cost no step of their own.  Greedy sequences only; 0 = off.
        self.spec = 0

    def submit(self, req: Request) -> None:
        self.inbox.put(req)

    def _admit_new(self) -> None:
        fresh = []
        while len(self.live) + len(fresh) < self.engine.max_seqs:
            try:
                req = self.inbox.get(block=not self.live and not fresh, timeout=0.05)
            except queue.Empty:
                break
            if len(req.prompt_ids) + req.max_tokens > self.context_tokens:
                req.out.put(("error", "the request needs %d tokens of context, the engine was started with -c %d"
                             % (len(req.prompt_ids) + req.max_tokens, self.context_tokens)))
                continue
            slot = self._reuse_idle(req)
            if slot is None:
                try:
                    slot, evicted = self.engine.admit_evicting(0)
                except Exception as e:  # pool exhausted by live sequences: refuse, nothing changed
                    req.out.put(("error", "no room for another sequence: %s" % e))
                    continue
                self.stats["evicted"] += len(evicted)
                for s in evicted:
                    self.idle.pop(s, None)
                if req.temperature > 0:  # from the first generated token on (the prefill step draws it)
                    self.engine.sampling(slot, req.temperature, req.top_p, req.seed)
            req.slot = slot
            fresh.append(req)
        if fresh:
            self._make_room(sum((len(r.prompt_ids) - r.cached_tokens) // 16 + 2 for r in fresh))
            try:
                first = self.engine.prefill([r.slot for r in fresh],
                                            [np.asarray(r.prompt_ids[r.cached_tokens:], np.int32) for r in fresh])[0]
            except Exception as e:  # the requests that were being admitted hear of it too, and their slots go back
                for r in fresh:
                    r.out.put(("error", "engine: %s" % e))
                    try:
                        self.engine.release(r.slot)
                    except Exception:
                        pass
                raise
            for r, tok in zip(fresh, first):
                self.stats["prefill_tokens"] += len(r.prompt_ids) - r.cached_tokens
                r.history = list(r.prompt_ids)
                r.engine_len = len(r.history)
                self.live[r.slot] = r
                self._deliver(r, int(tok))

    def _reuse_idle(self, req: Request):
        """The idle sequence whose pages hold the longest prefix of the request's prompt, cut back to that prefix and
        pinned again; None when no idle sequence shares min_prefix tokens (or the engine cannot cut sequences)."""
        if not self.idle or not hasattr(self.engine, "truncate"):
            return None
        best, best_len = None, 0
        for slot, held in self.idle.items():
            n, lim = 0, min(len(held), len(req.prompt_ids) - 1)  # at least one token is left to run: its logits are needed
            while n < lim and held[n] == req.prompt_ids[n]:
                n += 1
            if n > best_len:
                best, best_len = slot, n
        if best is None or best_len < self.min_prefix:
            return None
        del self.idle[best]
        try:
            self.engine.truncate(best, best_len)
            self.engine.pin(best, True)
            self.engine.sampling(best, req.temperature if req.temperature > 0 else 0.0, req.top_p, req.seed)
        except Exception:  # (for instance a page ring that no longer holds the window before the cut): start afresh
            try:
                self.engine.release(best)
            except Exception:
                pass
            return None
        req.cached_tokens = best_len
        self.stats["prefix_hits"] += 1
        self.stats["prefix_tokens"] += best_len
        return best

    def _deliver(self, r: Request, tok: int) -> None:
        r.generated += 1
        self.stats["generated"] += 1
        eos = tok == self.tokenizer.eos
        done = r.generated >= r.max_tokens or eos or r.cancelled
        if eos:
            r.finish = "stop"
        else:
            r.out.put(("token", tok))
            r.text += self.tokenizer.token_bytes(tok)
        # stop sequences: the text ends before the first occurrence; bytes that could still turn out to be the start of
        # one are held back until the next token decides
        upto = len(r.text)
        if r.stop:
            hits = [p for p in (r.text.find(s, max(0, r.sent - len(s) + 1)) for s in r.stop) if p >= 0]
            if hits:
                upto, done, r.finish = min(hits), True, "stop"
            elif not done:
                for s in r.stop:
                    for k in range(min(len(s) - 1, len(r.text) - r.sent), 0, -1):
                        if r.text.endswith(s[:k]):
                            upto = min(upto, len(r.text) - k)
                            break
        if upto > r.sent:
            r.out.put(("bytes", bytes(r.text[r.sent:upto])))
            r.sent = upto
        if done:
            usage = {"prompt_tokens": len(r.prompt_ids), "completion_tokens": r.generated,
                     "total_tokens": len(r.prompt_ids) + r.generated, "finish_reason": r.finish}
            if r.cached_tokens:
                usage["prompt_tokens_details"] = {"cached_tokens": r.cached_tokens}
            r.out.put(("done", usage))
            self._settle(r)
            if hasattr(self.engine, "truncate") and len(r.history) >= self.min_prefix:
                self.engine.pin(r.slot, False)  # stays in the pool for the conversation's next turn, evictable
                self.idle[r.slot] = r.history
            else:
                self.engine.release(r.slot)
            self.live.pop(r.slot, None)
            self.last.pop(r.slot, None)
        else:
            self.last[r.slot] = tok

    def _make_room(self, pages: int) -> None:
        """Idle sequences give their pages back, longest idle first, until `pages` are free: a live sequence that grows
        never fails for pages that a finished conversation is only keeping in case it returns."""
        if not self.idle or not hasattr(self.engine, "free_pages"):
            return
        while self.idle and self.engine.free_pages() < pages:
            slot = next(iter(self.idle))  # dicts keep insertion order: the one that has been idle longest
            del self.idle[slot]
            self.engine.release(slot)
            self.stats["evicted"] += 1

    def _settle(self, r: Request) -> None:
        """Cut the engine's sequence back to the tokens that count (rejected drafts ran through the layers too)."""
        if getattr(r, "engine_len", 0) > len(r.history):
            self.engine.truncate(r.slot, len(r.history))
        r.engine_len = len(r.history)

    def _drafts(self, r: Request, last: int) -> list[int]:
        """Up to self.spec tokens that followed the previous occurrence of (second to last token, last token)."""
        if self.spec <= 0 or r.temperature > 0 or not r.history or not hasattr(self.engine, "truncate"):
            return []
        h = r.history
        for i in range(max(r.indexed, 2), len(h)):  # index "h[i-2] h[i-1]" -> i as the history grows
            r.ngram[(h[i - 2], h[i - 1])] = i
        r.indexed = len(h)
        at = r.ngram.get((h[-1], last))
        if at is None:
            return []
        room = min(self.spec, r.max_tokens - r.generated - 1, self.context_tokens - len(h) - 2)
        return [int(t) for t in h[at:at + max(0, room)]]

    def run(self) -> None:
        self.ready.set()
        while not self.stop.is_set():
            try:
                self._admit_new()
                if not self.live:
                    continue
                slots = sorted(self.live)
                fed = {s: [self.last[s]] + self._drafts(self.live[s], self.last[s]) for s in slots}
                self._make_room(sum(len(x) for x in fed.values()) // 16 + len(slots))
                nxt, _ = self.engine.step(slots, [len(fed[s]) for s in slots], [t for s in slots for t in fed[s]])
                self.stats["steps"] += 1
                row = 0
                for s in slots:
                    r, x = self.live[s], fed[s]
                    y = [int(t) for t in nxt[row:row + len(x)]]
                    row += len(x)
                    r.engine_len = len(r.history) + len(x)
                    # y[i] follows x[i]; draft x[i + 1] stands if it is what the model says after x[i]
                    for i in range(len(x)):
                        r.history.append(x[i])  # its K and V are in the pages and it counts
                        self._deliver(r, y[i])
                        if s not in self.live or i + 1 == len(x) or x[i + 1] != y[i]:
                            break
                        self.stats["drafts_accepted"] = self.stats.get("drafts_accepted", 0) + 1
                    if s in self.live:
                        self._settle(r)
            except Exception as e:  # an engine error ends every request in flight with a message, not a hang
                for r in list(self.live.values()):
                    r.out.put(("error", "engine: %s" % e))
                    try:
                        self.engine.release(r.slot)  # the pages go back even when the step failed
                    except Exception:
                        pass
                self.live.clear()
                self.last.clear()


class EngineAdapter:
    """eidola_b200.host.Engine with the three calls the loop needs."""

    def __init__(self, eng, cfg):
        self.eng, self.max_seqs = eng, cfg.max_seqs

    def admit_evicting(self, context_len):
        slot, evicted = self.eng.admit_evicting(context_len)
        self.eng.pin(slot, True)  # a sequence that is being served is never a victim
        return slot, evicted

    def prefill(self, slots, prompts):
        return self.eng.prefill(slots, prompts)

    def step(self, slots, q_lens, tokens):
        return self.eng.step(slots, q_lens, tokens)

    def sampling(self, slot, temperature, top_p, seed):
        self.eng.sampling(slot, temperature, top_p, seed)

    def truncate(self, slot, new_len):
        self.eng.truncate(slot, new_len)

    def pin(self, slot, pinned):
        self.eng.pin(slot, pinned)

    def free_pages(self):
        return self.eng.free_pages()

    def release(self, slot):
        self.eng.release(slot)


def make_handler(loop: EngineLoop, alias: str):
    class Handler(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, fmt, *args):  # stderr stays for failures: the client keeps its last 30 lines
            pass

        def _json(self, code, obj):
            body = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(body)))
            self.end_headers()
            self.wfile.write(body)

        def do_GET(self):
            if self.path.split("?")[0] == "/health":
                if loop.ready.is_set():
                    self._json(200, {"status": "ok"})
                else:
                    self._json(503, {"error": {"message": "loading model", "type": "unavailable_error", "code": 503}})
            elif self.path.split("?")[0] == "/v1/models":
                self._json(200, {"object": "list", "data": [{"id": alias, "object": "model", "owned_by": "eidola_b200"}]})
            else:
                self._json(404, {"error": {"message": "not found", "type": "not_found_error", "code": 404}})

        def do_POST(self):
            if self.path.split("?")[0] != "/v1/chat/completions":
                return self._json(404, {"error": {"message": "not found", "type": "not_found_error", "code": 404}})
            try:
                n = int(self.headers.get("Content-Length", "0"))
                body = json.loads(self.rfile.read(n) or b"{}")
                assert isinstance(body, dict) and isinstance(body.get("messages"), list) and body["messages"]
            except Exception:
                return self._json(400, {"error": {"message": "body must be JSON with a non-empty `messages` array",
                                                  "type": "invalid_request_error", "code": 400}})
            if not loop.ready.is_set():
                return self._json(503, {"error": {"message": "loading model", "type": "unavailable_error", "code": 503}})
            stream = bool(body.get("stream"))
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))
            try:
                req = make_request(loop.tokenizer, body)
            except ValueError as e:
                return self._json(400, {"error": {"message": str(e), "type": "invalid_request_error", "code": 400}})
            loop.submit(req)
            rid, created = "chatcmpl-%x" % id(req), int(time.time())
            base = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": body.get("model") or alias}
            if not stream:
                toks, text, usage = [], bytearray(), None
                while True:
                    kind, val = req.out.get()
                    if kind == "token":
                        toks.append(val)
                    elif kind == "bytes":
                        text += val
                    elif kind == "done":
                        usage = dict(val)
                        break
                    else:
                        return self._json(500, {"error": {"message": str(val), "type": "server_error", "code": 500}})
                finish = usage.pop("finish_reason")
                return self._json(200, {"id": rid, "object": "chat.completion", "created": created, "model": base["model"],
                                        "choices": [{"index": 0, "finish_reason": finish,
                                                     "message": {"role": "assistant", "content": text.decode("utf-8", errors="replace")},
                                                     **({"token_ids": toks} if body.get("return_token_ids") else {})}],
                                        "usage": usage})
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Connection", "close")
            self.end_headers()

            def event(obj):
                self.wfile.write(b"data: " + (obj if isinstance(obj, bytes) else json.dumps(obj).encode()) + b"\n\n")
                self.wfile.flush()

            # a token may end inside a UTF-8 sequence: text leaves when its bytes are complete
            utf8 = codecs.getincrementaldecoder("utf-8")(errors="replace")
            try:
                event(dict(base, choices=[{"index": 0, "delta": {"role": "assistant", "content": ""}, "finish_reason": None}]))
                while True:
                    kind, val = req.out.get()
                    if kind == "token":
                        continue
                    if kind == "bytes":
                        text = utf8.decode(val)
                        if text:
                            event(dict(base, choices=[{"index": 0, "delta": {"content": text}, "finish_reason": None}]))
                    elif kind == "done":
                        tail = utf8.decode(b"", final=True)
                        if tail:
                            event(dict(base, choices=[{"index": 0, "delta": {"content": tail}, "finish_reason": None}]))
                        usage = dict(val)
                        event(dict(base, choices=[{"index": 0, "delta": {}, "finish_reason": usage.pop("finish_reason")}]))
                        if include_usage:
                            event(dict(base, choices=[], usage=usage))
                        event(b"[DONE]")
                        break
                    else:
                        event({"error": {"message": str(val), "type": "server_error", "code": 500}})
                        break
            except (BrokenPipeError, ConnectionResetError):
                req.cancelled = True  # the client went away: the loop ends the sequence at its next token and releases it
            self.close_connection = True

    return Handler


def serve(loop: EngineLoop, host: str, port: int, alias: str) -> ThreadingHTTPServer:
    httpd = ThreadingHTTPServer((host, port), make_handler(loop, alias))
    httpd.daemon_threads = True
    return httpd


def build_engine(args):
    import eidola_b200 as eb
    from eidola_b200.capi import make_config
    eb.capi.call("eb_device_set", eb.capi.c_i32(args.device))
    ctx = args.ctx
    pages_per_seq = ctx // 16 + 2
    shapes = {
        "tiny": dict(n_layers=2, hidden=512, n_q_heads=8, n_kv_heads=2, n_experts=8, inter=512, vocab=4096),
        "20b": dict(n_layers=24, hidden=2880, n_q_heads=64, n_kv_heads=8, n_experts=32, inter=2880, vocab=201088),
    }[args.shape]
    dims = dict(window=128, top_k=4, **shapes)
    if args.model and args.model.endswith(".gguf") and not args.random_init:
        from .tokenizer import shape_from_gguf
        dims.update(shape_from_gguf(args.model))  # the file's own dimensions, where its metadata states them
    cfg = make_config(num_pages=args.seqs * pages_per_seq, max_seqs=args.seqs, max_pages_per_seq=pages_per_seq,
                      max_tokens=max(args.seqs * 6, min(ctx, 2048)), max_q_len=6, seed=args.seed, **dims)
    eng = eb.Engine(cfg)
    if args.model and args.model.endswith(".gguf") and not args.random_init:
        eng.load_gguf(args.model)
    return EngineAdapter(eng, cfg)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("-m", "--model", default="")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8080)
    ap.add_argument("--alias", default="eidola-b200")
    ap.add_argument("-c", "--ctx", type=int, default=8192)
    ap.add_argument("-ngl", "--n-gpu-layers", type=int, default=999)  # everything runs on the GPU; accepted for the contract
    ap.add_argument("--jinja", action="store_true")                   # the file's chat template is always used when it has one
    ap.add_argument("--no-webui", action="store_true")
    ap.add_argument("--shape", default="20b", choices=["tiny", "20b"], help="decoder shape when the weights are random-init")
    ap.add_argument("--random-init", action="store_true", help="ignore -m and use the seeded weights")
    ap.add_argument("--seqs", type=int, default=64, help="concurrent sequences")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--spec-lookup", type=int, default=0,
                    help="draft up to this many tokens per step from the sequence's own earlier text and verify them in the step (0 = off)")
    ap.add_argument("--device", type=int, default=0)
    args, unknown = ap.parse_known_args(argv)
    if unknown:  # other llama-server options a caller may pass: said once on stderr, then ignored
        print("eidola_b200.server: ignoring options it does not know: %s" % " ".join(unknown), file=sys.stderr, flush=True)
    holder = {}
    loop = EngineLoop(None, args.ctx)
    loop.spec = max(0, min(args.spec_lookup, 5))  # the engine is created with max_q_len 6: one token and five drafts
    httpd = serve(loop, args.host, args.port, args.alias)   # the socket answers 503 on /health while the model loads
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        loop.engine = build_engine(args)
        if args.model and args.model.endswith(".gguf") and not args.random_init:
            from .tokenizer import BpeTokenizer
            tok = BpeTokenizer.from_gguf(args.model)  # the file's vocabulary, merges and chat template, when it has them
            if tok is not None:
                loop.tokenizer = tok
    except Exception as e:  # the client shows the last lines of stderr when its engine exits
        print("eidola_b200.server: cannot start the engine: %s" % e, file=sys.stderr, flush=True)
        return 1
    loop.start()
    holder["loop"] = loop
    try:
        while loop.is_alive():
            time.sleep(0.2)
    except KeyboardInterrupt:
        pass
    loop.stop.set()
    httpd.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
