"""CPU: the engine process's HTTP contract against a scripted engine, read the way the reference's client reads it.

The reference tests its engine boundary with a scripted peer on the other side of HTTP
(crates/eidola-app-core/tests/chat_harness/mod.rs); here the roles are swapped: the server under test is ours, the
engine behind it is scripted (next token = last token + 1), and the test plays the client: `/health` must answer 200,
a blocking completion must carry `choices[0].message.content` and `usage`, a streamed one must arrive as `data:` events
with `choices[0].delta.content`, a `usage` event when `stream_options.include_usage` is set, and `[DONE]`
(crates/eidola-app-core/src/lib.rs:7232-7340)."""
import json
import threading
import time
import urllib.request

import numpy as np

from eidola_b200.server import ByteTokenizer, EngineLoop, serve


class ScriptedEngine:
    """Counts up from the last prompt byte; records what the loop asked of it."""
    max_seqs = 4

    def __init__(self):
        self.free = list(range(self.max_seqs))
        self.calls = []

    def admit_evicting(self, context_len):
        return self.free.pop(0), []

    def prefill(self, slots, prompts):
        self.calls.append(("prefill", list(slots), [len(p) for p in prompts]))
        return (np.array([(int(p[-1]) + 1) % 256 or 1 for p in prompts], np.int32),)

    def step(self, slots, q_lens, tokens):
        import time
        time.sleep(0.003)  # a decode step takes milliseconds: requests that arrive meanwhile join the next one
        self.calls.append(("step", list(slots)))
        return np.array([(t + 1) % 256 or 1 for t in tokens], np.int32), None

    def sampling(self, slot, temperature, top_p, seed):
        self.calls.append(("sampling", slot, temperature, top_p, seed))

    def release(self, slot):
        self.free.append(slot)


def _start():
    eng = ScriptedEngine()
    loop = EngineLoop(eng, context_tokens=512)
    httpd = serve(loop, "127.0.0.1", 0, "test-model")
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    return eng, loop, httpd, "http://127.0.0.1:%d" % httpd.server_address[1]


def _post(url, body):
    req = urllib.request.Request(url + "/v1/chat/completions", data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    return urllib.request.urlopen(req, timeout=30)


def test_health_then_blocking_and_streamed_completions():
    eng, loop, httpd, url = _start()
    try:
        try:
            urllib.request.urlopen(url + "/health", timeout=5)
            assert False, "healthy before the engine loop is up"
        except urllib.error.HTTPError as e:
            assert e.code == 503                                  # the socket answers while the model loads
        loop.start()
        assert loop.ready.wait(5)
        assert json.load(urllib.request.urlopen(url + "/health", timeout=5)) == {"status": "ok"}
        body = {"model": "test-model", "messages": [{"role": "user", "content": "hi"}], "max_completion_tokens": 5}
        out = json.load(_post(url, body))
        prompt = ByteTokenizer.template(body["messages"])
        want = bytes((prompt[-1] + 1 + i) % 256 for i in range(5)).decode("utf-8", errors="replace")
        assert out["choices"][0]["message"]["content"] == want and out["choices"][0]["finish_reason"] == "length"
        assert out["usage"] == {"prompt_tokens": len(prompt), "completion_tokens": 5, "total_tokens": len(prompt) + 5}
        # streamed, parsed as the client does: data: lines, usage, choices[0].delta.content, [DONE]
        resp = _post(url, dict(body, stream=True, stream_options={"include_usage": True}))
        assert resp.headers["Content-Type"] == "text/event-stream"
        text, usage, finished = "", None, False
        for event in resp.read().decode().split("\n\n"):
            for line in event.splitlines():
                if not line.startswith("data:"):
                    continue
                payload = line[5:].lstrip()
                if payload == "[DONE]":
                    finished = True
                    continue
                j = json.loads(payload)
                usage = j.get("usage") or usage
                if j.get("choices"):
                    text += j["choices"][0]["delta"].get("content") or ""
        assert finished and text == want and usage["completion_tokens"] == 5 and usage["prompt_tokens"] == len(prompt)
        assert eng.free and sorted(eng.free) == [0, 1, 2, 3]      # every sequence was released
    finally:
        loop.stop.set()
        httpd.shutdown()


def test_requests_that_overlap_share_decode_steps_and_bad_requests_are_refused():
    eng, loop, httpd, url = _start()
    loop.start()
    try:
        results = {}

        def client(i):
            body = {"model": "m", "messages": [{"role": "user", "content": "q%d" % i}], "max_completion_tokens": 40}
            results[i] = json.load(_post(url, body))

        ts = [threading.Thread(target=client, args=(i,)) for i in range(3)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(30)
        assert all(results[i]["usage"]["completion_tokens"] == 40 for i in range(3))
        steps = [c for c in eng.calls if c[0] == "step"]
        assert any(len(c[1]) > 1 for c in steps)                   # continuous batching: several sequences in one step
        assert len(steps) < 3 * 40
        for bad in (b"not json", json.dumps({"model": "m"}).encode(), json.dumps({"messages": []}).encode()):
            try:
                urllib.request.urlopen(urllib.request.Request(url + "/v1/chat/completions", data=bad), timeout=5)
                assert False
            except urllib.error.HTTPError as e:
                assert e.code == 400 and "error" in json.load(e)
        # sampling fields reach the engine before the sequence's first step; greedy requests never touch them
        assert not any(c[0] == "sampling" for c in eng.calls)
        json.load(_post(url, {"messages": [{"role": "user", "content": "s"}], "max_completion_tokens": 3, "temperature": 0.7,
                              "top_p": 0.9, "seed": 5}))
        samp = [c for c in eng.calls if c[0] == "sampling"]
        assert len(samp) == 1 and samp[0][2:] == (0.7, 0.9, 5)
        assert eng.calls.index(samp[0]) < max(i for i, c in enumerate(eng.calls) if c[0] == "prefill")
        for bad_field in ({"temperature": 2.5}, {"temperature": -1}, {"top_p": 1.5}, {"temperature": "hot"}):
            try:
                _post(url, dict({"messages": [{"role": "user", "content": "s"}]}, **bad_field))
                assert False
            except urllib.error.HTTPError as e:
                assert e.code == 400
        try:  # more context than the engine was started with: refused with a message, like the reference's -c cap
            _post(url, {"messages": [{"role": "user", "content": "x" * 600}], "max_completion_tokens": 10})
            assert False
        except urllib.error.HTTPError as e:
            assert e.code == 500 and "context" in json.load(e)["error"]["message"]
    finally:
        loop.stop.set()
        httpd.shutdown()


def test_a_file_tokenizer_serves_templates_and_streams_whole_characters():
    """With the vocabulary and chat template of a model file the prompt is the template's rendering, and streamed text
    leaves only when the bytes of a character are complete (tokens may end inside a UTF-8 sequence)."""
    from tests.test_tokenizer import _tok
    tok = _tok()
    reply = tok.encode("é東 ok")

    class Replaying(ScriptedEngine):
        def prefill(self, slots, prompts):
            self.calls.append(("prefill", list(slots), [list(map(int, p)) for p in prompts]))
            self.pos = {s: 1 for s in slots}
            return (np.array([reply[0]] * len(slots), np.int32),)

        def step(self, slots, q_lens, tokens):
            out = []
            for s in slots:
                out.append(reply[self.pos[s]] if self.pos[s] < len(reply) else tok.eos)
                self.pos[s] += 1
            return np.array(out, np.int32), None

    eng = Replaying()
    loop = EngineLoop(eng, context_tokens=512, tokenizer=tok)
    httpd = serve(loop, "127.0.0.1", 0, "test-model")
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = "http://127.0.0.1:%d" % httpd.server_address[1]
    loop.start()
    try:
        msgs = [{"role": "user", "content": "hello fox"}]
        out = json.load(_post(url, {"messages": msgs, "max_completion_tokens": 64}))
        assert out["choices"][0]["message"]["content"] == "é東 ok" and out["choices"][0]["finish_reason"] == "stop"
        sent = [c for c in eng.calls if c[0] == "prefill"][0][2][0]
        assert sent == tok.template(msgs)
        assert tok.decode(sent, skip_control=False).endswith("<|start|>user<|message|>hello fox<|end|><|start|>assistant<|message|>")
        resp = _post(url, {"messages": msgs, "max_completion_tokens": 64, "stream": True})
        pieces = []
        for event in resp.read().decode().split("\n\n"):
            for line in event.splitlines():
                if line.startswith("data:") and line[5:].strip() != "[DONE]":
                    j = json.loads(line[5:])
                    if j.get("choices") and j["choices"][0]["delta"].get("content"):
                        pieces.append(j["choices"][0]["delta"]["content"])
        assert "".join(pieces) == "é東 ok" and "�" not in "".join(pieces)
        assert len(pieces) < len(reply)  # the bytes of é and 東 arrived over several tokens and left as whole characters
    finally:
        loop.stop.set()
        httpd.shutdown()


def _replaying_server(tok, reply_text):
    reply = tok.encode(reply_text)

    class Replaying(ScriptedEngine):
        def prefill(self, slots, prompts):
            self.calls.append(("prefill", list(slots), [list(map(int, p)) for p in prompts]))
            self.pos = {s: 1 for s in slots}
            return (np.array([reply[0]] * len(slots), np.int32),)

        def step(self, slots, q_lens, tokens):
            out = []
            for s in slots:
                out.append(reply[self.pos[s]] if self.pos[s] < len(reply) else tok.eos)
                self.pos[s] += 1
            return np.array(out, np.int32), None

    eng = Replaying()
    loop = EngineLoop(eng, context_tokens=512, tokenizer=tok)
    httpd = serve(loop, "127.0.0.1", 0, "test-model")
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    loop.start()
    return eng, loop, httpd, "http://127.0.0.1:%d" % httpd.server_address[1]


def _stream_text(resp):
    pieces, finish = [], None
    for event in resp.read().decode().split("\n\n"):
        for line in event.splitlines():
            if line.startswith("data:") and line[5:].strip() != "[DONE]":
                j = json.loads(line[5:])
                if j.get("choices"):
                    finish = j["choices"][0].get("finish_reason") or finish
                    if j["choices"][0]["delta"].get("content"):
                        pieces.append(j["choices"][0]["delta"]["content"])
    return pieces, finish


def test_stop_sequences_end_the_text_before_their_first_occurrence():
    """`stop` of the reference server's request type (crates/eidola-server/src/types.rs): up to four strings; the reply
    ends before the first of them, nothing of it leaks into a stream, and the sequence is released."""
    from tests.test_tokenizer import _tok
    tok = _tok()
    eng, loop, httpd, url = _replaying_server(tok, "hello world, the fox END and more")
    try:
        msgs = [{"role": "user", "content": "hi"}]
        out = json.load(_post(url, {"messages": msgs, "max_completion_tokens": 64, "stop": ["END", " wor"]}))
        assert out["choices"][0]["message"]["content"] == "hello" and out["choices"][0]["finish_reason"] == "stop"
        assert out["usage"]["completion_tokens"] < len(tok.encode("hello world, the fox END and more"))
        out = json.load(_post(url, {"messages": msgs, "max_completion_tokens": 64, "stop": "END"}))
        assert out["choices"][0]["message"]["content"] == "hello world, the fox "
        pieces, finish = _stream_text(_post(url, {"messages": msgs, "max_completion_tokens": 64, "stop": ["END"], "stream": True}))
        assert "".join(pieces) == "hello world, the fox " and finish == "stop" and not any("E" in p for p in pieces)
        # a stop sequence that never comes: the whole reply, ended by the end-of-sequence token
        out = json.load(_post(url, {"messages": msgs, "max_completion_tokens": 64, "stop": ["ENDE", "xyz"]}))
        assert out["choices"][0]["message"]["content"] == "hello world, the fox END and more" and out["choices"][0]["finish_reason"] == "stop"
        out = json.load(_post(url, {"messages": msgs, "max_completion_tokens": 3}))
        assert out["choices"][0]["finish_reason"] == "length" and out["usage"]["completion_tokens"] == 3
        for bad in ({"stop": ["a", "b", "c", "d", "e"]}, {"stop": 5}, {"stop": [1]}):
            try:
                _post(url, dict({"messages": msgs}, **bad))
                assert False
            except urllib.error.HTTPError as e:
                assert e.code == 400
        assert sorted(eng.free) == [0, 1, 2, 3]
    finally:
        loop.stop.set()
        httpd.shutdown()


def test_tools_reach_the_chat_template():
    from tests.test_tokenizer import TEMPLATE, _tok
    tok = _tok()
    tok.chat_template = "{% if tools %}tools {{ tools | length }} {{ tools[0]['function']['name'] }} {% endif %}" + TEMPLATE
    eng, loop, httpd, url = _replaying_server(tok, "ok")
    try:
        tools = [{"type": "function", "function": {"name": "lookup", "parameters": {"type": "object"}}}]
        json.load(_post(url, {"messages": [{"role": "user", "content": "hi"}], "max_completion_tokens": 4, "tools": tools, "tool_choice": "auto"}))
        sent = [c for c in eng.calls if c[0] == "prefill"][-1][2][0]
        assert tok.decode(sent, skip_control=False).startswith("tools 1 lookup ")
    finally:
        loop.stop.set()
        httpd.shutdown()


def test_a_client_that_goes_away_frees_its_sequence_and_an_engine_error_frees_them_all():
    import socket
    eng, loop, httpd, url = _start()
    loop.start()
    try:
        # a streaming client that hangs up after the first bytes: the sequence ends long before max_completion_tokens
        host, port = httpd.server_address
        body = json.dumps({"messages": [{"role": "user", "content": "x"}], "max_completion_tokens": 400, "stream": True}).encode()
        with socket.create_connection((host, port)) as sk:
            sk.sendall(b"POST /v1/chat/completions HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: %d\r\n\r\n" % len(body) + body)
            sk.recv(256)
            sk.setsockopt(socket.SOL_SOCKET, socket.SO_LINGER, __import__("struct").pack("ii", 1, 0))  # close with a reset
        deadline = time.time() + 10
        while time.time() < deadline and len(eng.free) < 4:
            time.sleep(0.02)
        assert sorted(eng.free) == [0, 1, 2, 3]
        assert len([c for c in eng.calls if c[0] == "step"]) < 380  # (400 tokens were asked for)
        # an engine that fails a step: every request in flight gets the message, every slot goes back
        real_step = eng.step

        def failing(slots, q_lens, tokens):
            raise RuntimeError("device lost")
        eng.step = failing
        try:
            _post(url, {"messages": [{"role": "user", "content": "y"}], "max_completion_tokens": 8})
            assert False
        except urllib.error.HTTPError as e:
            assert e.code == 500 and "device lost" in json.load(e)["error"]["message"]
        eng.step = real_step
        assert sorted(eng.free) == [0, 1, 2, 3]
        out = json.load(_post(url, {"messages": [{"role": "user", "content": "z"}], "max_completion_tokens": 4}))
        assert out["usage"]["completion_tokens"] == 4  # the loop lives on
    finally:
        loop.stop.set()
        httpd.shutdown()


def test_the_next_turn_of_a_conversation_prefills_only_what_is_new():
    """A chat client sends the whole conversation with every turn: the pages of the finished turn stay in the pool and the
    next request that starts with the same tokens is cut back to the common prefix and prefills the rest."""
    class Caching(ScriptedEngine):
        def __init__(self):
            super().__init__()
            self.len = {}

        def admit_evicting(self, context_len):
            if not self.free:  # evict the least recently admitted idle sequence
                victim = next(s for s in self.len if not self.pinned.get(s))
                self.len.pop(victim)
                self.free.append(victim)
                self.calls.append(("evict", victim))
                slot = self.free.pop(0)
                self.len[slot], self.pinned[slot] = 0, True
                return slot, [victim]
            slot = self.free.pop(0)
            self.len[slot] = 0
            self.pinned = getattr(self, "pinned", {})
            self.pinned[slot] = True
            return slot, []

        def prefill(self, slots, prompts):
            for s, p in zip(slots, prompts):
                self.len[s] += len(p)
            return super().prefill(slots, prompts)

        def step(self, slots, q_lens, tokens):
            for s in slots:
                self.len[s] += 1
            return super().step(slots, q_lens, tokens)

        def truncate(self, slot, new_len):
            assert 0 < new_len <= self.len[slot]
            self.calls.append(("truncate", slot, new_len))
            self.len[slot] = new_len

        def pin(self, slot, pinned):
            self.pinned[slot] = pinned

        def release(self, slot):
            self.len.pop(slot, None)
            super().release(slot)

    eng = Caching()
    eng.pinned = {}
    loop = EngineLoop(eng, context_tokens=2048)
    httpd = serve(loop, "127.0.0.1", 0, "test-model")
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = "http://127.0.0.1:%d" % httpd.server_address[1]
    loop.start()
    try:
        turn1 = [{"role": "user", "content": "tell me about foxes, briefly please"}]
        a = json.load(_post(url, {"messages": turn1, "max_completion_tokens": 6}))
        assert "prompt_tokens_details" not in a["usage"]
        p1 = ByteTokenizer.template(turn1)
        turn2 = turn1 + [{"role": "assistant", "content": a["choices"][0]["message"]["content"]}, {"role": "user", "content": "and dogs?"}]
        b = json.load(_post(url, {"messages": turn2, "max_completion_tokens": 6}))
        p2 = ByteTokenizer.template(turn2)
        cached = b["usage"]["prompt_tokens_details"]["cached_tokens"]
        # the pages hold the first prompt and the five reply tokens that were fed back (the sixth never ran); the second
        # prompt repeats all of it
        assert p2[:len(p1)] == p1
        assert cached == len(p1) + 5 and b["usage"]["prompt_tokens"] == len(p2)
        pre = [c for c in eng.calls if c[0] == "prefill"]
        assert pre[0][2] == [len(p1)] and pre[1][2] == [len(p2) - cached]  # only the new tokens ran
        assert ("truncate", pre[1][1][0], cached) in eng.calls and pre[1][1] == pre[0][1]  # the same slot, cut back
        assert loop.stats["prefix_hits"] == 1 and loop.stats["prefix_tokens"] == cached
        # an unrelated conversation gets a sequence of its own; idle ones are evicted when the slots run out
        for i in range(5):
            json.load(_post(url, {"messages": [{"role": "user", "content": "%d: something else entirely, long enough" % i}], "max_completion_tokens": 2}))
        assert any(c[0] == "evict" for c in eng.calls)
        assert all(s in eng.len for s in loop.idle) and len(loop.idle) <= eng.max_seqs
    finally:
        loop.stop.set()
        httpd.shutdown()


def test_drafts_from_the_sequence_itself_are_verified_in_the_step_and_change_nothing_but_the_step_count():
    """Lookup drafts: when the last two tokens occurred before, the tokens that followed are fed along and verified in the
    same step.  The reply is the one plain decoding gives; it only takes fewer steps when the text repeats."""
    class Cyclic(ScriptedEngine):
        """The next token of t is t % 7 + 65: the text runs in a cycle of seven letters."""
        def __init__(self):
            super().__init__()
            self.len, self.max_len = {}, {}

        def admit_evicting(self, context_len):
            slot, ev = super().admit_evicting(context_len)
            self.len[slot] = 0
            return slot, ev

        def prefill(self, slots, prompts):
            for s, p in zip(slots, prompts):
                self.len[s] += len(p)
            self.calls.append(("prefill", list(slots), [len(p) for p in prompts]))
            return (np.array([int(p[-1]) % 7 + 65 for p in prompts], np.int32),)

        def step(self, slots, q_lens, tokens):
            self.calls.append(("step", list(slots), list(q_lens)))
            for s, q in zip(slots, q_lens):
                self.len[s] += q
            return np.array([int(t) % 7 + 65 for t in tokens], np.int32), None

        def truncate(self, slot, new_len):
            assert new_len <= self.len[slot]
            self.calls.append(("truncate", slot, new_len))
            self.len[slot] = new_len

        def pin(self, slot, pinned):
            pass

    replies, steps = [], []
    for spec in (0, 4):
        eng = Cyclic()
        loop = EngineLoop(eng, context_tokens=512)
        loop.spec = spec
        httpd = serve(loop, "127.0.0.1", 0, "test-model")
        threading.Thread(target=httpd.serve_forever, daemon=True).start()
        loop.start()
        try:
            url = "http://127.0.0.1:%d" % httpd.server_address[1]
            out = json.load(_post(url, {"messages": [{"role": "user", "content": "go"}], "max_completion_tokens": 40, "return_token_ids": True}))
            replies.append(out["choices"][0]["token_ids"])
            steps.append(len([c for c in eng.calls if c[0] == "step"]))
            assert out["usage"]["completion_tokens"] == 40 and out["choices"][0]["finish_reason"] == "length"
            if spec:
                qs = [c[2][0] for c in eng.calls if c[0] == "step"]
                assert max(qs) == 5 and loop.stats["drafts_accepted"] >= 20
                # the engine's sequence ends where the text ends: prompt + 39 tokens that ran (the 40th never did)
                prompt_len = [c for c in eng.calls if c[0] == "prefill"][0][2][0]
                assert eng.len[0] == prompt_len + 39
            # a sampled request is never drafted for
            json.load(_post(url, {"messages": [{"role": "user", "content": "go"}], "max_completion_tokens": 30, "temperature": 0.5}))
            assert all(c[2] == [1] for c in eng.calls[-25:] if c[0] == "step")
        finally:
            loop.stop.set()
            httpd.shutdown()
    assert replies[0] == replies[1] and len(replies[0]) == 40
    assert steps[1] < steps[0] // 2, steps


def test_idle_conversations_give_their_pages_back_when_live_ones_need_them():
    class Pool(ScriptedEngine):
        """16 tokens per page, 16 pages: a finished conversation's pages stay held until somebody releases it."""
        pages = 16

        def __init__(self):
            super().__init__()
            self.len = {}

        def admit_evicting(self, context_len):
            slot, ev = super().admit_evicting(context_len)
            self.len[slot] = 0
            return slot, ev

        def _grow(self, slot, n):
            need = -(-(self.len[slot] + n) // 16) - -(-self.len[slot] // 16)
            if need > self.free_pages():
                raise RuntimeError("out of pages")
            self.len[slot] += n

        def free_pages(self):
            return self.pages - sum(-(-n // 16) for n in self.len.values())

        def prefill(self, slots, prompts):
            for s, p in zip(slots, prompts):
                self._grow(s, len(p))
            return super().prefill(slots, prompts)

        def step(self, slots, q_lens, tokens):
            for s, q in zip(slots, q_lens):
                self._grow(s, q)
            return super().step(slots, q_lens, tokens)

        def truncate(self, slot, new_len):
            self.len[slot] = new_len

        def pin(self, slot, pinned):
            pass

        def release(self, slot):
            self.len.pop(slot, None)
            super().release(slot)

    eng = Pool()
    loop = EngineLoop(eng, context_tokens=512)
    httpd = serve(loop, "127.0.0.1", 0, "test-model")
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = "http://127.0.0.1:%d" % httpd.server_address[1]
    loop.start()
    try:
        # three conversations of 4 pages each stay idle (4 pages free); a fourth that needs 6 must still run to its end
        for i in range(3):
            out = json.load(_post(url, {"messages": [{"role": "user", "content": chr(65 + i) * 26}], "max_completion_tokens": 8}))  # no common prefix
            assert out["usage"]["completion_tokens"] == 8
        assert len(loop.idle) == 3 and eng.free_pages() == 4
        out = json.load(_post(url, {"messages": [{"role": "user", "content": "x" * 30}], "max_completion_tokens": 40}))
        assert out["usage"]["completion_tokens"] == 40 and out["choices"][0]["finish_reason"] == "length"
        assert len(loop.idle) < 4 and loop.stats["evicted"] >= 1
    finally:
        loop.stop.set()
        httpd.shutdown()
