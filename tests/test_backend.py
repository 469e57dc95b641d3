"""CPU: the `ChatBackend` mirror (eidola_b200/backend.py) against a scripted engine -- the happy paths and the scripted
failures the reference's own harness plays (crates/eidola-app-core/tests/chat_harness/mod.rs:100-108: a stream that
aborts in the middle, a backend that drops the request before any response)."""
import queue

import numpy as np
import pytest

from eidola_b200.backend import EidolaB200Backend, ServerError
from eidola_b200.server import ByteTokenizer, EngineLoop
from tests.test_server_contract import ScriptedEngine

REQ = {"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_completion_tokens": 6}


def _backend(engine=None):
    eng = engine or ScriptedEngine()
    loop = EngineLoop(eng, context_tokens=512)
    loop.start()
    assert loop.ready.wait(5)
    return eng, loop, EidolaB200Backend(loop, "tiny@local")


def _drain(rx):
    events = []
    while True:
        ev = rx.get(timeout=10)
        events.append(ev)
        if isinstance(ev, ServerError) or ev.kind == "done":
            return events


def test_send_list_models_and_a_stream_that_ends_with_usage():
    eng, loop, be = _backend()
    try:
        assert be.list_models()["data"][0]["id"] == "tiny@local"
        r = be.send(REQ)
        prompt = ByteTokenizer.template(REQ["messages"])
        assert r.meta.usage == {"prompt_tokens": len(prompt), "completion_tokens": 6, "total_tokens": len(prompt) + 6}
        assert r.meta.backend_model == "tiny@local" and r.meta.tee_type is None and r.meta.provider == "eidola_b200"
        assert r.response["usage"] == r.meta.usage and r.response["choices"][0]["finish_reason"] == "length"
        want = bytes((prompt[-1] + 1 + i) % 256 for i in range(6)).decode("utf-8", errors="replace")
        assert r.response["choices"][0]["message"]["content"] == want
        rx = be.send_stream(dict(REQ, stream=True, stream_options={"include_usage": True}))
        assert rx.maxsize == 32                                   # bounded, as the reference's channel is
        events = _drain(rx)
        assert events[-1].kind == "done" and events[-1].meta.usage == r.meta.usage   # usage is mandatory at the end
        chunks = [e for e in events if e.kind == "chunk"]
        assert "".join(c.chunk["choices"][0]["delta"].get("content", "") for c in chunks) == want
        assert chunks[-1].chunk["choices"][0]["finish_reason"] == "length"
        stamps = [e.instant for e in events]
        assert stamps == sorted(stamps)                          # stamped where they were produced, in order
        assert sorted(eng.free) == [0, 1, 2, 3]
    finally:
        loop.stop.set()


def test_the_request_type_is_strict():
    eng, loop, be = _backend()
    try:
        for bad, needle in [(dict(REQ, frequency_penalty=1.0), "unknown field `frequency_penalty`"), ({"messages": REQ["messages"]}, "`model`"),
                            (dict(REQ, messages=[]), "messages"), (dict(REQ, temperature=3.0), "temperature"), (dict(REQ, stop=[1]), "stop")]:
            with pytest.raises(ServerError) as err:
                be.send(bad)
            assert err.value.kind == "InvalidRequest" and needle in err.value.message
        assert not [c for c in eng.calls if c[0] == "prefill"]     # nothing reached the engine
    finally:
        loop.stop.set()


def test_a_stream_that_aborts_in_the_middle_ends_with_an_error_and_no_done():
    class MidAbort(ScriptedEngine):
        def step(self, slots, q_lens, tokens):
            if len([c for c in self.calls if c[0] == "step"]) >= 3:
                raise RuntimeError("connection reset by peer")
            return super().step(slots, q_lens, tokens)

    eng, loop, be = _backend(MidAbort())
    try:
        events = _drain(be.send_stream(dict(REQ, max_completion_tokens=40, stream=True)))
        assert isinstance(events[-1], ServerError) and events[-1].kind == "BackendError" and "reset" in events[-1].message
        assert 1 <= len([e for e in events if not isinstance(e, ServerError) and e.kind == "chunk"]) <= 5
        assert not any(not isinstance(e, ServerError) and e.kind == "done" for e in events)   # no usage, no Done
        assert sorted(eng.free) == [0, 1, 2, 3]                   # the slot went back
        with pytest.raises(ServerError) as err:                    # the blocking call surfaces the same failure
            be.send(dict(REQ, max_completion_tokens=40))
        assert err.value.kind == "BackendError"
    finally:
        loop.stop.set()


def test_a_backend_that_drops_the_request_before_any_response():
    class DropBefore(ScriptedEngine):
        def prefill(self, slots, prompts):
            raise RuntimeError("engine went away")

    eng, loop, be = _backend(DropBefore())
    try:
        events = _drain(be.send_stream(dict(REQ, stream=True)))
        assert len(events) == 1 and isinstance(events[0], ServerError) and events[0].kind == "BackendError"
    finally:
        loop.stop.set()
    # an engine loop that is not running at all: unavailable, before anything is queued
    dead = EngineLoop(ScriptedEngine(), context_tokens=512)
    be2 = EidolaB200Backend(dead, "m")
    for call in (lambda: be2.send(REQ), lambda: be2.send_stream(REQ), be2.list_models):
        with pytest.raises(ServerError) as err:
            call()
        assert err.value.kind == "BackendUnavailable"
    assert dead.inbox.qsize() == 0


def test_a_receiver_that_is_dropped_ends_the_sequence():
    eng, loop, be = _backend()
    be.abandon_after = 0.2
    try:
        rx = be.send_stream(dict(REQ, max_completion_tokens=400, stream=True))  # far more events than the channel holds
        import time
        deadline = time.time() + 10
        while time.time() < deadline and len(eng.free) < 4:
            time.sleep(0.05)                                       # nobody reads rx
        assert sorted(eng.free) == [0, 1, 2, 3] and rx.full()
        assert len([c for c in eng.calls if c[0] == "step"]) < 300
    finally:
        loop.stop.set()
