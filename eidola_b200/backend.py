"""The reference server's `ChatBackend` over an in-process engine loop.

The reference's server reaches its model through one trait (crates/eidola-server/src/backend.rs:87-108):

    send(&ChatCompletionRequest)        -> Result<BackendResponse, ServerError>
    list_models()                       -> Result<ModelsResponse, ServerError>
    send_stream(&ChatCompletionRequest) -> Result<mpsc::Receiver<Result<BackendStreamEvent, ServerError>>, ServerError>

whose one implementation forwards to a remote provider over HTTPS (backend.rs:421-615).  This module is the same
interface in front of libeidola_b200: same method names, argument meaning and error behaviour, in Python because the
engine loop, tokenizer and chat template around the C ABI are Python here and there is no Rust toolchain (the Rust
`impl ChatBackend` that talks to the engine process over loopback is in INTEGRATION.md).  What carries over:

* the request is the reference's strict type (types.rs:10-66, `deny_unknown_fields`): an unknown field is an error;
* `send_stream` returns a BOUNDED channel of 32 events (backend.rs:597-610): `Chunk(chunk, instant)` ... `Done(meta,
  instant)`, every event stamped when the reader took it from the engine, not when the consumer received it, so that a
  slow consumer does not stretch the timings (backend.rs:62-78);
* `usage` is mandatory in the final metadata: refunds are computed from it (backend.rs:487-498); a stream that ends
  without it ends with an error, never with a `Done`;
* errors are the two kinds the handlers tell apart: the backend cannot be reached / is not ready (`BackendUnavailable`,
  the handlers' 503) and the backend answered with a failure (`BackendError`, 502).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field

from .server import EngineLoop, make_request

REQUEST_FIELDS = {"model", "messages", "max_completion_tokens", "temperature", "top_p", "stream", "stream_options", "stop", "tools",
                  "tool_choice"}


class ServerError(Exception):
    """kind: "InvalidRequest" (400), "BackendUnavailable" (503) or "BackendError" (502)."""

    def __init__(self, kind: str, message: str):
        super().__init__("%s: %s" % (kind, message))
        self.kind, self.message = kind, message


@dataclass
class BackendMeta:
    provider: str
    chat_id: str | None
    backend_model: str
    tee_type: str | None          # None: this engine does not run inside an enclave
    usage: dict | None            # {prompt_tokens, completion_tokens, total_tokens}


@dataclass
class BackendResponse:
    response: dict                # the OpenAI-format completion
    meta: BackendMeta


@dataclass
class BackendStreamEvent:
    kind: str                     # "chunk" | "done"
    instant: float                # time.monotonic() when the reader took it from the engine
    chunk: dict | None = None     # kind == "chunk": a chat.completion.chunk
    meta: BackendMeta | None = None
    finish_reason: str | None = field(default=None)


class EidolaB200Backend:
    """`ChatBackend` for an EngineLoop that is already running (the loop owns the engine handle)."""

    provider = "eidola_b200"
    abandon_after = 30.0  # seconds a full channel may stay untouched before its receiver counts as dropped

    def __init__(self, loop: EngineLoop, model: str):
        self.loop, self.model = loop, model

    # ---- the trait
    def list_models(self) -> dict:
        if not self.loop.ready.is_set():
            raise ServerError("BackendUnavailable", "the engine is still loading")
        return {"object": "list", "data": [{"id": self.model, "object": "model", "owned_by": self.provider}]}

    def send(self, request: dict) -> BackendResponse:
        req, rid = self._submit(request)
        text, usage = bytearray(), None
        while True:
            kind, val = req.out.get()
            if kind == "bytes":
                text += val
            elif kind == "done":
                usage = dict(val)
                break
            elif kind == "error":
                raise ServerError("BackendError", str(val))
        finish = usage.pop("finish_reason")
        response = {"id": rid, "object": "chat.completion", "created": int(time.time()), "model": self.model,
                    "choices": [{"index": 0, "finish_reason": finish,
                                 "message": {"role": "assistant", "content": text.decode("utf-8", errors="replace")}}],
                    "usage": usage}
        return BackendResponse(response, BackendMeta(self.provider, rid, self.model, None, usage))

    def send_stream(self, request: dict) -> "queue.Queue":
        """A bounded queue of BackendStreamEvent (or ServerError, after which nothing follows).  Errors before the first
        event are raised here, as the trait returns them before handing out the receiver."""
        import codecs
        req, rid = self._submit(request)
        out: queue.Queue = queue.Queue(maxsize=32)
        base = {"id": rid, "object": "chat.completion.chunk", "created": int(time.time()), "model": self.model}

        def put(ev) -> bool:
            """False when the consumer has not taken an event for `abandon_after` seconds: the receiver is taken for
            dropped (the reference's sender sees a closed channel then), the sequence is ended and the reader leaves."""
            try:
                out.put(ev, timeout=self.abandon_after)
                return True
            except queue.Full:
                req.cancelled = True
                return False

        def reader():
            utf8 = codecs.getincrementaldecoder("utf-8")(errors="replace")
            while True:
                kind, val = req.out.get()
                now = time.monotonic()  # the stamp of the moment the engine produced it
                if kind == "bytes":
                    text = utf8.decode(val)
                    if text and not put(BackendStreamEvent("chunk", now, dict(base, choices=[{"index": 0, "delta": {"content": text}, "finish_reason": None}]))):
                        return
                elif kind == "done":
                    usage = dict(val)
                    finish = usage.pop("finish_reason")
                    tail = utf8.decode(b"", final=True)
                    if tail:
                        put(BackendStreamEvent("chunk", now, dict(base, choices=[{"index": 0, "delta": {"content": tail}, "finish_reason": None}])))
                    put(BackendStreamEvent("chunk", now, dict(base, choices=[{"index": 0, "delta": {}, "finish_reason": finish}])))
                    put(BackendStreamEvent("done", now, meta=BackendMeta(self.provider, rid, self.model, None, usage), finish_reason=finish))
                    return
                elif kind == "error":
                    put(ServerError("BackendError", str(val)))  # no Done: a stream without usage is a failed stream
                    return

        threading.Thread(target=reader, daemon=True).start()
        return out

    # ---- shared
    def _submit(self, request: dict):
        if not isinstance(request, dict):
            raise ServerError("InvalidRequest", "the request must be an object")
        unknown = sorted(set(request) - REQUEST_FIELDS)
        if unknown:  # deny_unknown_fields
            raise ServerError("InvalidRequest", "unknown field `%s`, expected one of %s" % (unknown[0], ", ".join("`%s`" % f for f in sorted(REQUEST_FIELDS))))
        if not isinstance(request.get("model"), str):
            raise ServerError("InvalidRequest", "missing field `model`")
        if not self.loop.ready.is_set() or not self.loop.is_alive():
            raise ServerError("BackendUnavailable", "the engine is not running")
        try:
            req = make_request(self.loop.tokenizer, request)
        except ValueError as e:
            raise ServerError("InvalidRequest", str(e)) from None
        self.loop.submit(req)
        return req, "chatcmpl-%x" % id(req)
