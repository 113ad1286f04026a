"""HTTP front end of the serving engine.

Endpoints of the continuous-batching design (docs/new/RONN-Continuous-Batching-Branch-Prompt.md:377-395):
``POST /v1/completions`` and ``POST /v1/chat/completions`` (optionally streamed as server-sent events),
``DELETE /v1/requests/{id}``, ``GET /v1/health``, ``GET /v1/metrics`` (Prometheus text).  Prompts are token ids
(``prompt_token_ids``) or, when the app was created with a tokenizer (``serving/tokenizer.py``), text (``prompt`` /
chat ``messages``).  One background thread owns the engine and runs its iteration loop; HTTP
handlers only enqueue requests and wait on per-request events.

Admission goes through ``core.session_manager.RequestAdmission`` (the serving form of the reference's SessionManager
limits, crates/ronn-core/src/session.rs:17-120): a cap on requests in flight, a cap per client and a per-request
deadline; a refused request gets HTTP 429, one that outlives its deadline is cancelled and gets HTTP 504.  Per-request
state (event, token stream, engine record) is dropped when the handler has sent the result, a client that disconnects
from a stream cancels its request, and after ``max_failed_steps`` consecutive failed iterations every unfinished
request is failed instead of being retried for ever.
"""
from __future__ import annotations

import asyncio
import json
import threading
import time
from typing import Dict, List, Optional

from pydantic import BaseModel

from .engine import LLMEngine
from .request import Priority, SamplingParams


class CompletionRequest(BaseModel):
    prompt_token_ids: List[int] = []
    prompt: Optional[str] = None
    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repeat_penalty: float = 1.0
    seed: Optional[int] = None
    stop_token_sequences: List[List[int]] = []
    stream: bool = False
    priority: str = "normal"


class ChatMessage(BaseModel):
    role: str = "user"
    content: str = ""


class ChatRequest(BaseModel):
    messages: List[ChatMessage]
    max_tokens: int = 16
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    repeat_penalty: float = 1.0
    seed: Optional[int] = None
    stop: List[str] = []
    stream: bool = False
    priority: str = "normal"


class EngineLoop:
    """Owns an ``LLMEngine`` on one thread: submissions and cancellations are queued and applied between iterations."""

    def __init__(self, engine: LLMEngine, idle_sleep: float = 0.001, max_failed_steps: int = 5):
        self.engine = engine
        self.idle_sleep = idle_sleep
        self.max_failed_steps = max_failed_steps
        self._failed_in_a_row = 0
        self._lock = threading.Lock()
        self._pending: List[tuple] = []
        self._cancel: List[int] = []
        self._events: Dict[int, threading.Event] = {}
        self._streams: Dict[int, List[int]] = {}
        self._released: set = set()
        self._next_id = 1
        self._stop = threading.Event()
        self.error: Optional[str] = None
        self._thread = threading.Thread(target=self._run, daemon=True, name="ronn-engine-loop")
        engine.on_token = self._on_token
        self._thread.start()

    def _on_token(self, req, tok: int) -> None:
        with self._lock:
            self._streams.setdefault(req.id, []).append(tok)

    def submit(self, tokens: List[int], params: SamplingParams, priority: Priority = Priority.NORMAL) -> int:
        with self._lock:
            rid = self._next_id
            self._next_id += 1
            self._events[rid] = threading.Event()
            self._pending.append((rid, tokens, params, priority))
        return rid

    def cancel(self, rid: int) -> None:
        with self._lock:
            self._cancel.append(rid)

    def wait(self, rid: int, timeout: Optional[float] = None) -> bool:
        ev = self._events.get(rid)
        return ev.wait(timeout) if ev is not None else False

    def drain_stream(self, rid: int) -> List[int]:
        with self._lock:
            toks = self._streams.get(rid, [])
            if toks:
                self._streams[rid] = []
            return toks

    def result(self, rid: int):
        """The request record (finished or not), or None when it is unknown."""
        return self.engine.requests.get(rid)

    def release(self, rid: int) -> None:
        """The handler has read the result: drop the event, the token stream and the engine's record.  A request that
        is still running (client went away) is cancelled first."""
        r = self.engine.requests.get(rid)
        if r is None or not r.finished:
            self.cancel(rid)
            with self._lock:
                self._released.add(rid)
            return
        with self._lock:
            self._events.pop(rid, None)
            self._streams.pop(rid, None)
        self.engine.release(rid)

    def tracked(self) -> int:
        with self._lock:
            return len(self._events)

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=5)

    def _run(self) -> None:
        eng = self.engine
        while not self._stop.is_set():
            with self._lock:
                pending, self._pending = self._pending, []
                cancels, self._cancel = self._cancel, []
            for rid, toks, params, prio in pending:
                try:
                    eng.add_request(toks, params, prio, request_id=rid)
                except Exception as e:               # rejected at admission: report through the request record
                    from .request import FinishReason, Request
                    r = Request(rid, toks, params, prio)
                    r.finish_reason, r.error, r._final_tokens = FinishReason.ERROR, str(e), []
                    eng.requests[rid] = r
                    self._events[rid].set()
            for rid in cancels:
                eng.cancel(rid)
                self._signal(rid)
            if not eng.has_unfinished():
                time.sleep(self.idle_sleep)
                continue
            try:
                out = eng.step()
                self._failed_in_a_row = 0
                for r in out:                        # only the requests of this step can have finished in it
                    if r.finished:
                        self._signal(r.id)
            except Exception as e:                   # failed step: requests were re-queued by the engine
                self.error = str(e)
                self._failed_in_a_row += 1
                if self._failed_in_a_row >= self.max_failed_steps:
                    for rid in eng.fail_unfinished(f"{self._failed_in_a_row} consecutive iterations failed: {e}"):
                        self._signal(rid)
                    self._failed_in_a_row = 0
                else:
                    time.sleep(0.01)

    def _signal(self, rid: int) -> None:
        """A request reached its end: wake its handler, or clean up at once when the handler has already gone."""
        with self._lock:
            ev = self._events.get(rid)
            gone = rid in self._released
            if gone:
                self._released.discard(rid)
                self._events.pop(rid, None)
                self._streams.pop(rid, None)
        if gone:
            self.engine.release(rid)
        elif ev is not None:
            ev.set()


def create_app(engine: LLMEngine, tokenizer=None, admission=None):
    from fastapi import FastAPI, HTTPException, Request as HttpRequest
    from fastapi.responses import PlainTextResponse, StreamingResponse

    from ..core.session_manager import RequestAdmission

    app = FastAPI(title="ronn_b200")
    loop = EngineLoop(engine)
    app.state.loop = loop
    adm = admission or RequestAdmission(max_in_flight=4 * engine.cfg.max_num_seqs)
    app.state.admission = adm

    def _admit(http: HttpRequest):
        client = http.client.host if http is not None and http.client else "local"
        ticket = adm.acquire(client)
        if ticket is None:
            raise HTTPException(status_code=429, detail="too many requests in flight")
        return ticket

    async def _until_done(rid: int, ticket, step: float = 0.05) -> None:
        """Wait for the request; past the admission deadline it is cancelled and the client gets 504."""
        while not await _wait(rid, step):
            if adm.expired(ticket):
                loop.release(rid)
                adm.release(ticket, error=True)
                raise HTTPException(status_code=504, detail="request exceeded the server's deadline")

    def _result(rid: int):
        r = loop.result(rid)
        if r is None:
            raise HTTPException(status_code=410, detail="request record is gone")
        if r.error:
            raise HTTPException(status_code=400 if r.finish_reason is None or not r.output_tokens else 500, detail=r.error)
        return {"id": rid, "object": "text_completion",
                "choices": [{"index": 0, "token_ids": r.output_tokens,
                             "text": tokenizer.decode(r.output_tokens) if tokenizer is not None else None,
                             "finish_reason": r.finish_reason.value if r.finish_reason else None}],
                "usage": {"prompt_tokens": len(r.prompt_tokens), "completion_tokens": len(r.output_tokens)}}

    def _priority(name: str) -> Priority:
        try:
            return Priority[name.upper()]
        except KeyError:
            raise HTTPException(status_code=400, detail=f"unknown priority '{name}'") from None

    async def _wait(rid: int, step: float) -> bool:
        return await asyncio.get_running_loop().run_in_executor(None, loop.wait, rid, step)

    @app.post("/v1/chat/completions")
    async def chat_completions(req: ChatRequest, http: HttpRequest = None):
        if tokenizer is None:
            raise HTTPException(status_code=400, detail="the server was started without a tokenizer")
        if not req.messages:
            raise HTTPException(status_code=400, detail="messages must not be empty")
        from .tokenizer import render_chat
        prompt = tokenizer.encode(render_chat([m.model_dump() for m in req.messages]))
        params = SamplingParams(max_new_tokens=req.max_tokens, temperature=req.temperature, top_k=req.top_k,
                                top_p=req.top_p, repeat_penalty=req.repeat_penalty, seed=req.seed,
                                stop_sequences=[tokenizer.encode(s_) for s_ in req.stop if s_])
        prio = _priority(req.priority)
        ticket = _admit(http)
        rid = loop.submit(prompt, params, prio)
        if not req.stream:
            await _until_done(rid, ticket)
            try:
                r = loop.result(rid)
                if r is None or r.error:
                    raise HTTPException(status_code=400, detail=r.error if r is not None else "request record is gone")
                return {"id": rid, "object": "chat.completion",
                        "choices": [{"index": 0, "message": {"role": "assistant", "content": tokenizer.decode(r.output_tokens)},
                                     "token_ids": r.output_tokens,
                                     "finish_reason": r.finish_reason.value if r.finish_reason else None}],
                        "usage": {"prompt_tokens": len(r.prompt_tokens), "completion_tokens": len(r.output_tokens)}}
            finally:
                loop.release(rid)
                adm.release(ticket)

        async def events():
            sent: List[int] = []
            text = ""
            try:
                while True:
                    done = await _wait(rid, 0.01)
                    new = loop.drain_stream(rid)
                    if new:
                        sent.extend(new)
                        full = tokenizer.decode(sent)            # decode the whole prefix: a character may span tokens
                        delta, text = full[len(text):], full
                        chunk = {"id": rid, "object": "chat.completion.chunk",
                                 "choices": [{"index": 0, "delta": {"content": delta}, "token_ids": new}]}
                        yield f"data: {json.dumps(chunk)}\n\n"
                    if done or adm.expired(ticket):
                        r = loop.result(rid)
                        fin = {"id": rid, "object": "chat.completion.chunk",
                               "choices": [{"index": 0, "delta": {},
                                            "finish_reason": (r.finish_reason.value if r is not None and r.finish_reason
                                                              else ("deadline" if not done else None))}]}
                        yield f"data: {json.dumps(fin)}\n\n"
                        yield "data: [DONE]\n\n"
                        return
            finally:                                             # also runs when the client disconnects mid-stream
                loop.release(rid)
                adm.release(ticket)
        return StreamingResponse(events(), media_type="text/event-stream")

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest, http: HttpRequest = None):
        if not req.prompt_token_ids and req.prompt:
            if tokenizer is None:
                raise HTTPException(status_code=400, detail="text prompts need a tokenizer; send prompt_token_ids")
            req.prompt_token_ids = tokenizer.encode(req.prompt)
        if not req.prompt_token_ids:
            raise HTTPException(status_code=400, detail="prompt_token_ids must not be empty")
        params = SamplingParams(max_new_tokens=req.max_tokens, temperature=req.temperature, top_k=req.top_k,
                                top_p=req.top_p, repeat_penalty=req.repeat_penalty, seed=req.seed,
                                stop_sequences=req.stop_token_sequences)
        prio = _priority(req.priority)
        ticket = _admit(http)
        rid = loop.submit(list(req.prompt_token_ids), params, prio)
        if not req.stream:
            await _until_done(rid, ticket)
            try:
                return _result(rid)
            finally:
                loop.release(rid)
                adm.release(ticket)

        async def events():
            try:
                while True:
                    done = await _wait(rid, 0.01)
                    for tok in loop.drain_stream(rid):
                        yield f"data: {json.dumps({'id': rid, 'token_id': tok})}\n\n"
                    if done or adm.expired(ticket):
                        r = loop.result(rid)
                        reason = r.finish_reason.value if r is not None and r.finish_reason else ("deadline" if not done else None)
                        yield f"data: {json.dumps({'id': rid, 'finish_reason': reason})}\n\n"
                        yield "data: [DONE]\n\n"
                        return
            finally:                                             # also runs when the client disconnects mid-stream
                loop.release(rid)
                adm.release(ticket)
        return StreamingResponse(events(), media_type="text/event-stream")

    @app.delete("/v1/requests/{rid}")
    async def cancel(rid: int):
        if rid not in engine.requests and rid not in loop._events:
            raise HTTPException(status_code=404, detail="unknown request")
        loop.cancel(rid)
        return {"id": rid, "cancelled": True}

    @app.get("/v1/health")
    async def health():
        return {"status": "ok" if loop.error is None else "degraded", "last_error": loop.error,
                "waiting": engine.sched.num_waiting, "running": engine.sched.num_running,
                "free_blocks": engine.sched.num_free_blocks, "tracked_requests": loop.tracked(),
                "admission": adm.snapshot()}

    @app.get("/v1/metrics", response_class=PlainTextResponse)
    async def metrics():
        return engine.metrics.prometheus()

    return app
