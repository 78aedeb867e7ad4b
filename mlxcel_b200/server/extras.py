"""Server features around the core routes: CORS, request logging, live settings, the Responses
store (TTL, background jobs, cancel, compaction), resumable stream sessions and in-flight control.

Reference counterparts: src/server/cors.rs (llama-server b10621 CORS behaviour), logging.rs
(destination / format / verbosity / redaction), runtime_settings*.rs + routes/settings.rs
(authenticated live settings, opt-in), responses_store.rs (LRU + TTL), routes/responses_background*.rs,
responses_compaction*, stream_session.rs (ring buffers of SSE frames, resumed by conversation id
and last event id), and the ``/v1/chat/completions/control`` route of src/server/app.rs:284.
"""
from __future__ import annotations

import asyncio
import contextvars
import json
import logging
import sys
import time
import uuid
from collections import OrderedDict, deque

from fastapi import Request
from fastapi.responses import JSONResponse, Response, StreamingResponse

# per-request header values the generation path reads (priority lane, conversation id)
REQUEST_CTX: contextvars.ContextVar[dict] = contextvars.ContextVar("mlxcel_request_ctx", default={})

LOG = logging.getLogger("mlxcel_b200.server")


# ----------------------------------------------------------------------------- logging
class _JsonFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        d = {"ts": round(record.created, 3), "level": record.levelname.lower(), "msg": record.getMessage()}
        d.update(getattr(record, "fields", {}) or {})
        return json.dumps(d, ensure_ascii=False)


class LogControl:
    """Destination (stderr or a file), format (text | json), verbosity (0 errors … 3 debug) and
    redaction of request bodies, changeable while the server runs."""

    LEVELS = {0: logging.ERROR, 1: logging.WARNING, 2: logging.INFO, 3: logging.DEBUG}

    def __init__(self, dest: str | None = None, fmt: str = "text", verbosity: int = 1, redact: bool = True):
        self.dest, self.fmt, self.verbosity, self.redact = dest, fmt, verbosity, redact
        self.handler: logging.Handler | None = None
        self.apply()

    def apply(self) -> None:
        if self.handler is not None:
            LOG.removeHandler(self.handler)
            self.handler.close()
        self.handler = logging.FileHandler(self.dest) if self.dest else logging.StreamHandler(sys.stderr)
        self.handler.setFormatter(_JsonFormatter() if self.fmt == "json"
                                  else logging.Formatter("%(asctime)s %(levelname)s %(message)s"))
        LOG.addHandler(self.handler)
        LOG.setLevel(self.LEVELS.get(int(self.verbosity), logging.INFO))
        LOG.propagate = False

    def set(self, verbosity=None, fmt=None, redact=None) -> None:
        if verbosity is not None:
            self.verbosity = max(0, min(3, int(verbosity)))
        if fmt in ("text", "json"):
            self.fmt = fmt
        if redact is not None:
            self.redact = bool(redact)
        self.apply()

    def body_for_log(self, body) -> str:
        """Request bodies carry user text: with redaction on only the shape is logged."""
        if not self.redact:
            return json.dumps(body, ensure_ascii=False)[:2000]
        if isinstance(body, dict):
            keep = {k: v for k, v in body.items() if k in ("model", "stream", "max_tokens", "temperature", "n")}
            if "messages" in body:
                keep["messages"] = f"<{len(body['messages'])} messages>"
            if "prompt" in body:
                p = body["prompt"]
                keep["prompt"] = f"<{len(p)} {'chars' if isinstance(p, str) else 'items'}>"
            return json.dumps(keep)
        return "<redacted>"


# ----------------------------------------------------------------------------- responses store
class ResponsesStore:
    """LRU + TTL store of Responses API objects (completed, in progress, cancelled)."""

    def __init__(self, capacity: int = 256, ttl_s: float = 3600.0, clock=time.monotonic):
        self.capacity, self.ttl_s, self.clock = capacity, ttl_s, clock
        self.items: "OrderedDict[str, tuple[float, dict]]" = OrderedDict()
        self.stats = dict(puts=0, hits=0, misses=0, expired=0, evicted=0)

    def _sweep(self) -> None:
        now = self.clock()
        for k in [k for k, (t, _) in self.items.items() if now - t > self.ttl_s]:
            del self.items[k]
            self.stats["expired"] += 1

    def put(self, rid: str, obj: dict) -> None:
        self._sweep()
        self.items[rid] = (self.clock(), obj)
        self.items.move_to_end(rid)
        self.stats["puts"] += 1
        while len(self.items) > self.capacity:
            self.items.popitem(last=False)
            self.stats["evicted"] += 1

    def get(self, rid: str) -> dict | None:
        self._sweep()
        e = self.items.get(rid)
        if e is None:
            self.stats["misses"] += 1
            return None
        self.items.move_to_end(rid)
        self.stats["hits"] += 1
        return e[1]

    # mapping-style access used by the core routes
    def __contains__(self, rid) -> bool:
        return self.get(rid) is not None

    def __getitem__(self, rid) -> dict:
        r = self.get(rid)
        if r is None:
            raise KeyError(rid)
        return r

    def __setitem__(self, rid, obj) -> None:
        self.put(rid, obj)

    def __len__(self) -> int:
        return len(self.items)

    def pop(self, rid, default=None):
        e = self.items.pop(rid, None)
        return e[1] if e is not None else default

    def __iter__(self):
        return iter(list(self.items))


def compact_messages(messages: list[dict], count_tokens, budget: int, keep_last: int = 2) -> tuple[list[dict], int]:
    """Conversation compaction: system messages and the last ``keep_last`` turns always stay; older
    turns are dropped oldest-first until the rendered prompt fits ``budget`` tokens. Returns the kept
    messages and how many were dropped."""
    system = [m for m in messages if m.get("role") == "system"]
    rest = [m for m in messages if m.get("role") != "system"]
    dropped = 0
    while len(rest) > keep_last and count_tokens(system + rest) > budget:
        rest.pop(0)
        dropped += 1
    return system + rest, dropped


# ----------------------------------------------------------------------------- stream sessions
class StreamSessions:
    """Resumable server-sent-event streams: every frame of a stream that carries a conversation id
    is kept in a bounded ring with a running event id; a client that lost its connection asks for
    the frames after the last id it saw."""

    def __init__(self, max_streams: int = 64, max_frames: int = 4096, ttl_s: float = 600.0):
        self.max_streams, self.max_frames, self.ttl_s = max_streams, max_frames, ttl_s
        self.streams: "OrderedDict[str, dict]" = OrderedDict()

    def open(self, conv_id: str) -> dict:
        self._sweep()
        st = dict(frames=deque(maxlen=self.max_frames), next_id=0, done=False, touched=time.monotonic(),
                  cond=asyncio.Condition(), request_id=None)
        self.streams[conv_id] = st
        self.streams.move_to_end(conv_id)
        while len(self.streams) > self.max_streams:
            self.streams.popitem(last=False)
        return st

    async def push(self, st: dict, frame: bytes, done: bool = False) -> int:
        async with st["cond"]:
            eid = st["next_id"]
            st["frames"].append((eid, frame))
            st["next_id"] += 1
            st["done"] = st["done"] or done
            st["touched"] = time.monotonic()
            st["cond"].notify_all()
        return eid

    def lookup(self, conv_id: str) -> dict | None:
        self._sweep()
        return self.streams.get(conv_id)

    def _sweep(self) -> None:
        now = time.monotonic()
        for k in [k for k, s in self.streams.items() if s["done"] and now - s["touched"] > self.ttl_s]:
            del self.streams[k]

    async def replay(self, st: dict, after: int):
        """Frames with id > ``after``, then live frames until the stream ends."""
        sent = after
        while True:
            async with st["cond"]:
                pending = [(i, f) for i, f in st["frames"] if i > sent]
                if not pending and not st["done"]:
                    try:
                        await asyncio.wait_for(st["cond"].wait(), timeout=30.0)
                    except asyncio.TimeoutError:
                        return
                    continue
                done = st["done"]
            for i, f in pending:
                yield i, f
                sent = i
            if done and not pending:
                return
            if done and sent >= st["next_id"] - 1:
                return


def frame_with_id(frame: bytes, eid: int) -> bytes:
    return b"id: " + str(eid).encode() + b"\n" + frame


# ----------------------------------------------------------------------------- histograms
class Histogram:
    def __init__(self, buckets: list[float]):
        self.buckets, self.counts, self.total, self.n = list(buckets), [0] * len(buckets), 0.0, 0

    def observe(self, v: float) -> None:
        self.total += v
        self.n += 1
        for i, b in enumerate(self.buckets):
            if v <= b:
                self.counts[i] += 1

    def render(self, name: str, help_: str) -> list[str]:
        out = [f"# HELP {name} {help_}", f"# TYPE {name} histogram"]
        for b, c in zip(self.buckets, self.counts):
            out.append(f'{name}_bucket{{le="{b}"}} {c}')
        out += [f'{name}_bucket{{le="+Inf"}} {self.n}', f"{name}_sum {round(self.total, 6)}", f"{name}_count {self.n}"]
        return out


# ----------------------------------------------------------------------------- installation
SETTABLE = {
    "default_max_tokens": int, "default_temperature": float, "thinking_budget": int, "log_verbosity": int,
    "log_format": str, "log_redact": bool, "prefill_chunk_size": int, "max_queue_depth": int, "cors_origins": list,
}


def install_extras(app, state) -> None:
    """Adds the middleware and routes of this module to the application. ``state`` gains ``settings``,
    ``responses`` (a :class:`ResponsesStore`), ``streams``, ``inflight`` and ``log``."""
    from .app import _err

    if not hasattr(state, "log") or state.log is None:
        state.log = LogControl()
    if not isinstance(getattr(state, "responses", None), ResponsesStore):
        state.responses = ResponsesStore()
    state.streams = StreamSessions()
    state.inflight = {}                   # public id (chat / response id) -> GenRequest
    state.background = {}                 # response id -> asyncio.Task
    if not getattr(state, "cors_origins", None):
        state.cors_origins = ["*"]
    state.settings = dict(default_max_tokens=None, default_temperature=None,
                          thinking_budget=getattr(state, "default_thinking_budget", None))
    state.hist = dict(ttft=Histogram([0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10, 30]),
                      decode_tps=Histogram([1, 5, 10, 25, 50, 100, 250, 500, 1000, 2500]))

    # ---- CORS + request context + access log (one middleware: order matters for preflights)
    @app.middleware("http")
    async def cors_and_context(request: Request, call_next):
        origin = request.headers.get("origin")
        allowed = state.cors_origins
        allow = "*" if "*" in allowed else (origin if origin in allowed else None)
        if request.method == "OPTIONS" and request.headers.get("access-control-request-method"):
            # preflight: answered here, never reaches authentication (browsers send it without credentials)
            h = {"Access-Control-Allow-Methods": "GET, POST, PUT, DELETE, OPTIONS",
                 "Access-Control-Allow-Headers": request.headers.get("access-control-request-headers", "*"),
                 "Access-Control-Max-Age": "86400", "Vary": "Origin"}
            if allow:
                h["Access-Control-Allow-Origin"] = allow
            return Response(status_code=204 if allow else 403, headers=h)
        try:
            prio = int(request.headers.get("x-priority", "0") or 0)
        except ValueError:
            prio = 0
        tok = REQUEST_CTX.set({"priority": prio, "conversation_id": request.headers.get("x-conversation-id"),
                               "last_event_id": request.headers.get("last-event-id")})
        t0 = time.perf_counter()
        try:
            resp = await call_next(request)
        finally:
            REQUEST_CTX.reset(tok)
        if allow:
            resp.headers["Access-Control-Allow-Origin"] = allow
            resp.headers.setdefault("Vary", "Origin")
        elif "access-control-allow-origin" in resp.headers:
            del resp.headers["access-control-allow-origin"]
        LOG.info("%s %s -> %d", request.method, request.url.path, resp.status_code,
                 extra={"fields": {"method": request.method, "path": request.url.path, "status": resp.status_code,
                                   "ms": round((time.perf_counter() - t0) * 1e3, 2)}})
        return resp

    # ---- live settings (opt-in)
    @app.get("/v1/settings")
    async def get_settings():
        if not getattr(state, "settings_enabled", False):
            return _err(404, "live settings are disabled (start the server with --enable-settings)", "not_found_error")
        e = state.worker.view().ecfg
        return {**state.settings, "log_verbosity": state.log.verbosity, "log_format": state.log.fmt,
                "log_redact": state.log.redact, "prefill_chunk_size": e.prefill_chunk_alone,
                "max_queue_depth": e.max_queue_depth, "cors_origins": state.cors_origins}

    @app.api_route("/v1/settings", methods=["POST", "PUT", "PATCH"])
    async def put_settings(body: dict):
        if not getattr(state, "settings_enabled", False):
            return _err(404, "live settings are disabled (start the server with --enable-settings)", "not_found_error")
        if not state.api_keys:
            return _err(403, "live settings need an API key on the server (--api-key)", "forbidden")
        bad = [k for k in body if k not in SETTABLE]
        if bad:
            return _err(400, f"unknown settings: {bad}; settable: {sorted(SETTABLE)}")
        try:
            vals = {k: (None if v is None else SETTABLE[k](v)) for k, v in body.items()}
        except (TypeError, ValueError) as e:
            return _err(400, f"bad value: {e}")
        if vals.get("thinking_budget") is not None and vals["thinking_budget"] < -1:
            return _err(400, "thinking_budget must be >= -1")
        e = state.worker.view().ecfg
        for k, v in vals.items():
            if k in ("default_max_tokens", "default_temperature", "thinking_budget"):
                state.settings[k] = v
            elif k == "prefill_chunk_size" and v:
                e.prefill_chunk_alone, e.prefill_chunk_contended = int(v), min(512, int(v))
            elif k == "max_queue_depth" and v:
                e.max_queue_depth = int(v)
            elif k == "cors_origins" and v is not None:
                state.cors_origins = [str(x) for x in v] or ["*"]
        state.log.set(vals.get("log_verbosity"), vals.get("log_format"), vals.get("log_redact"))
        return await get_settings()

    # ---- in-flight control
    @app.post("/v1/chat/completions/control")
    async def chat_control(body: dict):
        """``{"id": "chatcmpl-…", "action": "cancel"}`` ends a generation that is still running (the
        stream then closes with finish_reason "stop"); ``"action": "status"`` reports it."""
        rid = str(body.get("id", ""))
        req = state.inflight.get(rid)
        action = body.get("action", "status")
        if action not in ("cancel", "status"):
            return _err(400, "action must be cancel or status")
        if req is None:
            return _err(404, f"no generation in flight with id {rid!r}", "not_found_error")
        if action == "cancel":
            state.worker.cancel(req)
            return {"id": rid, "status": "cancelling", "tokens_generated": req.n_emitted}
        return {"id": rid, "status": "running", "tokens_generated": req.n_emitted}

    # ---- responses: cancel / compaction (background creation lives in the core route)
    @app.post("/v1/responses/{rid}/cancel")
    async def cancel_response(rid: str):
        r = state.responses.get(rid)
        if r is None:
            return _err(404, "response not found", "not_found_error")
        task = state.background.get(rid)
        if r.get("status") in ("queued", "in_progress"):
            req = state.inflight.get(rid)
            if req is not None:
                state.worker.cancel(req)
            if task is not None:
                task.cancel()
            r["status"] = "cancelled"
        return {k: v for k, v in r.items() if not k.startswith("_")}

    @app.post("/v1/responses/compact")
    async def compact_response(body: dict):
        """Returns a shortened conversation (``input`` items) that fits ``max_input_tokens``: system
        messages and the latest turns stay, the oldest turns go first."""
        from .app import _responses_input_messages
        msgs = _responses_input_messages(state, body)
        budget = int(body.get("max_input_tokens") or state.worker.engine.ecfg.max_model_len // 2)

        def count(ms):
            return len(state.tokenizer.encode(state.render(ms), add_special_tokens=False))
        before = count(msgs)
        kept, dropped = compact_messages(msgs, count, budget, keep_last=int(body.get("keep_last", 2)))
        return {"object": "response.compaction", "input": [{"role": m["role"], "content": m["content"]} for m in kept],
                "dropped_messages": dropped, "input_tokens_before": before, "input_tokens_after": count(kept)}

    # ---- resumable streams
    @app.get("/v1/stream")
    async def resume_stream(conversation_id: str, last_event_id: int = -1):
        st = state.streams.lookup(conversation_id)
        if st is None:
            return _err(404, "no stream with this conversation id", "not_found_error")

        async def gen():
            async for eid, frame in state.streams.replay(st, int(last_event_id)):
                yield frame_with_id(frame, eid)
        return StreamingResponse(gen(), media_type="text/event-stream")

    @app.get("/v1/streams/lookup")
    async def lookup_stream(conversation_id: str):
        st = state.streams.lookup(conversation_id)
        if st is None:
            return _err(404, "no stream with this conversation id", "not_found_error")
        return {"conversation_id": conversation_id, "done": st["done"], "next_event_id": st["next_id"],
                "buffered": len(st["frames"]), "first_buffered_id": st["frames"][0][0] if st["frames"] else None}


async def tee_stream(state, gen, conv_id: str | None):
    """Passes SSE frames through; with a conversation id every frame is also kept for resumption and
    carries an ``id:`` line. The generation keeps filling the session when the client disconnects."""
    if not conv_id:
        async for frame in gen:
            yield frame
        return
    st = state.streams.open(conv_id)
    q: asyncio.Queue = asyncio.Queue()

    async def pump():
        try:
            async for frame in gen:
                eid = await state.streams.push(st, frame)
                q.put_nowait(frame_with_id(frame, eid))
        finally:
            await state.streams.push(st, b"", done=True)
            q.put_nowait(None)

    task = asyncio.create_task(pump())      # detached from the client connection on purpose
    st["task"] = task
    while True:
        item = await q.get()
        if item is None:
            return
        yield item
