"""Replica front: one listener in front of several single-model servers.

Two deployments share this front (an ASGI application over aiohttp clients):

* **Data-parallel replicas** (``serve --dp N``): N complete servers of the same model, one per GPU,
  each with its own engine, KV pool and prefix cache. A request goes to the replica with the fewest
  requests in flight (ties: round robin); a conversation that names itself (``X-Conversation-Id``
  or ``prompt_cache_key``) sticks to the replica that served it last, so its prefix cache hits.
  Streaming responses pass through chunk by chunk. A replica that refuses connections is marked
  down and re-probed after a cool-down (the reference's router failover,
  docs/CONTINUOUS_BATCHING.md:1019-1054; its request routers live in
  src/distributed/disaggregated/routing.rs: ``RoundRobinRouter``, ``LoadBalancedRouter``).
* **Disaggregated prefill / decode** (``--prefill-url … --decode-url …``): the prompt is prefilled
  on a prefill-role server, its KV blocks travel as one blob
  (``/v1/internal/kv/export`` → ``/v1/internal/kv/import``) to a decode-role server, and the
  original request is then served there from the imported prefix (reference
  src/distributed/disaggregated/*, src/server/router_front.rs). Requests whose prompt the front
  cannot see as text or token ids (chat messages need the template) go straight to a decode server.

The front holds no model; `/health`, `/metrics` and `/v1/models` aggregate the backends.
"""
from __future__ import annotations

import asyncio
import itertools
import json
import time
from dataclasses import dataclass, field


@dataclass
class Backend:
    url: str
    role: str = "replica"            # replica | prefill | decode
    in_flight: int = 0
    served: int = 0
    failures: int = 0
    down_until: float = 0.0
    last_error: str = ""

    def available(self, now: float) -> bool:
        return now >= self.down_until


class Balancer:
    """Least-outstanding-requests choice with sticky conversations and failure cool-down."""

    def __init__(self, backends: list[Backend], cooldown_s: float = 5.0, clock=time.monotonic):
        if not backends:
            raise ValueError("the front needs at least one backend")
        self.backends, self.cooldown_s, self.clock = backends, cooldown_s, clock
        self._rr = itertools.count()
        self.sticky: dict[str, Backend] = {}

    def pick(self, role: str = "replica", key: str | None = None) -> Backend:
        now = self.clock()
        pool = [b for b in self.backends if b.role == role and b.available(now)]
        if not pool:
            pool = [b for b in self.backends if b.role == role]      # all down: try anyway, oldest failure first
            if not pool:
                raise LookupError(f"no backend with role {role!r}")
            pool.sort(key=lambda b: b.down_until)
            return pool[0]
        if key and key in self.sticky and self.sticky[key] in pool:
            return self.sticky[key]
        low = min(b.in_flight for b in pool)
        ties = [b for b in pool if b.in_flight == low]
        b = ties[next(self._rr) % len(ties)]
        if key:
            self.sticky[key] = b
            if len(self.sticky) > 4096:
                self.sticky.pop(next(iter(self.sticky)))
        return b

    def failed(self, b: Backend, err: str) -> None:
        b.failures += 1
        b.last_error = err
        b.down_until = self.clock() + self.cooldown_s
        for k in [k for k, v in self.sticky.items() if v is b]:
            del self.sticky[k]


_HOP = {"connection", "keep-alive", "transfer-encoding", "te", "trailer", "upgrade", "proxy-authorization",
        "proxy-authenticate", "content-length", "host"}


class FrontApp:
    """ASGI application: forwards every request to a backend chosen by the balancer."""

    def __init__(self, balancer: Balancer, disaggregated: bool = False, timeout_s: float = 3600.0):
        self.lb, self.disagg, self.timeout_s = balancer, disaggregated, timeout_s
        self._session = None
        self.stats = dict(requests=0, handoffs=0, handoff_bytes=0, retries=0)

    async def _http(self):
        import aiohttp
        if self._session is None:
            self._session = aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=self.timeout_s))
        return self._session

    async def __call__(self, scope, receive, send):
        if scope["type"] == "lifespan":
            while True:
                msg = await receive()
                if msg["type"] == "lifespan.startup":
                    await send({"type": "lifespan.startup.complete"})
                elif msg["type"] == "lifespan.shutdown":
                    if self._session is not None:
                        await self._session.close()
                    await send({"type": "lifespan.shutdown.complete"})
                    return
        if scope["type"] != "http":
            return
        body = b""
        while True:
            msg = await receive()
            body += msg.get("body", b"")
            if not msg.get("more_body"):
                break
        path, method = scope["path"], scope["method"]
        headers = {k.decode(): v.decode() for k, v in scope["headers"]}
        if path == "/health":
            return await self._health(send)
        if path == "/front/stats":
            return await self._json(send, 200, dict(self.stats, backends=[vars(b) for b in self.lb.backends]))
        self.stats["requests"] += 1
        key = headers.get("x-conversation-id")
        parsed = None
        if body and headers.get("content-type", "").startswith("application/json"):
            try:
                parsed = json.loads(body)
                key = key or parsed.get("prompt_cache_key") or parsed.get("user")
            except ValueError:
                parsed = None
        role = "decode" if self.disagg else "replica"
        forced = None
        if self.disagg and method == "POST" and isinstance(parsed, dict) and path in ("/v1/completions", "/completion", "/completions"):
            forced = await self._handoff(parsed, key)     # the decode server that now holds the prompt's blocks
        qs = scope.get("query_string", b"").decode()
        last_err = "no backend"
        for attempt in range(2):            # one retry on another backend when the first refuses the connection
            try:
                b = forced if (forced is not None and attempt == 0) else self.lb.pick(role, key)
            except LookupError as e:
                return await self._json(send, 503, {"error": {"message": str(e), "type": "unavailable"}})
            try:
                return await self._forward(b, method, path, qs, headers, body, send)
            except _ConnectFailed as e:
                self.lb.failed(b, str(e))
                self.stats["retries"] += 1
                last_err = str(e)
        return await self._json(send, 502, {"error": {"message": f"backend unreachable: {last_err}", "type": "bad_gateway"}})

    async def _handoff(self, body: dict, key):
        """Prefill on a prefill-role server and import the KV blob on the decode server that will take
        the request (sticky key or least loaded). Returns that decode server, or None when the
        hand-off did not happen (the request is then served by a decode server from scratch)."""
        prompt = body.get("prompt")
        if not isinstance(prompt, (str, list)) or not prompt:
            return None
        try:
            pre = self.lb.pick("prefill")
            dec = self.lb.pick("decode", key)
        except LookupError:
            return None
        http = await self._http()
        try:
            pre.in_flight += 1
            async with http.post(pre.url + "/v1/internal/kv/export", json={"prompt": prompt}) as r:
                if r.status != 200:
                    return None
                blob = await r.read()
        except Exception as e:
            self.lb.failed(pre, f"{type(e).__name__}: {e}")
            return None
        finally:
            pre.in_flight -= 1
            pre.served += 1
        try:
            async with http.post(dec.url + "/v1/internal/kv/import", data=blob,
                                 headers={"content-type": "application/octet-stream"}) as r:
                if r.status == 200:
                    self.stats["handoffs"] += 1
                    self.stats["handoff_bytes"] += len(blob)
                    return dec
        except Exception as e:
            self.lb.failed(dec, f"{type(e).__name__}: {e}")
        return None

    async def _forward(self, b: Backend, method, path, qs, headers, body, send):
        import aiohttp
        http = await self._http()
        url = b.url + path + (("?" + qs) if qs else "")
        fwd = {k: v for k, v in headers.items() if k not in _HOP}
        b.in_flight += 1
        started = False
        try:
            try:
                resp = await http.request(method, url, data=body if body else None, headers=fwd)
            except (aiohttp.ClientConnectorError, aiohttp.ServerDisconnectedError, ConnectionError, OSError) as e:
                raise _ConnectFailed(f"{b.url}: {type(e).__name__}: {e}") from None
            async with resp:
                out_headers = [(k.lower().encode(), v.encode()) for k, v in resp.headers.items() if k.lower() not in _HOP]
                out_headers.append((b"x-served-by", b.url.encode()))
                await send({"type": "http.response.start", "status": resp.status, "headers": out_headers})
                started = True
                async for chunk in resp.content.iter_any():
                    await send({"type": "http.response.body", "body": chunk, "more_body": True})
                await send({"type": "http.response.body", "body": b"", "more_body": False})
        except _ConnectFailed:
            raise
        except Exception as e:
            if not started:
                raise _ConnectFailed(f"{b.url}: {type(e).__name__}: {e}") from None
            await send({"type": "http.response.body", "body": b"", "more_body": False})
        finally:
            b.in_flight -= 1
            b.served += 1

    async def _health(self, send):
        http = await self._http()
        states = []
        for b in self.lb.backends:
            try:
                async with http.get(b.url + "/health") as r:
                    states.append(dict(url=b.url, role=b.role, ok=r.status == 200))
            except Exception as e:
                self.lb.failed(b, f"{type(e).__name__}: {e}")
                states.append(dict(url=b.url, role=b.role, ok=False))
        ok = any(s["ok"] for s in states if s["role"] in ("replica", "decode"))
        await self._json(send, 200 if ok else 503, {"status": "ok" if ok else "error", "backends": states})

    @staticmethod
    async def _json(send, status: int, obj) -> None:
        data = json.dumps(obj).encode()
        await send({"type": "http.response.start", "status": status,
                    "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(data)).encode())]})
        await send({"type": "http.response.body", "body": data})


class _ConnectFailed(Exception):
    pass


def create_front_app(replicas: list[str] | None = None, prefill: list[str] | None = None,
                     decode: list[str] | None = None, cooldown_s: float = 5.0) -> FrontApp:
    backends = [Backend(u.rstrip("/"), "replica") for u in replicas or []]
    backends += [Backend(u.rstrip("/"), "prefill") for u in prefill or []]
    backends += [Backend(u.rstrip("/"), "decode") for u in decode or []]
    disagg = bool(prefill or decode)
    if disagg and not decode:
        raise ValueError("a disaggregated front needs at least one decode server")
    return FrontApp(Balancer(backends, cooldown_s=cooldown_s), disaggregated=disagg)
