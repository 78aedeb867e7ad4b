"""Router mode: one HTTP front for a pool of models, loaded on demand and evicted least-recently-used.

Reference behaviour (src/server/router_server.rs, router_models.rs, router_presets.rs): the server is
started with a models directory (or an INI file of presets) instead of one model; requests name
their model in the ``model`` field; at most ``--models-max`` models are resident, the least recently
used one is unloaded when another has to come in; ``GET /models`` lists every known model with its
state, ``POST /models/load`` / ``/models/unload`` move one explicitly.

Here the front is a small ASGI application: it buffers the request body, reads ``model`` from the
JSON, makes that model resident (each resident model is a complete single-model application from
``server/app.py`` with its own engine worker thread) and replays the request into it, so streaming
responses pass through untouched. Loading is serialised by one lock; a model being used by a
request in flight is never evicted.
"""
from __future__ import annotations

import asyncio
import configparser
import json
import time
from collections import OrderedDict
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable


@dataclass
class ModelEntry:
    name: str
    path: str
    options: dict = field(default_factory=dict)   # preset options (ctx_size, parallel, ...)
    app: object | None = None                      # resident: the single-model ASGI application
    state: object | None = None
    in_flight: int = 0
    loaded_at: float = 0.0
    last_used: float = 0.0
    loads: int = 0


def discover_models(models_dir: str | None = None, presets_ini: str | None = None) -> dict[str, ModelEntry]:
    """Every sub-directory with a ``config.json`` is a model named after the directory; an INI file
    adds (or overrides) entries: ``[name]`` sections with ``model = <path>`` and engine options."""
    out: dict[str, ModelEntry] = {}
    if models_dir:
        for p in sorted(Path(models_dir).iterdir()):
            if (p / "config.json").exists():
                out[p.name] = ModelEntry(p.name, str(p))
    if presets_ini:
        ini = configparser.ConfigParser()
        ini.read(presets_ini)
        for sec in ini.sections():
            opts = dict(ini[sec])
            path = opts.pop("model", opts.pop("path", None))
            if not path:
                raise ValueError(f"{presets_ini}: section [{sec}] has no model path")
            out[sec] = ModelEntry(sec, path, opts)
    return out


class ModelPool:
    """Known models, the resident subset (LRU order) and the loader that builds one application."""

    def __init__(self, entries: dict[str, ModelEntry], loader: Callable[[ModelEntry], tuple], max_loaded: int = 1,
                 default: str | None = None):
        if not entries:
            raise ValueError("router mode needs at least one model")
        self.entries = entries
        self.loader = loader
        self.max_loaded = max(1, int(max_loaded))
        self.default = default or next(iter(entries))
        self.resident: OrderedDict[str, ModelEntry] = OrderedDict()
        self.lock = asyncio.Lock()
        self.events: list[dict] = []                 # load / unload history (bounded)

    def _event(self, kind: str, name: str) -> None:
        self.events.append(dict(event=kind, model=name, time=time.time()))
        del self.events[:-256]

    def _unload(self, e: ModelEntry) -> None:
        worker = getattr(e.state, "worker", None)
        if worker is not None:
            worker.shutdown()
        e.app = e.state = None
        self.resident.pop(e.name, None)
        self._event("unloaded", e.name)

    async def acquire(self, name: str) -> ModelEntry:
        e = self.entries.get(name)
        if e is None:
            raise KeyError(name)
        async with self.lock:
            if e.app is None:
                while len(self.resident) >= self.max_loaded:
                    victim = next((v for v in self.resident.values() if v.in_flight == 0), None)
                    if victim is None:
                        raise RuntimeError("every resident model is busy; raise --models-max or retry")
                    self._unload(victim)
                self._event("loading", name)
                e.app, e.state = await asyncio.get_running_loop().run_in_executor(None, self.loader, e)
                e.loaded_at = time.time()
                e.loads += 1
                self.resident[name] = e
                self._event("loaded", name)
            self.resident.move_to_end(name)
            e.last_used = time.time()
            e.in_flight += 1
            return e

    def release(self, e: ModelEntry) -> None:
        e.in_flight -= 1

    async def unload(self, name: str) -> bool:
        async with self.lock:
            e = self.entries.get(name)
            if e is None or e.app is None:
                return False
            if e.in_flight:
                raise RuntimeError("model is serving requests")
            self._unload(e)
            return True

    def listing(self) -> list[dict]:
        return [dict(id=e.name, object="model", owned_by="mlxcel_b200", path=e.path,
                     status="loaded" if e.app is not None else "unloaded", in_flight=e.in_flight, loads=e.loads,
                     last_used=e.last_used) for e in self.entries.values()]

    def shutdown(self) -> None:
        for e in list(self.resident.values()):
            self._unload(e)


def default_loader(device: str = "cuda", api_keys: set[str] | None = None, engine_defaults: dict | None = None):
    """Loader that builds a single-model application from a checkpoint directory."""
    def load(e: ModelEntry):
        from ..engine.engine import EngineConfig
        from ..llm import LLM
        from .app import ServerState, create_app
        from .worker import ModelWorker

        opts = dict(engine_defaults or {})
        opts.update(e.options)
        ec = EngineConfig()
        for key, attr in (("ctx_size", "max_model_len"), ("parallel", "max_batch"), ("num_blocks", "num_blocks"),
                          ("block_size", "block_size"), ("kv_bits", "kv_bits")):
            if key in opts:
                setattr(ec, attr, int(opts[key]))
        llm = LLM.from_pretrained(e.path, device=opts.get("device", device), engine_config=ec)
        worker = ModelWorker(llm.engine, llm.tokenizer, e.name)
        state = ServerState(worker, llm.tokenizer, e.name, api_keys=api_keys)
        return create_app(state), state
    return load


class RouterApp:
    """ASGI front: ``/models*`` are answered here, everything else goes to the model the body names."""

    def __init__(self, pool: ModelPool):
        self.pool = pool

    async def __call__(self, scope, receive, send):
        if scope["type"] == "lifespan":
            while True:
                msg = await receive()
                if msg["type"] == "lifespan.startup":
                    await send({"type": "lifespan.startup.complete"})
                elif msg["type"] == "lifespan.shutdown":
                    self.pool.shutdown()
                    await send({"type": "lifespan.shutdown.complete"})
                    return
        if scope["type"] != "http":
            return
        body = b""
        while True:
            msg = await receive()
            if msg["type"] == "http.disconnect":
                return
            body += msg.get("body", b"")
            if not msg.get("more_body"):
                break
        path, method = scope["path"].rstrip("/") or "/", scope["method"]
        if path in ("/models", "/v1/models") and method == "GET":
            return await self._json(send, 200, dict(object="list", data=self.pool.listing()))
        if path == "/models/events" and method == "GET":
            return await self._json(send, 200, dict(events=self.pool.events))
        payload = {}
        if body[:1] == b"{":
            try:
                payload = json.loads(body)
            except ValueError:
                return await self._json(send, 400, dict(error=dict(message="invalid JSON body")))
        name = payload.get("model") if isinstance(payload, dict) else None
        if path in ("/models/load", "/models/unload") and method == "POST":
            if name not in self.pool.entries:
                return await self._json(send, 404, dict(error=dict(message=f"unknown model {name!r}")))
            try:
                if path.endswith("/unload"):
                    done = await self.pool.unload(name)
                    return await self._json(send, 200, dict(model=name, status="unloaded", changed=done))
                e = await self.pool.acquire(name)
                self.pool.release(e)
                return await self._json(send, 200, dict(model=name, status="loaded"))
            except RuntimeError as ex:
                return await self._json(send, 409, dict(error=dict(message=str(ex))))
        name = name or self.pool.default
        if name not in self.pool.entries:
            return await self._json(send, 404, dict(error=dict(message=f"unknown model {name!r}",
                                                               type="invalid_request_error")))
        try:
            e = await self.pool.acquire(name)
        except RuntimeError as ex:
            return await self._json(send, 503, dict(error=dict(message=str(ex))))
        replayed = False

        async def replay():
            nonlocal replayed
            if not replayed:
                replayed = True
                return {"type": "http.request", "body": body, "more_body": False}
            return await receive()

        try:
            await e.app(scope, replay, send)
        finally:
            self.pool.release(e)

    @staticmethod
    async def _json(send, status: int, obj) -> None:
        data = json.dumps(obj).encode()
        await send({"type": "http.response.start", "status": status,
                    "headers": [(b"content-type", b"application/json"), (b"content-length", str(len(data)).encode())]})
        await send({"type": "http.response.body", "body": data})


def create_router_app(models_dir: str | None = None, presets_ini: str | None = None, max_loaded: int = 1,
                      device: str = "cuda", api_keys: set[str] | None = None, default: str | None = None,
                      loader=None, engine_defaults: dict | None = None) -> RouterApp:
    entries = discover_models(models_dir, presets_ini)
    pool = ModelPool(entries, loader or default_loader(device, api_keys, engine_defaults), max_loaded, default)
    return RouterApp(pool)
