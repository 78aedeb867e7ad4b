"""Python client: talks to a running server, or starts and owns one.

Counterpart of the reference's pure-Python package (python/src/mlxcel/_client.py, _server.py): a
thin wrapper over the OpenAI / llama-server compatible HTTP API plus a helper that launches
``mlxcel serve`` as a child process, waits for ``/health`` and shuts it down with the client.
"""
from __future__ import annotations

import json
import subprocess
import sys
import time
from typing import Iterator

import requests


class MlxcelError(RuntimeError):
    pass


class Client:
    def __init__(self, base_url: str = "http://127.0.0.1:8080", api_key: str | None = None, timeout: float = 600.0,
                 session=None):
        self.base = base_url.rstrip("/")
        self.timeout = timeout
        self.http = session or requests.Session()
        self.headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}

    # ------------------------------------------------------------------ plumbing
    def _post(self, path: str, body: dict, stream: bool = False):
        r = self.http.post(self.base + path, json=body, headers=self.headers, timeout=self.timeout, stream=stream)
        if r.status_code >= 400:
            raise MlxcelError(f"{path}: HTTP {r.status_code}: {r.text[:500]}")
        return r

    def _get(self, path: str):
        r = self.http.get(self.base + path, headers=self.headers, timeout=self.timeout)
        if r.status_code >= 400:
            raise MlxcelError(f"{path}: HTTP {r.status_code}: {r.text[:500]}")
        return r.json()

    @staticmethod
    def _sse(resp) -> Iterator[dict]:
        for raw in resp.iter_lines():
            line = raw.decode() if isinstance(raw, bytes) else raw
            if not line.startswith("data:"):
                continue
            data = line[5:].strip()
            if data == "[DONE]":
                return
            yield json.loads(data)

    # ------------------------------------------------------------------ API
    def health(self) -> bool:
        try:
            return self._get("/health").get("status") == "ok"
        except Exception:
            return False

    def models(self) -> list[str]:
        return [m["id"] for m in self._get("/v1/models")["data"]]

    def chat(self, messages: list[dict], **params) -> str:
        out = self._post("/v1/chat/completions", {"messages": messages, **params}).json()
        return out["choices"][0]["message"].get("content") or ""

    def chat_stream(self, messages: list[dict], **params) -> Iterator[str]:
        resp = self._post("/v1/chat/completions", {"messages": messages, "stream": True, **params}, stream=True)
        for ev in self._sse(resp):
            for ch in ev.get("choices", []):
                piece = ch.get("delta", {}).get("content")
                if piece:
                    yield piece

    def complete(self, prompt: str, **params) -> str:
        return self._post("/v1/completions", {"prompt": prompt, **params}).json()["choices"][0]["text"]

    def embed(self, texts: list[str] | str) -> list[list[float]]:
        out = self._post("/v1/embeddings", {"input": texts}).json()
        return [d["embedding"] for d in out["data"]]

    def rerank(self, query: str, documents: list[str], top_n: int | None = None) -> list[dict]:
        body = {"query": query, "documents": documents}
        if top_n is not None:
            body["top_n"] = top_n
        return self._post("/v1/rerank", body).json()["results"]

    def tokenize(self, text: str) -> list[int]:
        return self._post("/tokenize", {"content": text}).json()["tokens"]

    def detokenize(self, tokens: list[int]) -> str:
        return self._post("/detokenize", {"tokens": tokens}).json()["content"]

    def lora_adapters(self) -> list[dict]:
        return self._get("/lora-adapters")

    def set_lora_scales(self, scales: list[dict]) -> list[dict]:
        return self._post("/lora-adapters", scales).json()   # type: ignore[arg-type]


class ManagedServer:
    """``with ManagedServer(model_dir, port=8081) as client: client.chat(...)``"""

    def __init__(self, model: str, port: int = 8080, host: str = "127.0.0.1", extra_args: list[str] | None = None,
                 startup_timeout: float = 600.0, api_key: str | None = None):
        self.cmd = [sys.executable, "-m", "mlxcel_b200.cli", "serve", "-m", str(model), "--host", host, "--port",
                    str(port), *(extra_args or [])]
        if api_key:
            self.cmd += ["--api-key", api_key]
        self.client = Client(f"http://{host}:{port}", api_key=api_key)
        self.startup_timeout = startup_timeout
        self.proc: subprocess.Popen | None = None

    def start(self) -> Client:
        self.proc = subprocess.Popen(self.cmd)
        deadline = time.time() + self.startup_timeout
        while time.time() < deadline:
            if self.proc.poll() is not None:
                raise MlxcelError(f"server exited with code {self.proc.returncode}")
            if self.client.health():
                return self.client
            time.sleep(0.5)
        self.stop()
        raise MlxcelError("server did not become healthy in time")

    def stop(self) -> None:
        if self.proc is not None and self.proc.poll() is None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.proc = None

    def __enter__(self) -> Client:
        return self.start()

    def __exit__(self, *exc) -> None:
        self.stop()


class AsyncClient:
    """asyncio counterpart of :class:`Client` over aiohttp (reference python/src/mlxcel: the async client)::

        async with AsyncClient("http://127.0.0.1:8080") as c:
            async for piece in c.chat_stream([{"role": "user", "content": "hi"}], max_tokens=32):
                print(piece, end="")
    """

    def __init__(self, base_url: str = "http://127.0.0.1:8080", api_key: str | None = None, timeout: float = 600.0):
        self.base = base_url.rstrip("/")
        self.timeout = timeout
        self.headers = {"Authorization": f"Bearer {api_key}"} if api_key else {}
        self._session = None

    async def __aenter__(self) -> "AsyncClient":
        import aiohttp
        self._session = aiohttp.ClientSession(headers=self.headers, timeout=aiohttp.ClientTimeout(total=self.timeout))
        return self

    async def __aexit__(self, *exc) -> None:
        await self.close()

    async def close(self) -> None:
        if self._session is not None:
            await self._session.close()
            self._session = None

    def _http(self):
        if self._session is None:
            raise MlxcelError("use 'async with AsyncClient(...)' (no open session)")
        return self._session

    async def _post(self, path: str, body: dict) -> dict:
        async with self._http().post(self.base + path, json=body) as r:
            if r.status >= 400:
                raise MlxcelError(f"{path}: HTTP {r.status}: {(await r.text())[:500]}")
            return await r.json()

    async def _get(self, path: str) -> dict:
        async with self._http().get(self.base + path) as r:
            if r.status >= 400:
                raise MlxcelError(f"{path}: HTTP {r.status}: {(await r.text())[:500]}")
            return await r.json()

    async def health(self) -> bool:
        try:
            return (await self._get("/health")).get("status") == "ok"
        except Exception:
            return False

    async def models(self) -> list[str]:
        return [m["id"] for m in (await self._get("/v1/models"))["data"]]

    async def chat(self, messages: list[dict], **params) -> str:
        r = await self._post("/v1/chat/completions", {"messages": messages, **params})
        return r["choices"][0]["message"]["content"] or ""

    async def chat_stream(self, messages: list[dict], **params):
        body = {"messages": messages, "stream": True, **params}
        async with self._http().post(self.base + "/v1/chat/completions", json=body) as r:
            if r.status >= 400:
                raise MlxcelError(f"/v1/chat/completions: HTTP {r.status}: {(await r.text())[:500]}")
            async for raw in r.content:
                line = raw.decode().strip()
                if not line.startswith("data:"):
                    continue
                data = line[5:].strip()
                if data == "[DONE]":
                    return
                ev = json.loads(data)
                if "error" in ev:
                    raise MlxcelError(str(ev["error"]))
                for ch in ev.get("choices") or []:
                    piece = (ch.get("delta") or {}).get("content")
                    if piece:
                        yield piece

    async def complete(self, prompt: str, **params) -> str:
        return (await self._post("/v1/completions", {"prompt": prompt, **params}))["choices"][0]["text"]

    async def embed(self, texts: list[str] | str) -> list[list[float]]:
        r = await self._post("/v1/embeddings", {"input": texts})
        return [d["embedding"] for d in r["data"]]

    async def rerank(self, query: str, documents: list[str], top_n: int | None = None, **params) -> list[dict]:
        body = {"query": query, "documents": documents, **params}
        if top_n:
            body["top_n"] = top_n
        return (await self._post("/v1/rerank", body))["results"]

    async def tokenize(self, text: str) -> list[int]:
        return (await self._post("/tokenize", {"content": text}))["tokens"]
