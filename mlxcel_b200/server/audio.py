"""Speech routes of the OpenAI API for speech-to-text checkpoints:
``POST /v1/audio/transcriptions`` and ``POST /v1/audio/translations`` (multipart form: ``file``, optional
``language``, ``response_format`` json | text | verbose_json | srt | vtt, ``model``). ``/v1/audio/speech``
(text-to-speech) answers 501: no speech synthesis model is built here
(reference routes: src/server/app.rs:374-403, src/server/routes/audio*.rs; upload limit 100 MiB)."""
from __future__ import annotations

import asyncio
import threading
import time

from fastapi import FastAPI, File, Form, Request, UploadFile
from fastapi.responses import JSONResponse, PlainTextResponse

MAX_UPLOAD = 100 << 20


def _stamp(t: float, sep: str) -> str:
    ms = int(round(t * 1000))
    return f"{ms // 3600000:02d}:{ms // 60000 % 60:02d}:{ms // 1000 % 60:02d}{sep}{ms % 1000:03d}"


def create_audio_app(transcriber, model_id: str, api_keys: set[str] | None = None) -> FastAPI:
    app = FastAPI(title="mlxcel_b200 audio")
    lock = threading.Lock()                 # one request on the model at a time (its kernels share scratch)
    started = time.time()

    def _err(code, msg, typ="invalid_request_error"):
        return JSONResponse(status_code=code, content={"error": {"message": msg, "type": typ}})

    @app.middleware("http")
    async def auth(request: Request, call_next):
        if api_keys and request.url.path not in ("/health",):
            key = request.headers.get("authorization", "").removeprefix("Bearer ").strip() or request.headers.get("x-api-key", "")
            if key not in api_keys:
                return _err(401, "invalid API key", "authentication_error")
        return await call_next(request)

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    @app.get("/models")
    async def models():
        return {"object": "list", "data": [{"id": model_id, "object": "model", "created": int(started), "owned_by": "mlxcel_b200"}]}

    @app.get("/metrics")
    async def metrics():
        s = transcriber.stats
        return PlainTextResponse("".join(f"mlxcel_audio_{k} {v}\n" for k, v in s.items()))

    async def _run(file: UploadFile, language, response_format, task):
        from ..audio import decode_audio
        data = await file.read()
        if len(data) > MAX_UPLOAD:
            return _err(413, "audio upload exceeds 100 MiB")
        try:
            samples = decode_audio(data)
        except ValueError as e:
            return _err(400, str(e))

        def work():
            with lock:
                return transcriber.transcribe(samples, language=language or None, task=task)
        try:
            r = await asyncio.get_running_loop().run_in_executor(None, work)
        except ValueError as e:
            return _err(400, str(e))
        fmt = (response_format or "json").lower()
        if fmt == "text":
            return PlainTextResponse(r["text"] + "\n")
        if fmt in ("srt", "vtt"):
            sep = "," if fmt == "srt" else "."
            lines = ["WEBVTT", ""] if fmt == "vtt" else []
            for s in r["segments"]:
                if fmt == "srt":
                    lines.append(str(s["id"] + 1))
                lines += [f"{_stamp(s['start'], sep)} --> {_stamp(s['end'], sep)}", s["text"].strip(), ""]
            return PlainTextResponse("\n".join(lines))
        if fmt == "verbose_json":
            return {"task": r["task"], "language": r["language"], "duration": r["duration"], "text": r["text"],
                    "segments": [{k: s[k] for k in ("id", "start", "end", "text", "tokens")} for s in r["segments"]]}
        if fmt != "json":
            return _err(400, f"unknown response_format {response_format!r}")
        return {"text": r["text"]}

    @app.post("/v1/audio/transcriptions")
    @app.post("/audio/transcriptions")
    async def transcriptions(file: UploadFile = File(...), model: str = Form(None), language: str = Form(None),
                             response_format: str = Form("json"), prompt: str = Form(None), temperature: float = Form(0.0)):
        return await _run(file, language, response_format, "transcribe")

    @app.post("/v1/audio/translations")
    @app.post("/audio/translations")
    async def translations(file: UploadFile = File(...), model: str = Form(None), response_format: str = Form("json"),
                           prompt: str = Form(None), temperature: float = Form(0.0)):
        return await _run(file, None, response_format, "translate")

    @app.post("/v1/audio/speech")
    @app.post("/audio/speech")
    async def speech():
        return _err(501, "text-to-speech is not available: this server hosts a speech-to-text model", "not_supported")

    return app
