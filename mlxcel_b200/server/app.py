"""FastAPI application: OpenAI, Anthropic and llama-server compatible routes.

Route inventory follows the reference's (src/server/app.rs:275-560): ``/v1/chat/completions``,
``/v1/completions``, ``/v1/responses``, ``/v1/messages`` (+ ``/count_tokens``), ``/v1/embeddings``,
``/v1/models``, native ``/completion``, ``/tokenize``, ``/detokenize``, ``/apply-template``,
``/infill``, ``/props``, ``/slots``, ``/metrics``, ``/health``, ``/v1/cache/{stats,reset}``,
``/lora-adapters``. Streaming uses server-sent events.
"""
from __future__ import annotations

import asyncio
import json
import os
import time
import uuid

from fastapi import FastAPI, Request
from fastapi.responses import JSONResponse, PlainTextResponse, StreamingResponse

from ..engine import SamplingParams
from .chat_template import TemplateRenderError, render_chat
from .structured import constraint_from_request
from .tool_calls import IncrementalToolCallStreamer, parse_tool_calls, split_reasoning
from .worker import GenRequest, ModelWorker


def _err(status: int, message: str, etype: str = "invalid_request_error"):
    return JSONResponse(status_code=status, content={"error": {"message": message, "type": etype, "code": status}})


def sampling_from_body(b: dict, default_max: int = 512) -> SamplingParams:
    g = b.get
    stop = g("stop") or []
    if isinstance(stop, str):
        stop = [stop]
    mt = g("max_completion_tokens", g("max_tokens", g("n_predict", default_max)))
    if mt is None or int(mt) < 0:
        mt = default_max
    lb = g("logit_bias") or {}
    if isinstance(lb, list):   # llama-server form [[id, bias], ...]
        lb = {int(k): (float("-inf") if v is False else float(v)) for k, v in lb}
    else:
        lb = {int(k): float(v) for k, v in lb.items()}
    return SamplingParams(
        max_tokens=int(mt), temperature=float(g("temperature", 0.8) if g("temperature") is not None else 0.8),
        top_k=int(g("top_k", 0) or 0), top_p=float(g("top_p", 1.0) if g("top_p") is not None else 1.0),
        min_p=float(g("min_p", 0.0) or 0.0), typical_p=float(g("typical_p", g("typ_p", 1.0)) or 1.0),
        top_n_sigma=float(g("top_n_sigma", 0.0) or 0.0),
        repetition_penalty=float(g("repetition_penalty", g("repeat_penalty", 1.0)) or 1.0),
        repetition_context_size=int(g("repetition_context_size", g("repeat_last_n", 64)) or 64),
        frequency_penalty=float(g("frequency_penalty", 0.0) or 0.0),
        presence_penalty=float(g("presence_penalty", 0.0) or 0.0),
        dry_multiplier=float(g("dry_multiplier", 0.0) or 0.0), dry_base=float(g("dry_base", 1.75) or 1.75),
        dry_allowed_length=int(g("dry_allowed_length", 2) or 2),
        xtc_probability=float(g("xtc_probability", 0.0) or 0.0), xtc_threshold=float(g("xtc_threshold", 0.1) or 0.1),
        mirostat=int(g("mirostat", 0) or 0), mirostat_tau=float(g("mirostat_tau", 5.0) or 5.0),
        mirostat_eta=float(g("mirostat_eta", 0.1) or 0.1), dynatemp_range=float(g("dynatemp_range", 0.0) or 0.0),
        dynatemp_exponent=float(g("dynatemp_exponent", 1.0) or 1.0),
        seed=(int(g("seed")) if g("seed") is not None and int(g("seed")) >= 0 else None), stop=list(stop),
        ignore_eos=bool(g("ignore_eos", False)), logprobs=bool(g("logprobs", False)) or bool(g("n_probs", 0)),
        top_logprobs=int(g("top_logprobs", 0) or 0), logit_bias=lb, min_tokens=int(g("min_tokens", 0) or 0),
        loop_max_pattern=int(g("max_pattern_size", 0) or 0), loop_min_pattern=int(g("min_pattern_size", 4) or 4),
        loop_min_count=int(g("min_count", 8) or 8),
        thinking_budget=_thinking_budget(b, int(mt)),
    )


def _thinking_budget(b: dict, max_tokens: int) -> int | None:
    """Per-request thinking budget (primary spelling ``thinking_budget_tokens``, vLLM's
    ``thinking_token_budget`` and Qwen's ``thinking_budget``): -1 / absent = unbounded, 0 = close the
    block at once, N > 0 = cap. Other negatives and caps beyond ``max_tokens`` are request errors
    (src/server/thinking_budget.rs value rules)."""
    raw = b.get("thinking_budget_tokens", b.get("thinking_token_budget", b.get("thinking_budget")))
    if raw is None:
        return None
    try:
        v = int(raw)
    except (TypeError, ValueError):
        raise ValueError(f"thinking_budget_tokens must be an integer (got {raw!r})")
    if v < -1:
        raise ValueError(f"thinking_budget_tokens must be >= -1 (got {v}); use -1 for unlimited, 0 for immediate "
                         f"end, or a positive cap")
    if v > max_tokens > 0:
        raise ValueError(f"thinking_budget_tokens ({v}) exceeds max_tokens ({max_tokens})")
    return v          # -1 stays explicit: it switches a server-side default off for this request


class ServerState:
    def __init__(self, worker: ModelWorker, tokenizer, model_id: str, api_keys: set[str] | None = None,
                 chat_template: str | None = None):
        self.worker, self.tokenizer, self.model_id = worker, tokenizer, model_id
        self.api_keys = api_keys or set()
        self.chat_template = chat_template or getattr(tokenizer, "chat_template", None)
        self.started = time.time()
        from .extras import ResponsesStore
        self.responses = ResponsesStore()             # LRU + TTL (responses_store.rs)
        self.lora = None      # LoraManager when the weights are dense
        self.slot_save_path: str | None = None     # --slot-save-path: directory for /slots/{id}?action=save

    def render(self, messages, tools=None, **kw) -> str:
        return render_chat(messages, self.chat_template, tools=tools,
                           bos_token=getattr(self.tokenizer, "bos_token", "") or "",
                           eos_token=getattr(self.tokenizer, "eos_token", "") or "", **kw)

    def eos_params(self, sp: SamplingParams) -> SamplingParams:
        ids = [i for i in self.tokenizer.eos_ids() if i is not None]
        sp.stop_token_ids = sorted(set(sp.stop_token_ids) | set(ids))
        # thinking budget: request value, else the live / start-up default; the block's token ids come
        # from the tokenizer (no ids, nothing to enforce)
        settings = getattr(self, "settings", None) or {}
        if sp.thinking_budget is None:
            d = settings.get("thinking_budget", getattr(self, "default_thinking_budget", None))
            sp.thinking_budget = None if d in (None, -1) else int(d)
        sp.think_start_id = getattr(self.tokenizer, "think_open", None)
        sp.think_end_id = getattr(self.tokenizer, "think_close", None)
        from .extras import REQUEST_CTX
        ctx = REQUEST_CTX.get()
        if ctx.get("priority") and not sp.priority:
            sp.priority = int(ctx["priority"])        # X-Priority header -> priority lane of the queue
        return sp


class PromptWithMedia(list):
    """Prompt token ids that carry the decoded images of their placeholder tokens to the worker."""

    media: list | None = None


async def _generate(state: ServerState, prompt_ids, sp, constraint=None, public_id: str | None = None):
    """Async generator of GenEvents for one request. ``public_id`` (a chat / response id) makes the
    request reachable for ``/v1/chat/completions/control`` and ``/v1/responses/{id}/cancel``."""
    q: asyncio.Queue = asyncio.Queue()
    req = GenRequest(prompt_ids=prompt_ids, params=state.eos_params(sp), loop=asyncio.get_running_loop(), out=q,
                     constraint=constraint, request_id=uuid.uuid4().hex, media=getattr(prompt_ids, "media", None))
    inflight = getattr(state, "inflight", None)
    if public_id and inflight is not None:
        inflight[public_id] = req
    state.worker.submit(req)
    try:
        while True:
            ev = await q.get()
            if ev.kind == "done" and getattr(state, "hist", None) and ev.timings:
                state.hist["ttft"].observe(ev.timings["prompt_ms"] / 1e3)
                state.hist["decode_tps"].observe(ev.timings["predicted_per_second"])
            yield ev
            if ev.kind in ("done", "error"):
                return
    finally:
        if public_id and inflight is not None:
            inflight.pop(public_id, None)
        if req.seq_id is not None and req.seq_id in state.worker.by_seq:
            state.worker.cancel(req)


def _sse(obj) -> bytes:
    return f"data: {json.dumps(obj, ensure_ascii=False)}\n\n".encode()


def _finish_openai(reason: str, has_tools: bool) -> str:
    if has_tools:
        return "tool_calls"
    return {"stop": "stop", "stop_sequence": "stop", "length": "length", "repetition_loop": "stop",
            "cancelled": "stop"}.get(reason, "stop")


def create_app(state: ServerState) -> FastAPI:
    app = FastAPI(title="mlxcel_b200", version="0.1.0")
    tk = state.tokenizer

    @app.middleware("http")
    async def auth(request: Request, call_next):
        if state.api_keys and request.url.path not in ("/health", "/metrics"):
            key = request.headers.get("authorization", "").removeprefix("Bearer ").strip() or \
                request.headers.get("x-api-key", "")
            if key not in state.api_keys:
                return _err(401, "invalid API key", "authentication_error")
        return await call_next(request)

    from .extras import install_extras, tee_stream, REQUEST_CTX
    install_extras(app, state)      # CORS (outermost: preflights never reach the key check), logging, settings, ...

    @app.exception_handler(ValueError)
    async def bad_request(request: Request, exc: ValueError):
        return _err(400, str(exc))

    _parse_sampling = globals()["sampling_from_body"]

    def sampling_from_body(b: dict, default_max: int = 512) -> SamplingParams:
        """Request body -> sampling parameters, with the live defaults of ``/v1/settings`` filled in."""
        st = state.settings
        if st.get("default_max_tokens") and not any(k in b for k in ("max_tokens", "max_completion_tokens", "n_predict")):
            default_max = int(st["default_max_tokens"])
        if st.get("default_temperature") is not None and b.get("temperature") is None:
            b = {**b, "temperature": st["default_temperature"]}
        return _parse_sampling(b, default_max)

    # ------------------------------------------------------------------ basic
    @app.get("/health")
    async def health():
        if not state.worker.healthy:
            return JSONResponse(status_code=503, content={"status": "error"})
        return {"status": "ok"}

    @app.get("/v1/models")
    @app.get("/models")
    async def models():
        return {"object": "list", "data": [{"id": state.model_id, "object": "model", "created": int(state.started),
                                            "owned_by": "mlxcel_b200"}]}

    @app.get("/props")
    async def props():
        e = state.worker.view()
        return {"model_path": state.model_id, "total_slots": e.ecfg.max_batch, "chat_template": state.chat_template or "",
                "is_sleeping": bool(getattr(state.worker, "sleeping", False)),
                "default_generation_settings": {"n_ctx": e.ecfg.max_model_len, "params": {}},
                "build_info": "mlxcel_b200 0.1.0", "bos_token": getattr(tk, "bos_token", None),
                "eos_token": getattr(tk, "eos_token", None)}

    @app.get("/slots")
    async def slots():
        return state.worker.slots()

    @app.post("/slots/{slot_id}")
    async def slot_action(slot_id: int, request: Request, action: str = ""):
        """llama-server slot persistence (reference src/server/slot_persist.rs:15-60): ``save`` writes the
        token stream of the slot's last occupant to ``<slot-save-path>/<filename>``, ``restore`` reads
        one back and prefills it so that its KV blocks are in the prefix cache again, ``erase`` drops
        the cached prefixes."""
        if action not in ("save", "restore", "erase"):
            return _err(400, "action must be save, restore or erase")
        t0 = time.perf_counter()
        if action == "erase":
            n = state.worker.run_exclusive(lambda: state.worker.engine.bm.reset_prefix_cache(), name="cache_reset")
            return dict(id_slot=slot_id, n_erased=n)
        if not state.slot_save_path:
            return _err(501, "This server does not support slots action. Start it with `--slot-save-path`",
                        "not_supported_error")
        try:
            body = await request.json()
        except Exception:
            body = {}
        name = str(body.get("filename", ""))
        if not name or name != os.path.basename(name) or name.startswith("."):
            return _err(400, "filename must be a plain file name")
        path = os.path.join(state.slot_save_path, name)
        if action == "save":
            toks = state.worker.recent.get(slot_id)
            if toks is None:
                return _err(404, f"slot {slot_id} has no finished sequence to save")
            data = json.dumps(dict(model=state.model_id, tokens=toks)).encode()
            os.makedirs(state.slot_save_path, exist_ok=True)
            with open(path, "wb") as f:
                f.write(data)
            return dict(id_slot=slot_id, filename=name, n_saved=len(toks), n_written=len(data),
                        timings=dict(save_ms=(time.perf_counter() - t0) * 1e3))
        if not os.path.exists(path):
            return _err(404, f"no saved slot {name!r}")
        with open(path, "rb") as f:
            raw = f.read()
        saved = json.loads(raw)
        if saved.get("model") != state.model_id:
            return _err(400, f"slot file belongs to model {saved.get('model')!r}")
        toks = [int(t) for t in saved["tokens"]]
        async for ev in _generate(state, toks, SamplingParams(max_tokens=1, temperature=0.0)):
            if ev.kind == "error":
                return _err(500, ev.text or "restore failed", "server_error")
        return dict(id_slot=slot_id, filename=name, n_restored=len(toks), n_read=len(raw),
                    timings=dict(restore_ms=(time.perf_counter() - t0) * 1e3))

    @app.post("/v1/internal/kv/export")
    async def kv_export(body: dict):
        """Prefill role of a disaggregated deployment: prefill the prompt (text or token ids) and return
        its KV blocks as one binary blob for ``/v1/internal/kv/import`` of a decode-role server."""
        from fastapi.responses import Response

        from ..engine.handoff import export_prefix
        prompt = body.get("prompt", body.get("tokens"))
        if prompt is None:
            return _err(400, "prompt (text or token ids) is required")
        ids = _prompt_ids(prompt)
        try:
            blob = state.worker.run_exclusive(lambda: export_prefix(state.worker.engine, ids))
        except ValueError as e:
            return _err(400, str(e))
        return Response(content=blob, media_type="application/octet-stream",
                        headers={"x-kv-tokens": str(len(ids))})

    @app.post("/v1/internal/kv/import")
    async def kv_import(request: Request):
        from ..engine.handoff import import_prefix
        blob = await request.body()
        try:
            n = state.worker.run_exclusive(lambda: import_prefix(state.worker.engine, blob))
        except ValueError as e:
            return _err(400, str(e))
        return {"cached_tokens": n}

    @app.get("/metrics")
    async def metrics():
        from .metrics import render_metrics
        return PlainTextResponse(render_metrics(state))

    @app.get("/v1/cache/stats")
    async def cache_stats():
        return dict(state.worker.view().bm.stats())

    @app.post("/v1/cache/reset")
    async def cache_reset():
        return {"dropped_blocks": state.worker.engine.bm.reset_prefix_cache()}

    @app.get("/lora-adapters")
    async def lora_adapters():
        return state.lora.listing() if state.lora is not None else []

    @app.post("/lora-adapters")
    async def lora_set(body: list[dict]):
        """llama-server contract: ``[{"id": 0, "scale": 0.5}, ...]`` sets live adapter scales; an
        entry with ``"path"`` attaches a new adapter. Applied between engine steps."""
        if state.lora is None:
            return _err(400, "the server was started without LoRA support (dense weights are required)")

        def apply():
            for e in body:
                if "path" in e and e.get("id") not in state.lora.adapters:
                    state.lora.add(e["path"], float(e.get("scale", 1.0)), e.get("id"))
                else:
                    state.lora.set_scale(int(e["id"]), float(e.get("scale", 1.0)))
            state.worker.engine.bm.reset_prefix_cache()     # cached KV belongs to the old weights
            return state.lora.listing()

        try:
            return await asyncio.get_running_loop().run_in_executor(None, state.worker.run_exclusive, apply)
        except (KeyError, ValueError, FileNotFoundError) as e:
            return _err(400, f"{type(e).__name__}: {e}")

    @app.get("/")
    @app.get("/ui")
    async def webui():
        from fastapi.responses import HTMLResponse
        from .webui import INDEX_HTML
        return HTMLResponse(INDEX_HTML)

    @app.api_route("/tools", methods=["GET", "POST"])
    @app.api_route("/cors-proxy", methods=["GET", "POST"])
    async def disabled_llama_server_routes():
        return _err(403, "this endpoint is disabled", "forbidden")

    @app.get("/v1/internal/mtp-policy")
    async def mtp_policy():
        eng = state.worker.engine
        dr = getattr(eng, "drafter", None)
        st = eng.stats
        pol = getattr(eng, "spec_policy", None)
        return {"drafter": type(dr).__name__ if dr is not None else None,
                "max_draft": max(0, eng.spec_k - 1) if dr is not None else 0,
                "rounds": st.get("spec_rounds", 0), "drafted": st.get("spec_drafted", 0),
                "accepted": st.get("spec_accepted", 0),
                "acceptance": (st.get("spec_accepted", 0) / st["spec_drafted"]) if st.get("spec_drafted") else None,
                "policy": pol.snapshot() if pol is not None else None}

    @app.post("/v1/internal/mtp-policy")
    async def mtp_policy_set(body: dict):
        """``{"mode": "on" | "off" | "auto" | "reset"}``: pin speculation on or off, start a new profile, or
        also forget the persisted verdict (reference docs/mtp-policy-api.md)."""
        pol = getattr(state.worker.engine, "spec_policy", None)
        if pol is None:
            return _err(400, "no speculative drafter is attached to this server")
        try:
            state.worker.run_exclusive(lambda: pol.force(str(body.get("mode", ""))))
        except ValueError as e:
            return _err(400, str(e))
        return await mtp_policy()

    @app.post("/v1/rerank")
    @app.post("/v1/reranking")
    @app.post("/rerank")
    async def rerank(body: dict):
        """Reranking with a decoder LM: cosine similarity between last-token embeddings of the query and
        every document, or with ``"mode": "generative"`` the probability of "yes" after the yes/no
        judgement prompt (Qwen3-Reranker style). Cross-encoder checkpoints are served by the encoder app."""
        from .embeddings import embed_texts
        query, docs = body.get("query", ""), list(body.get("documents", []))
        docs_txt = [d if isinstance(d, str) else d.get("text", "") for d in docs]
        if not query or not docs_txt:
            return _err(400, "query and documents are required")
        if body.get("mode") == "generative":       # yes/no judgement prompt instead of embedding cosine
            from ..engine.scoring import generative_rerank
            eng = state.worker.engine
            scores = await asyncio.get_running_loop().run_in_executor(
                None, lambda: generative_rerank(eng.model, eng.cfg, tk, query, docs_txt, body.get("instruction"),
                                                eng.ecfg.block_size, eng.ecfg.max_model_len - 1))
            order = sorted(range(len(scores)), key=lambda i: -scores[i])[: int(body.get("top_n") or len(scores))]
            return {"model": state.model_id, "object": "list", "results": [
                {"index": i, "relevance_score": scores[i],
                 **({"document": {"text": docs_txt[i]}} if body.get("return_documents") else {})} for i in order]}
        vecs, ntok = await asyncio.get_running_loop().run_in_executor(None, embed_texts, state, [query, *docs_txt])
        qv = vecs[0]
        scores = [sum(a * b for a, b in zip(qv, v)) for v in vecs[1:]]
        order = sorted(range(len(scores)), key=lambda i: -scores[i])
        top_n = int(body.get("top_n") or len(order))
        res = [{"index": i, "relevance_score": scores[i],
                **({"document": {"text": docs_txt[i]}} if body.get("return_documents") else {})} for i in order[:top_n]]
        return {"model": state.model_id, "object": "list", "results": res,
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/tokenize")
    async def tokenize(body: dict):
        ids = tk.encode(body.get("content", ""), add_special_tokens=bool(body.get("add_special", False)))
        if body.get("with_pieces"):
            return {"tokens": [{"id": i, "piece": tk.decode([i], skip_special_tokens=False)} for i in ids]}
        return {"tokens": ids}

    @app.post("/detokenize")
    async def detokenize(body: dict):
        return {"content": tk.decode(body.get("tokens", []))}

    @app.post("/apply-template")
    async def apply_template(body: dict):
        try:
            return {"prompt": state.render(body.get("messages", []), **(body.get("chat_template_kwargs") or {}))}
        except TemplateRenderError as e:
            return _err(400, str(e))

    @app.post("/v1/messages/count_tokens")
    async def count_tokens(body: dict):
        msgs = _anthropic_messages(body)
        return {"input_tokens": len(tk.encode(state.render(msgs)))}

    # ------------------------------------------------------------------ completions
    async def _run_text(prompt_ids, sp, constraint=None, public_id=None):
        text, lps, toks, final = [], [], [], None
        async for ev in _generate(state, prompt_ids, sp, constraint, public_id=public_id):
            if ev.kind == "token":
                text.append(ev.text)
                toks.append(ev.token_id)
                if ev.logprob is not None:
                    lps.append(ev.logprob)
            elif ev.kind == "done":
                text.append(ev.text)
                final = ev
            elif ev.kind == "error":
                raise RuntimeError(ev.error)
        return "".join(text), toks, lps, final

    def _prompt_ids(prompt) -> list[int]:
        if isinstance(prompt, list) and prompt and isinstance(prompt[0], int):
            return prompt
        if isinstance(prompt, list):
            prompt = prompt[0] if prompt else ""
        ids = tk.encode(prompt, add_special_tokens=True)
        return ids or [getattr(tk, "bos_token_id", 0) or 0]

    async def _run_n(body: dict, ids, sp, constraint_factory):
        """``n`` independent samples of one prompt, run concurrently (the engine batches them and the prefix
        cache shares the prompt); sample i uses ``seed + i`` when a seed was given. Constraints are stateful,
        so each sample gets its own."""
        import copy
        n = max(1, min(int(body.get("n", 1) or 1), state.worker.engine.ecfg.max_batch))
        sps = []
        for i in range(n):
            spi = copy.deepcopy(sp)
            if spi.seed is not None:
                spi.seed = spi.seed + i
            sps.append(spi)
        return await asyncio.gather(*(_run_text(ids, spi, constraint_factory()) for spi in sps))

    def _sum_usage(runs) -> dict:
        u = dict(runs[0][3].usage)
        extra = sum(r[3].usage["completion_tokens"] for r in runs[1:])
        u["completion_tokens"] += extra
        u["total_tokens"] += extra
        return u

    @app.post("/v1/completions")
    async def completions(body: dict):
        sp = sampling_from_body(body, 16)
        ids = _prompt_ids(body.get("prompt", ""))
        cid, created = "cmpl-" + uuid.uuid4().hex[:24], int(time.time())
        try:
            constraint = constraint_from_request(tk, response_format=body.get("response_format"),
                                                 grammar=body.get("grammar"), json_schema=body.get("json_schema"))
        except ValueError as e:
            return _err(400, str(e))
        if body.get("stream"):
            async def gen():
                async for ev in _generate(state, ids, sp, constraint):
                    if ev.kind == "token" and ev.text:
                        yield _sse({"id": cid, "object": "text_completion", "created": created, "model": state.model_id,
                                    "choices": [{"index": 0, "text": ev.text, "finish_reason": None}]})
                    elif ev.kind == "done":
                        yield _sse({"id": cid, "object": "text_completion", "created": created, "model": state.model_id,
                                    "choices": [{"index": 0, "text": ev.text,
                                                 "finish_reason": _finish_openai(ev.finish_reason, False)}],
                                    "usage": ev.usage})
                    elif ev.kind == "error":
                        yield _sse({"error": {"message": ev.error}})
                yield b"data: [DONE]\n\n"
            return StreamingResponse(gen(), media_type="text/event-stream")
        if body.get("echo"):
            # prompt scoring (what evaluation harnesses ask for): the prompt comes back with the log-probability
            # of each of its tokens given the ones before; ``max_tokens: 0`` scores without generating
            from ..engine.scoring import sequence_logprobs
            eng = state.worker.engine
            plp = await asyncio.get_running_loop().run_in_executor(
                None, lambda: sequence_logprobs(eng.model, eng.cfg, ids, eng.ecfg.block_size).tolist())
            ptoks = [tk.decode([t], skip_special_tokens=False) for t in ids]
            offs, pos = [], 0
            for piece in ptoks:
                offs.append(pos)
                pos += len(piece)
            prompt_text = tk.decode(ids, skip_special_tokens=False)
            gen_text, gen_toks, gen_lps, usage, reason = "", [], [], None, "length"
            if int(body.get("max_tokens", 16) or 0) > 0:
                try:
                    gen_text, gen_toks, gen_lps, fin = await _run_text(ids, sp, constraint)
                except (RuntimeError, ValueError) as e:
                    return _err(400, str(e))
                usage, reason = fin.usage, _finish_openai(fin.finish_reason, False)
            choice = {"index": 0, "text": prompt_text + gen_text, "finish_reason": reason,
                      "logprobs": {"tokens": ptoks + [tk.decode([t]) for t in gen_toks],
                                   "token_logprobs": [None] + plp + (gen_lps if sp.logprobs else [None] * len(gen_toks)),
                                   "text_offset": offs}}
            return {"id": cid, "object": "text_completion", "created": created, "model": state.model_id, "choices": [choice],
                    "usage": usage or {"prompt_tokens": len(ids), "completion_tokens": 0, "total_tokens": len(ids)}}
        try:
            runs = await _run_n(body, ids, sp, lambda: constraint_from_request(
                tk, response_format=body.get("response_format"), grammar=body.get("grammar"), json_schema=body.get("json_schema")))
        except (RuntimeError, ValueError) as e:
            return _err(400, str(e))
        choices = []
        for i, (text, toks, lps, fin) in enumerate(runs):
            choice = {"index": i, "text": text, "finish_reason": _finish_openai(fin.finish_reason, False)}
            if sp.logprobs:
                choice["logprobs"] = {"token_logprobs": lps, "tokens": [tk.decode([t]) for t in toks]}
            choices.append(choice)
        return {"id": cid, "object": "text_completion", "created": created, "model": state.model_id,
                "choices": choices, "usage": _sum_usage(runs), "timings": runs[0][3].timings}

    @app.post("/completion")
    @app.post("/completions")
    async def native_completion(body: dict):
        sp = sampling_from_body(body, 512)
        ids = _prompt_ids(body.get("prompt", ""))
        try:
            constraint = constraint_from_request(tk, grammar=body.get("grammar"), json_schema=body.get("json_schema"))
        except Exception as e:
            return _err(400, f"grammar: {e}")
        if body.get("stream"):
            async def gen():
                async for ev in _generate(state, ids, sp, constraint):
                    if ev.kind == "token":
                        yield _sse({"content": ev.text, "tokens": [ev.token_id], "stop": False})
                    elif ev.kind == "done":
                        yield _sse({"content": ev.text, "stop": True, "stop_type": _stop_type(ev.finish_reason),
                                    "tokens_predicted": ev.usage["completion_tokens"],
                                    "tokens_evaluated": ev.usage["prompt_tokens"], "timings": ev.timings})
                    elif ev.kind == "error":
                        yield _sse({"error": {"message": ev.error}})
            return StreamingResponse(gen(), media_type="text/event-stream")
        try:
            text, toks, lps, fin = await _run_text(ids, sp, constraint)
        except (RuntimeError, ValueError) as e:
            return _err(400, str(e))
        return {"content": text, "tokens": toks, "id_slot": 0, "stop": True, "model": state.model_id,
                "stop_type": _stop_type(fin.finish_reason), "stopping_word": "",
                "tokens_predicted": fin.usage["completion_tokens"], "tokens_evaluated": fin.usage["prompt_tokens"],
                "tokens_cached": fin.timings["cache_n"], "truncated": False, "timings": fin.timings,
                "generation_settings": {"n_predict": sp.max_tokens, "temperature": sp.temperature, "top_k": sp.top_k,
                                        "top_p": sp.top_p, "min_p": sp.min_p, "seed": sp.seed}}

    @app.post("/infill")
    async def infill(body: dict):
        fim = getattr(tk, "fim", {}) or {}
        if not all(fim.get(k) is not None for k in ("prefix", "suffix", "middle")):
            return _err(501, "this model's tokenizer has no fill-in-the-middle tokens", "not_supported")
        ids = [fim["prefix"]] + tk.encode(body.get("input_prefix", "")) + [fim["suffix"]] + \
            tk.encode(body.get("input_suffix", "")) + [fim["middle"]]
        text, toks, lps, fin = await _run_text(ids, sampling_from_body(body, 128))
        return {"content": text, "tokens_predicted": fin.usage["completion_tokens"], "timings": fin.timings}

    # ------------------------------------------------------------------ chat completions
    def _load_audio(src):
        """An ``input_audio`` part's base64 payload (or a ``data:`` URL) → 16 kHz mono samples."""
        import base64

        from ..audio.wav import decode_audio
        if not isinstance(src, str):
            raise ValueError("audio must be base64 text or a data: URL")
        if src.startswith("data:"):
            src = src.partition(",")[2]
        elif src.startswith(("http://", "https://", "file://", "/")):
            raise ValueError("audio must be sent inline (base64); URLs and paths are not fetched")
        try:
            return decode_audio(base64.b64decode(src), 16000)
        except Exception as e:
            raise ValueError(f"audio could not be decoded: {e}") from None

    def _chat_prompt(body: dict):
        tools = body.get("tools")
        kwargs = dict(body.get("chat_template_kwargs") or {})
        if body.get("reasoning_effort"):
            kwargs.setdefault("reasoning_effort", body["reasoning_effort"])
        messages, images = body.get("messages", []), []
        vision = getattr(state.worker, "vision", None)
        audio_in = getattr(vision, "modality", "image") == "audio"
        part_types = ("input_audio", "audio_url", "audio") if audio_in else ("image_url", "image", "input_image")
        other = ("image_url", "image", "input_image") if audio_in else ("input_audio", "audio_url", "audio")
        parts_of = lambda kinds: any(isinstance(m.get("content"), list) and any(  # noqa: E731
            isinstance(p, dict) and p.get("type") in kinds for p in m["content"]) for m in messages)
        if parts_of(other) and (vision is not None or other[0] == "input_audio"):
            raise TemplateRenderError("this model takes no audio input" if other[0] == "input_audio" else "this model takes no image input")
        has_media = parts_of(part_types)
        if has_media:
            if vision is None:
                raise TemplateRenderError("this model takes no image input")
            from .chat_template import extract_media
            messages, sources = extract_media(messages, vision.placeholder_text, state.chat_template, audio=audio_in)
            try:
                if audio_in:
                    images = [_load_audio(src) for src in sources]
                else:
                    from ..multimodal import load_image
                    images = [load_image(src, media_root=getattr(state, "media_path", None),
                                         allow_remote=bool(getattr(state, "allow_remote_media", False))) for src in sources]
            except ValueError as e:
                raise TemplateRenderError(str(e)) from e
        text = state.render(messages, tools=tools, **kwargs)
        ids = tk.encode(text, add_special_tokens=False)
        ids = ids or [getattr(tk, "bos_token_id", 0) or 0]
        if images:
            ids = PromptWithMedia(ids)
            ids.media = images
            n_ph = sum(1 for t in ids if t == vision.image_token_id)
            if n_ph != len(images):
                raise TemplateRenderError(f"the rendered prompt has {n_ph} media placeholders for {len(images)} attachments")
        return ids, tools

    @app.post("/v1/chat/completions")
    @app.post("/chat/completions")
    async def chat_completions(body: dict):
        try:
            ids, tools = _chat_prompt(body)
        except TemplateRenderError as e:
            return _err(400, str(e))
        sp = sampling_from_body(body, 512)
        try:
            constraint = constraint_from_request(tk, response_format=body.get("response_format"),
                                                 grammar=body.get("grammar"))
        except Exception as e:
            return _err(400, f"response_format: {e}")
        allowed = {t["function"]["name"] for t in tools or [] if t.get("type") == "function"} or None
        use_tools = bool(tools) and body.get("tool_choice") != "none"
        cid, created = "chatcmpl-" + uuid.uuid4().hex[:24], int(time.time())
        base = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": state.model_id}
        if body.get("stream"):
            include_usage = bool((body.get("stream_options") or {}).get("include_usage"))

            async def gen():
                # tool calls stream as they are generated: the name first, then argument fragments
                filt = IncrementalToolCallStreamer(allowed) if use_tools else None
                yield _sse({**base, "choices": [{"index": 0, "delta": {"role": "assistant", "content": ""},
                                                 "finish_reason": None}]})
                async for ev in _generate(state, ids, sp, constraint, public_id=cid):
                    if ev.kind in ("token", "done"):
                        text, calls = (filt.feed(ev.text, final=ev.kind == "done") if filt else (ev.text, []))
                        if text:
                            yield _sse({**base, "choices": [{"index": 0, "delta": {"content": text},
                                                             "finish_reason": None}]})
                        for d in calls:
                            yield _sse({**base, "choices": [{"index": 0, "delta": {"tool_calls": [d]},
                                                             "finish_reason": None}]})
                        if ev.kind == "done":
                            yield _sse({**base, "choices": [{"index": 0, "delta": {},
                                                             "finish_reason": _finish_openai(ev.finish_reason, bool(filt and filt.n))}],
                                        "timings": ev.timings})
                            if include_usage:
                                yield _sse({**base, "choices": [], "usage": ev.usage})
                    elif ev.kind == "error":
                        yield _sse({"error": {"message": ev.error, "type": "server_error"}})
                yield b"data: [DONE]\n\n"
            conv = REQUEST_CTX.get().get("conversation_id")
            return StreamingResponse(tee_stream(state, gen(), conv), media_type="text/event-stream",
                                     headers={"X-Conversation-Id": conv} if conv else None)
        try:
            runs = await _run_n(body, ids, sp, lambda: constraint_from_request(
                tk, response_format=body.get("response_format"), grammar=body.get("grammar")))
        except (RuntimeError, ValueError) as e:
            return _err(400, str(e))
        choices = []
        for i, (text, toks, lps, fin) in enumerate(runs):
            reasoning, answer = split_reasoning(text)
            calls = []
            if use_tools:
                answer, calls = parse_tool_calls(answer, allowed)
            msg = {"role": "assistant", "content": answer if (answer or not calls) else None}
            if reasoning:
                msg["reasoning_content"] = reasoning
            if calls:
                msg["tool_calls"] = [c.to_openai() for c in calls]
            choice = {"index": i, "message": msg, "finish_reason": _finish_openai(fin.finish_reason, bool(calls))}
            if sp.logprobs:
                choice["logprobs"] = {"content": [{"token": tk.decode([t]), "logprob": lp} for t, lp in zip(toks, lps)]}
            choices.append(choice)
        return {"id": cid, "object": "chat.completion", "created": created, "model": state.model_id,
                "choices": choices, "usage": _sum_usage(runs), "timings": runs[0][3].timings}

    # ------------------------------------------------------------------ responses API
    def _responses_messages(body: dict) -> list[dict]:
        return _responses_input_messages(state, body)

    @app.post("/v1/responses")
    async def responses(body: dict):
        msgs = _responses_messages(body)
        try:
            ids = tk.encode(state.render(msgs), add_special_tokens=False)
        except TemplateRenderError as e:
            return _err(400, str(e))
        b2 = dict(body)
        b2["max_tokens"] = body.get("max_output_tokens", 512)
        sp = sampling_from_body(b2, 512)
        rid = "resp_" + uuid.uuid4().hex[:24]
        created = int(time.time())

        async def run() -> dict:
            text, toks, lps, fin = await _run_text(ids or [0], sp, public_id=rid)
            reasoning, answer = split_reasoning(text)
            out = {"id": rid, "object": "response", "created_at": created, "status": "completed",
                   "model": state.model_id,
                   "output": [{"type": "message", "id": "msg_" + uuid.uuid4().hex[:24], "role": "assistant",
                               "status": "completed",
                               "content": [{"type": "output_text", "text": answer, "annotations": []}]}],
                   "output_text": answer,
                   "usage": {"input_tokens": fin.usage["prompt_tokens"], "output_tokens": fin.usage["completion_tokens"],
                             "total_tokens": fin.usage["total_tokens"]}}
            if body.get("store", True) or body.get("background"):
                cur = state.responses.get(rid)
                if cur is not None and cur.get("status") == "cancelled":
                    return cur                      # cancelled while it ran: keep the cancelled record
                state.responses[rid] = {**out, "_messages": msgs + [{"role": "assistant", "content": answer}]}
            return out

        if body.get("background"):
            # background mode: the response object comes back at once (status "queued"), the generation
            # runs as a task of the server; GET /v1/responses/{id} polls, POST .../cancel stops it
            stub = {"id": rid, "object": "response", "created_at": created, "status": "queued", "model": state.model_id,
                    "output": [], "background": True, "_messages": msgs}
            state.responses[rid] = stub

            async def job():
                stub["status"] = "in_progress"
                try:
                    await run()
                except asyncio.CancelledError:
                    stub["status"] = "cancelled"
                    raise
                except Exception as e:
                    cur = state.responses.get(rid) or stub
                    if cur.get("status") != "cancelled":
                        cur["status"], cur["error"] = "failed", {"message": str(e)}
                finally:
                    state.background.pop(rid, None)
            state.background[rid] = asyncio.create_task(job())
            return {k: v for k, v in stub.items() if not k.startswith("_")}
        try:
            return await run()
        except (RuntimeError, ValueError) as e:
            return _err(400, str(e))

    @app.get("/v1/responses/{rid}")
    async def get_response(rid: str):
        r = state.responses.get(rid)
        if r is None:
            return _err(404, "response not found", "not_found_error")
        return {k: v for k, v in r.items() if not k.startswith("_")}

    @app.post("/v1/responses/input_tokens")
    async def responses_input_tokens(body: dict):
        return {"input_tokens": len(tk.encode(state.render(_responses_messages(body))))}

    # ------------------------------------------------------------------ anthropic messages
    @app.post("/v1/messages")
    async def messages(body: dict):
        msgs = _anthropic_messages(body)
        try:
            ids = tk.encode(state.render(msgs), add_special_tokens=False)
        except TemplateRenderError as e:
            return _err(400, str(e))
        b2 = dict(body)
        b2["stop"] = body.get("stop_sequences") or []
        sp = sampling_from_body(b2, 1024)
        mid = "msg_" + uuid.uuid4().hex[:24]
        if body.get("stream"):
            async def gen():
                def ev(name, data):
                    return f"event: {name}\ndata: {json.dumps(data)}\n\n".encode()
                yield ev("message_start", {"type": "message_start", "message": {
                    "id": mid, "type": "message", "role": "assistant", "model": state.model_id, "content": [],
                    "usage": {"input_tokens": len(ids), "output_tokens": 0}}})
                yield ev("content_block_start", {"type": "content_block_start", "index": 0,
                                                 "content_block": {"type": "text", "text": ""}})
                async for e in _generate(state, ids or [0], sp):
                    if e.kind in ("token", "done") and e.text:
                        yield ev("content_block_delta", {"type": "content_block_delta", "index": 0,
                                                         "delta": {"type": "text_delta", "text": e.text}})
                    if e.kind == "done":
                        yield ev("content_block_stop", {"type": "content_block_stop", "index": 0})
                        yield ev("message_delta", {"type": "message_delta",
                                                   "delta": {"stop_reason": _anthropic_stop(e.finish_reason)},
                                                   "usage": {"output_tokens": e.usage["completion_tokens"]}})
                        yield ev("message_stop", {"type": "message_stop"})
            return StreamingResponse(gen(), media_type="text/event-stream")
        try:
            text, toks, lps, fin = await _run_text(ids or [0], sp)
        except (RuntimeError, ValueError) as e:
            return _err(400, str(e))
        return {"id": mid, "type": "message", "role": "assistant", "model": state.model_id,
                "content": [{"type": "text", "text": text}], "stop_reason": _anthropic_stop(fin.finish_reason),
                "usage": {"input_tokens": fin.usage["prompt_tokens"], "output_tokens": fin.usage["completion_tokens"]}}

    # ------------------------------------------------------------------ embeddings
    @app.post("/v1/embeddings")
    @app.post("/embeddings")
    async def embeddings(body: dict):
        from .embeddings import embed_texts
        inp = body.get("input", body.get("content", ""))
        texts = [inp] if isinstance(inp, str) else list(inp)
        vecs, ntok = await asyncio.get_running_loop().run_in_executor(None, embed_texts, state, texts)
        return {"object": "list", "model": state.model_id,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/embedding")
    async def embedding_native(body: dict):
        """llama-server shape: ``[{"index": i, "embedding": [...]}, ...]`` for ``content`` (string or list)."""
        from .embeddings import embed_texts
        inp = body.get("content", body.get("input", ""))
        texts = [inp] if isinstance(inp, str) else list(inp)
        vecs, _ = await asyncio.get_running_loop().run_in_executor(None, embed_texts, state, texts)
        return [{"index": i, "embedding": v} for i, v in enumerate(vecs)]

    return app


def _responses_input_messages(state, body: dict) -> list[dict]:
    """Responses API ``instructions`` / ``previous_response_id`` / ``input`` -> chat messages."""
    msgs = []
    if body.get("instructions"):
        msgs.append({"role": "system", "content": body["instructions"]})
    prev = body.get("previous_response_id")
    prev_obj = state.responses.get(prev) if prev else None
    if prev_obj is not None:
        msgs += prev_obj.get("_messages", [])
    inp = body.get("input", "")
    if isinstance(inp, str):
        msgs.append({"role": "user", "content": inp})
    else:
        for item in inp:
            c = item.get("content", "")
            if isinstance(c, list):
                c = "".join(p.get("text", "") for p in c if isinstance(p, dict))
            msgs.append({"role": item.get("role", "user"), "content": c})
    return msgs


def _stop_type(reason: str) -> str:
    return {"stop": "eos", "stop_sequence": "word", "length": "limit"}.get(reason, "none")


def _anthropic_stop(reason: str) -> str:
    return {"stop": "end_turn", "stop_sequence": "stop_sequence", "length": "max_tokens"}.get(reason, "end_turn")


def _anthropic_messages(body: dict) -> list[dict]:
    msgs = []
    sysm = body.get("system")
    if isinstance(sysm, list):
        sysm = "".join(p.get("text", "") for p in sysm)
    if sysm:
        msgs.append({"role": "system", "content": sysm})
    for m in body.get("messages", []):
        c = m.get("content", "")
        if isinstance(c, list):
            c = "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") == "text")
        msgs.append({"role": m.get("role", "user"), "content": c})
    return msgs
