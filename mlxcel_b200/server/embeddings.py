"""Text embeddings from a decoder LM: last-token (or mean) pooling of the final hidden state,
L2-normalised (the Qwen3-embedding style path of the reference, src/embeddings/)."""
from __future__ import annotations

import torch

from ..models.decoder import StepBatch


@torch.inference_mode()
def embed_texts(state, texts: list[str], pooling: str = "last") -> tuple[list[list[float]], int]:
    eng = state.worker.engine
    model, dev = eng.model, eng.device
    out, ntok = [], 0
    from ..cache.kv_pool import KVPool
    for t in texts:
        ids = state.tokenizer.encode(t, add_special_tokens=True) or [0]
        ids = ids[: eng.ecfg.max_model_len - 1]
        T = len(ids)
        ntok += T
        nb = (T + eng.ecfg.block_size - 1) // eng.ecfg.block_size
        pool = KVPool(eng.cfg, nb, eng.ecfg.block_size, device=dev, tp_size=model.comm.tp_size,
                      num_layers=len(model.w.layers), dtype=model.w.final_norm.dtype)
        b = StepBatch(token_ids=torch.tensor(ids, dtype=torch.int32, device=dev),
                      positions=torch.arange(T, dtype=torch.int32, device=dev),
                      slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), num_prefill_seqs=1,
                      pf_block_tables=torch.arange(nb, dtype=torch.int32, device=dev)[None],
                      pf_cu_q=torch.tensor([0, T], dtype=torch.int32, device=dev),
                      pf_context_lens=torch.tensor([T], dtype=torch.int32, device=dev), pf_max_q_len=T)
        h = model.forward_hidden(b, pool.layers)
        if hasattr(model, "_norm"):          # the embedding is taken after the model's final norm
            h = model._norm(h, model.w.final_norm, model.w.extra.get("final_norm_b"))
        h = h.float()
        v = h[-1] if pooling == "last" else h.mean(0)
        v = v / v.norm().clamp_min(1e-12)
        out.append(v.cpu().tolist())
    return out, ntok


def pair_ids(tokenizer, query: str, doc: str, max_len: int = 512) -> tuple[list[int], list[int]]:
    """``[CLS] query [SEP] doc [SEP]`` with segment ids 0 / 1, built from two single-text encodings (the
    second one loses its leading [CLS] when the tokenizer adds one); the document is cut to fit."""
    a = tokenizer.encode(query, add_special_tokens=True) or [0]
    b = tokenizer.encode(doc, add_special_tokens=True) or [0]
    if len(b) > 1 and b[0] == a[0]:
        b = b[1:]
    a = a[: max(1, max_len // 2)]
    room = max(1, max_len - len(a))
    if len(b) > room:
        b = b[: room - 1] + b[-1:]
    return a + b, [0] * len(a) + [1] * len(b)


def rerank_scores(encoder, tokenizer, query: str, docs: list[str]) -> list[float]:
    """Relevance of every document to the query: the cross-encoder head (sigmoid of logit 0 for a
    one-label head, probability of the last label otherwise) when the checkpoint has one, else the
    cosine between mean-pooled embeddings (reference src/main.rs:266 ``mlxcel rerank``, ``/v1/rerank``)."""
    if getattr(encoder, "classifier", (None,))[0] is not None and not getattr(encoder, "token_head", False):
        out = []
        for d in docs:
            ids, types = pair_ids(tokenizer, query, d, encoder.max_len)
            lg = encoder.sequence_logits(ids, types)
            out.append(float(torch.sigmoid(lg[0]) if lg.numel() == 1 else torch.softmax(lg, -1)[-1]))
        return out
    q = encoder.embed(tokenizer.encode(query, add_special_tokens=True) or [0])
    return [float(q @ encoder.embed(tokenizer.encode(d, add_special_tokens=True) or [0])) for d in docs]


def tag_text(encoder, tokenizer, text: str, keep: set[str] | None = None, replacement: str | None = None,
             argmax: bool = False) -> dict:
    """Token classification over one text: BIO spans with their decoded surface text and a redacted copy
    (every span not in ``keep`` replaced by ``replacement`` or ``[ENTITY]``). Reference src/main.rs:281
    (``mlxcel tag``)."""
    from ..models.encoder import bio_spans

    ids = (tokenizer.encode(text, add_special_tokens=True) or [0])[: encoder.max_len]
    lg = encoder.token_logits(ids)
    prob = torch.softmax(lg, -1)
    names = [encoder.id2label.get(i, "O") for i in range(lg.shape[1])]
    if argmax:
        path = lg.argmax(-1).tolist()
    else:                                            # best path that is a valid BIO / BIOES sequence
        from ..models.encoder import bio_viterbi
        path = bio_viterbi(torch.log_softmax(lg, -1), names)
    lab = [names[i] for i in path]
    spans, pieces, last = [], [], 0
    for s, e, ent in bio_spans(lab):
        surface = tokenizer.decode(ids[s:e], skip_special_tokens=True).strip()
        spans.append(dict(entity=ent, start_token=s, end_token=e, text=surface,
                          score=float(prob[s:e].max(-1).values.mean())))
        if keep and ent in keep:
            continue
        pieces.append(tokenizer.decode(ids[last:s], skip_special_tokens=True))
        pieces.append(" " + (replacement if replacement is not None else f"[{ent}]") + " ")
        last = e
    pieces.append(tokenizer.decode(ids[last:], skip_special_tokens=True))
    return dict(spans=spans, redacted=" ".join("".join(pieces).split()))


def create_embedding_app(encoder, tokenizer, model_id: str, api_keys: set | None = None):
    """Embeddings-only server for encoder checkpoints (BERT family): ``/v1/embeddings`` (OpenAI shape),
    ``/embedding`` (llama-server shape), ``/v1/rerank`` (cross-encoder head or cosine), ``/v1/tag`` (token
    classification), ``/v1/models``, ``/health``."""
    from fastapi import FastAPI, Request
    from fastapi.responses import JSONResponse

    app = FastAPI()
    keys = api_keys or set()

    @app.middleware("http")
    async def auth(request: Request, call_next):
        if keys and request.url.path not in ("/health",):
            tok = request.headers.get("authorization", "").removeprefix("Bearer ").strip()
            if tok not in keys:
                return JSONResponse({"error": {"message": "invalid API key", "type": "authentication_error"}}, 401)
        return await call_next(request)

    def run(texts, pooling):
        vecs, ntok = [], 0
        for t in texts:
            ids = tokenizer.encode(t, add_special_tokens=True) or [0]
            ntok += len(ids)
            vecs.append(encoder.embed(ids, pooling).cpu().tolist())
        return vecs, ntok

    @app.get("/health")
    async def health():
        return {"status": "ok"}

    @app.get("/v1/models")
    async def models():
        return {"object": "list", "data": [{"id": model_id, "object": "model", "owned_by": "mlxcel_b200"}]}

    @app.post("/v1/embeddings")
    @app.post("/embeddings")
    async def embeddings(body: dict):
        inp = body.get("input", body.get("content", ""))
        texts = [inp] if isinstance(inp, str) else list(inp)
        vecs, ntok = run(texts, body.get("pooling") or getattr(encoder, "default_pooling", "mean"))
        return {"object": "list", "model": model_id,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/v1/rerank")
    @app.post("/v1/reranking")
    @app.post("/rerank")
    async def rerank(body: dict):
        docs = [d if isinstance(d, str) else d.get("text", "") for d in body.get("documents", [])]
        scores = rerank_scores(encoder, tokenizer, body.get("query", ""), docs)
        order = sorted(range(len(docs)), key=lambda i: -scores[i])[: int(body.get("top_n") or len(docs))]
        return {"model": model_id, "results": [{"index": i, "relevance_score": scores[i]} for i in order]}

    @app.post("/v1/tag")
    async def tag(body: dict):
        if not getattr(encoder, "token_head", False):
            return JSONResponse({"error": {"message": "model has no token-classification head"}}, 400)
        return tag_text(encoder, tokenizer, body.get("text", body.get("input", "")), set(body.get("keep") or []),
                        body.get("replacement"), bool(body.get("argmax", False)))

    @app.post("/embedding")
    async def embedding(body: dict):
        inp = body.get("content", body.get("input", ""))
        texts = [inp] if isinstance(inp, str) else list(inp)
        vecs, _ = run(texts, body.get("pooling", "mean"))
        return [{"index": i, "embedding": v} for i, v in enumerate(vecs)]

    return app
