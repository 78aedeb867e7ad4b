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


def create_embedding_app(encoder, tokenizer, model_id: str, api_keys: set | None = None):
    """Embeddings-only server for encoder checkpoints (BERT family): ``/v1/embeddings`` (OpenAI shape),
    ``/embedding`` (llama-server shape), ``/v1/models``, ``/health``."""
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
        vecs, ntok = run(texts, body.get("pooling", "mean"))
        return {"object": "list", "model": model_id,
                "data": [{"object": "embedding", "index": i, "embedding": v} for i, v in enumerate(vecs)],
                "usage": {"prompt_tokens": ntok, "total_tokens": ntok}}

    @app.post("/embedding")
    async def embedding(body: dict):
        inp = body.get("content", body.get("input", ""))
        texts = [inp] if isinstance(inp, str) else list(inp)
        vecs, _ = run(texts, body.get("pooling", "mean"))
        return [{"index": i, "embedding": v} for i, v in enumerate(vecs)]

    return app
