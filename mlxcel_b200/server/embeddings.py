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
        h = model.forward_hidden(b, pool.layers).float()
        v = h[-1] if pooling == "last" else h.mean(0)
        v = v / v.norm().clamp_min(1e-12)
        out.append(v.cpu().tolist())
    return out, ntok
