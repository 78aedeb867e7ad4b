"""Scoring without generation: per-token log-likelihoods of a given text and windowed perplexity.

Reference: ``DirectEngine::loglikelihoods`` (src/lib/mlxcel-core/src/engine/direct.rs) and the
perplexity example (examples/perplexity.rs). One prefill forward over a private KV pool per window;
the logits are taken for every row, in slices, so that a long window never holds ``[T, vocab]`` fp32
at once. State-space and hybrid executors get a scratch state slot that is released afterwards.
"""
from __future__ import annotations

import math

import torch

from ..models.decoder import StepBatch

_SCRATCH_SEQ = -7


@torch.inference_mode()
def sequence_logprobs(model, cfg, ids: list[int], block_size: int = 16, row_chunk: int = 512) -> torch.Tensor:
    """``log p(ids[t] | ids[:t])`` for t = 1 .. T-1 as an fp32 CPU tensor [T-1]."""
    from ..cache.kv_pool import KVPool

    T = len(ids)
    if T < 2:
        return torch.zeros(0)
    dev = model.device
    nb = (T + block_size - 1) // block_size
    comm = getattr(model, "comm", None)
    layers = getattr(model, "num_kv_layers", None)
    if layers is None:
        layers = len(model.w.layers)
    pool = KVPool(cfg, max(nb, 1), block_size, device=dev, tp_size=comm.tp_size if comm is not None else 1,
                  num_layers=max(layers, 1), dtype=model.w.final_norm.dtype)
    i32 = dict(dtype=torch.int32, device=dev)
    b = StepBatch(token_ids=torch.tensor(ids, **i32), positions=torch.arange(T, **i32), slot_mapping=torch.arange(T, **i32),
                  num_prefill_seqs=1, pf_block_tables=torch.arange(nb, **i32)[None], pf_cu_q=torch.tensor([0, T], **i32),
                  pf_context_lens=torch.tensor([T], **i32), pf_max_q_len=T, pf_cu_q_host=[0, T])
    b.seq_ids, b.pf_starts = [_SCRATCH_SEQ], [0]
    try:
        h = model.forward_hidden(b, pool.layers)
    finally:
        if getattr(model, "recurrent", False):
            model.release_seq(_SCRATCH_SEQ)
    tgt = torch.tensor(ids[1:], dtype=torch.long, device=dev)
    out = []
    for r0 in range(0, T - 1, row_chunk):
        rows = torch.arange(r0, min(r0 + row_chunk, T - 1), device=dev)
        lp = torch.log_softmax(model.logits(h, rows).float(), dim=-1)
        out.append(lp.gather(1, tgt[rows, None])[:, 0].cpu())
    return torch.cat(out)


def perplexity(model, cfg, ids: list[int], window: int = 2048, stride: int | None = None, block_size: int = 16,
               progress=None) -> dict:
    """Strided-window perplexity: windows of ``window`` tokens advance by ``stride`` (default: half a
    window); each window scores only the tokens the previous one did not, so that every token but the
    first is scored once with at least ``window - stride`` tokens of context."""
    stride = stride or max(1, window // 2)
    T = len(ids)
    nll, count, start, scored_to = 0.0, 0, 0, 1
    while scored_to < T:
        end = min(start + window, T)
        lp = sequence_logprobs(model, cfg, ids[start:end], block_size)         # lp[i] scores token start + 1 + i
        first = scored_to - (start + 1)
        nll -= float(lp[first:].sum())
        count += lp.numel() - first
        scored_to = end
        if progress:
            progress(scored_to, T)
        if end == T:
            break
        start += stride
    return dict(tokens=count, nll=nll, perplexity=math.exp(nll / max(count, 1)), window=window, stride=stride)
