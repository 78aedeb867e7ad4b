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
def prefill_hidden(model, cfg, ids: list[int], block_size: int = 16) -> torch.Tensor:
    """Final hidden states [T, H] of one text from a single prefill over a private KV pool."""
    from ..cache.kv_pool import KVPool

    T = len(ids)
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
        return model.forward_hidden(b, pool.layers)
    finally:
        if getattr(model, "recurrent", False):
            model.release_seq(_SCRATCH_SEQ)


@torch.inference_mode()
def sequence_logprobs(model, cfg, ids: list[int], block_size: int = 16, row_chunk: int = 512) -> torch.Tensor:
    """``log p(ids[t] | ids[:t])`` for t = 1 .. T-1 as an fp32 CPU tensor [T-1]."""
    T = len(ids)
    if T < 2:
        return torch.zeros(0)
    dev = model.device
    h = prefill_hidden(model, cfg, ids, block_size)
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


RERANK_SYSTEM = ('Judge whether the Document meets the requirements based on the Query and the Instruct provided. '
                 'Note that the answer can only be "yes" or "no".')
RERANK_INSTRUCTION = "Given a web search query, retrieve relevant passages that answer the query"


def rerank_prompt(query: str, doc: str, instruction: str | None = None) -> str:
    """The yes/no judgement prompt of the generative (Qwen3-Reranker style) rerankers, ChatML framing with
    an empty thinking block (reference src/rerank/, generative path)."""
    return (f"<|im_start|>system\n{RERANK_SYSTEM}<|im_end|>\n<|im_start|>user\n<Instruct>: "
            f"{instruction or RERANK_INSTRUCTION}\n<Query>: {query}\n<Document>: {doc}<|im_end|>\n"
            f"<|im_start|>assistant\n<think>\n\n</think>\n\n")


@torch.inference_mode()
def generative_rerank(model, cfg, tokenizer, query: str, docs: list[str], instruction: str | None = None,
                      block_size: int = 16, max_len: int = 8192) -> list[float]:
    """``p(yes) / (p(yes) + p(no))`` of the next token after the judgement prompt, per document."""
    yes, no = tokenizer.encode("yes", add_special_tokens=False)[0], tokenizer.encode("no", add_special_tokens=False)[0]
    out = []
    for d in docs:
        ids = tokenizer.encode(rerank_prompt(query, d, instruction), add_special_tokens=False)
        if len(ids) > max_len:                       # keep the head (instruction, query) and the tail (answer slot)
            ids = ids[: max_len - 64] + ids[-64:]
        h = prefill_hidden(model, cfg, ids, block_size)
        lg = model.logits(h, torch.tensor([len(ids) - 1], device=model.device)).float()[0]
        out.append(float(torch.softmax(torch.stack([lg[no], lg[yes]]), 0)[1]))
    return out
