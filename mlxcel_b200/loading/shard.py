"""Tensor / expert / pipeline sharding of a full set of decoder weights.

Shard plan (the reference's, src/distributed/tensor_parallel/plan_generator.rs:255-315 and
llama_runtime.rs:3179-3193): q/k/v and gate/up are column-parallel (split by heads / by FFN
columns), o_proj and down_proj are row-parallel (split along their input dimension), norms and
the embedding table are replicated, the LM head is vocab-parallel, MoE experts are distributed
round-robin-free in contiguous slices (rank r owns experts [r*E/ep, (r+1)*E/ep)).
KV heads must divide the tensor-parallel degree or be replicated (tp > Hkv).
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..models.weights import LayerWeights, ModelWeights, QuantizedTensor


def _rows(t, lo: int, hi: int):
    if t is None:
        return None
    if isinstance(t, QuantizedTensor):
        return QuantizedTensor(t.packed[..., lo:hi, :].contiguous(), t.scales[..., lo:hi, :].contiguous(),
                               None if t.biases is None else t.biases[..., lo:hi, :].contiguous(),
                               t.bits, t.group_size, t.mode)
    # stacked expert tensors [E, rows, cols]: rows are the middle axis
    return (t[lo:hi] if t.dim() < 3 else t[:, lo:hi]).contiguous()


def _cols(t, lo: int, hi: int):
    """Slice the input dimension [lo, hi) (must be group-aligned for quantized tensors)."""
    if t is None:
        return None
    if isinstance(t, QuantizedTensor):
        per_word = 32 // t.bits
        g = t.group_size
        if lo % g or hi % g or lo % per_word or hi % per_word:
            raise ValueError("quantized column shard must align to the quantization group")
        return QuantizedTensor(t.packed[..., lo // per_word:hi // per_word].contiguous(),
                               t.scales[..., lo // g:hi // g].contiguous(),
                               None if t.biases is None else t.biases[..., lo // g:hi // g].contiguous(),
                               t.bits, t.group_size, t.mode)
    return t[..., lo:hi].contiguous()


def _cat_rows(parts):
    parts = [p for p in parts if p is not None]
    if not parts:
        return None
    if isinstance(parts[0], QuantizedTensor):
        q = parts[0]
        return QuantizedTensor(torch.cat([p.packed for p in parts], dim=-2),
                               torch.cat([p.scales for p in parts], dim=-2),
                               None if q.biases is None else torch.cat([p.biases for p in parts], dim=-2),
                               q.bits, q.group_size, q.mode)
    return torch.cat(parts, dim=0)


def shard_layer(cfg: ModelConfig, lw: LayerWeights, rank: int, tp: int, ep_rank: int = 0,
                ep: int = 1) -> LayerWeights:
    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    if getattr(lw, "mla", None) is not None and tp > 1:
        raise NotImplementedError("tensor-parallel sharding of multi-head latent attention")
    if Hq % tp:
        raise ValueError("attention heads must divide the tensor-parallel degree")
    hq = Hq // tp
    q0 = rank * hq * D
    if Hkv >= tp:
        if Hkv % tp:
            raise ValueError("kv heads must divide the tensor-parallel degree")
        hkv = Hkv // tp
        kv0 = rank * hkv * D
    else:
        hkv = 1
        kv0 = (rank * Hkv // tp) * D   # replicated kv head serving this rank's q heads
    qs, ks, vs = Hq * D, Hkv * D, Hkv * D

    def qkv_rows(t):
        if t is None:
            return None
        if isinstance(t, torch.Tensor) and t.dim() == 1:
            return torch.cat([t[q0:q0 + hq * D], t[qs + kv0:qs + kv0 + hkv * D],
                              t[qs + ks + kv0:qs + ks + kv0 + hkv * D]]).contiguous()
        return _cat_rows([_rows(t, q0, q0 + hq * D), _rows(t, qs + kv0, qs + kv0 + hkv * D),
                          _rows(t, qs + ks + kv0, qs + ks + kv0 + hkv * D)])

    out = LayerWeights(ln1=lw.ln1, ln2=lw.ln2, wqkv=qkv_rows(lw.wqkv),
                       wo=_cols(lw.wo, q0, q0 + hq * D), bqkv=qkv_rows(lw.bqkv), bo=lw.bo,
                       q_norm=lw.q_norm, k_norm=lw.k_norm,
                       sinks=None if lw.sinks is None else lw.sinks[rank * hq:(rank + 1) * hq].contiguous(),
                       post_attn_norm=lw.post_attn_norm, post_mlp_norm=lw.post_mlp_norm)
    out.ln1_b, out.ln2_b = lw.ln1_b, lw.ln2_b
    if lw.w_gate_up is not None and cfg.extra.get("mlp") == "plain":
        i = cfg.intermediate_size // tp                 # non-gated MLP: rows of fc, columns of proj
        out.w_gate_up = _rows(lw.w_gate_up, rank * i, (rank + 1) * i)
        out.w_down = _cols(lw.w_down, rank * i, (rank + 1) * i)
        out.b_gate_up = None if lw.b_gate_up is None else lw.b_gate_up[rank * i:(rank + 1) * i].contiguous()
        out.b_down = lw.b_down
    elif lw.w_gate_up is not None:
        I = cfg.intermediate_size
        i = I // tp
        out.w_gate_up = _cat_rows([_rows(lw.w_gate_up, rank * i, (rank + 1) * i),
                                   _rows(lw.w_gate_up, I + rank * i, I + (rank + 1) * i)])
        out.w_down = _cols(lw.w_down, rank * i, (rank + 1) * i)
        if lw.b_gate_up is not None:
            out.b_gate_up = torch.cat([lw.b_gate_up[rank * i:(rank + 1) * i],
                                       lw.b_gate_up[I + rank * i:I + (rank + 1) * i]]).contiguous()
        out.b_down = lw.b_down
    if lw.router_w is not None:
        E = cfg.num_experts
        out.router_w, out.router_b = lw.router_w, lw.router_b
        e0, e1 = ep_rank * E // ep, (ep_rank + 1) * E // ep

        def experts(t):
            if t is None:
                return None
            if isinstance(t, QuantizedTensor):
                return QuantizedTensor(t.packed[e0:e1].contiguous(), t.scales[e0:e1].contiguous(),
                                       None if t.biases is None else t.biases[e0:e1].contiguous(),
                                       t.bits, t.group_size, t.mode)
            return t[e0:e1].contiguous()

        out.experts_gate_up, out.experts_down = experts(lw.experts_gate_up), experts(lw.experts_down)
        out.experts_gate_up_b, out.experts_down_b = experts(lw.experts_gate_up_b), experts(lw.experts_down_b)
        # the shared expert (when present) is tensor-parallel like a dense MLP
        if lw.shared_gate_up is not None:
            S = cfg.shared_expert_intermediate_size
            si = S // tp
            out.shared_gate_up = _cat_rows([_rows(lw.shared_gate_up, rank * si, (rank + 1) * si),
                                            _rows(lw.shared_gate_up, S + rank * si, S + (rank + 1) * si)])
            out.shared_down = _cols(lw.shared_down, rank * si, (rank + 1) * si)
            out.shared_gate = lw.shared_gate
    return out


def shard_weights(cfg: ModelConfig, full: ModelWeights, rank: int, tp: int, *, ep: int | None = None,
                  layers: range | None = None, vocab_parallel: bool = True, ep_rank: int | None = None) -> ModelWeights:
    """Slice a full (unsharded) model for tensor-parallel rank ``rank`` of ``tp`` (experts are
    expert-parallel over the same ranks unless ``ep`` says otherwise) and pipeline layers ``layers``."""
    ep = tp if ep is None else ep
    idx = layers if layers is not None else range(len(full.layers))
    # ``ep_rank`` given: expert sharding independent of the tensor-parallel rank (data-parallel attention)
    lws = [shard_layer(cfg, full.layers[i], rank, tp, rank % ep if ep_rank is None else ep_rank, ep) for i in idx]
    V = cfg.vocab_size
    lm_head = full.lm_head
    if vocab_parallel and tp > 1 and V % tp == 0:
        vl = V // tp
        lm_head = _rows(full.lm_head, rank * vl, (rank + 1) * vl)
    return ModelWeights(embed=full.embed, layers=lws, final_norm=full.final_norm, lm_head=lm_head,
                        extra=dict(full.extra))


def partition_layers(num_layers: int, stages: int, weights: list[float] | None = None) -> list[range]:
    """Contiguous pipeline partition balancing per-layer cost (auto partition of the reference,
    src/distributed/pipeline/partition.rs): equal cost unless ``weights`` is given."""
    w = weights or [1.0] * num_layers
    total = sum(w)
    out, start, acc = [], 0, 0.0
    for s in range(stages):
        target = total * (s + 1) / stages
        end = start
        while end < num_layers and (acc + w[end] <= target + 1e-9 or end == start):
            acc += w[end]
            end += 1
        remaining_stages = stages - s - 1
        end = min(end, num_layers - remaining_stages)
        out.append(range(start, end))
        start = end
    if start < num_layers:
        out[-1] = range(out[-1].start, num_layers)
    return out
