"""Sparse MoE block of the decoder executor.

Router GEMM → top-k routing → local gather of the routed rows → grouped gate/up GEMM with the
gated activation fused → grouped down GEMM → weighted combine (+ residual). Under expert
parallelism every rank holds E / ep experts; tokens are replicated (attention is tensor
parallel), so the only collective is the all-reduce of the partial outputs.
Reference: MLPBlock.forward (src/models/gpt_oss.rs:402-446), SwitchGLU
(src/models/switch_layers.rs:98-220), shared experts of Qwen2-MoE.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import moe as moe_ops
from .weights import LayerWeights, QuantizedTensor


def _dense(w):
    if isinstance(w, QuantizedTensor):
        from ..ops import quant
        return quant.dequantize(w)
    return w


def _shared_expert(cfg, lw: LayerWeights, x: torch.Tensor) -> torch.Tensor:
    si = lw.shared_gate_up.shape[0] // 2 if not isinstance(lw.shared_gate_up, QuantizedTensor) \
        else lw.shared_gate_up.shape[-2] // 2
    a = ops.glu_linear(x, _dense(lw.shared_gate_up), si, cfg.hidden_act)
    s = ops.linear(a, _dense(lw.shared_down))
    if lw.shared_gate is not None:
        g = torch.sigmoid(ops.linear(x, lw.shared_gate).float())
        s = (s.float() * g).to(s.dtype)
    return s


def moe_null(cfg, lw: LayerWeights, comm, dtype, device) -> None:
    """This rank's part of a MoE layer when it has no tokens this tick: it sends nothing, serves the
    rows the other ranks route to its experts, and reads nothing back."""
    k, H = cfg.num_experts_per_tok, cfg.hidden_size
    gu, dn = lw.experts_gate_up, lw.experts_down
    comm.a2a.moe(torch.empty(0, H, dtype=dtype, device=device), torch.empty(0, k, dtype=torch.int32, device=device),
                 torch.empty(0, k, dtype=torch.float32, device=device), gu, dn, gu.shape[-2] // 2, cfg.hidden_act,
                 lw.experts_gate_up_b, lw.experts_down_b, residual=None, alpha=cfg.swiglu_alpha, limit=cfg.swiglu_limit)


def moe_forward(cfg, lw: LayerWeights, x: torch.Tensor, h: torch.Tensor, comm) -> torch.Tensor:
    """Returns the new residual stream ``h + moe(x)`` (bf16 [T, H])."""
    if cfg.moe_route_mode == "sparsemixer":
        logits = ops.linear(x, lw.router_w, bias=lw.router_b)
        ids, wts = moe_ops.route_sparsemixer(logits, cfg.extra.get("router_jitter", 0.01))
    elif cfg.moe_route_mode == "sigmoid_group":
        r = cfg.extra["moe_routing"]
        logits = x.float() @ lw.router_w.float().t()            # the router runs in fp32
        ids, wts = moe_ops.route_sigmoid_grouped(logits, cfg.num_experts_per_tok, lw.router_b, r["n_group"],
                                                 r["topk_group"], cfg.norm_topk_prob, r["scale"], r.get("score", "sigmoid"),
                                                 r.get("norm_min", 1e-20), r.get("group_score", "top2sum"))
    elif cfg.moe_route_mode == "sigmoid_input":
        # Llama 4: top-1 expert; the sigmoid of its logit scales the expert's INPUT (so it passes
        # through the activation), the output is summed unweighted
        logits = ops.linear(x, lw.router_w, bias=lw.router_b)
        top, ids = logits.float().topk(1, dim=-1)
        x_shared, x = x, (x.float() * torch.sigmoid(top)).to(x.dtype)
        ids, wts = ids.to(torch.int32).contiguous(), torch.ones_like(top)
    else:
        logits = ops.linear(x, lw.router_w, bias=lw.router_b)
        ids, wts = moe_ops.route(logits, cfg.num_experts_per_tok, cfg.moe_route_mode, cfg.norm_topk_prob)
    if cfg.moe_route_mode != "sigmoid_input":
        x_shared = x
    a2a = getattr(comm, "a2a", None)
    if a2a is not None:
        # token-sharded ranks: rows travel to the experts' owners and come back (parallel/dp_ep.py)
        gu, dn = lw.experts_gate_up, lw.experts_down
        out = a2a.moe(x, ids.int().contiguous(), wts.float().contiguous(), gu, dn, gu.shape[-2] // 2, cfg.hidden_act,
                      lw.experts_gate_up_b, lw.experts_down_b, residual=h, alpha=cfg.swiglu_alpha, limit=cfg.swiglu_limit)
        if lw.shared_gate_up is not None:
            out = (out.float() + _shared_expert(cfg, lw, x_shared).float()).to(out.dtype)
        return out
    ep, ep_rank = comm.ep_size, comm.ep_rank
    # packed expert weights stay packed: the grouped GEMM unpacks the tiles of routed experts only
    gate_up, down = lw.experts_gate_up, lw.experts_down
    El = gate_up.shape[0]
    inter = gate_up.shape[-2] // 2
    first = ep_rank == 0 or ep == 1
    # with balanced routing 1 / ep of the (token, k) pairs land on this rank's experts: that estimate
    # picks the decode or the prefill expert kernels
    hint = max(1, x.shape[0] * ids.shape[1] // ep) if ep > 1 else None
    out = moe_ops.moe_experts(x, ids, wts, gate_up, down, inter, cfg.hidden_act, lw.experts_gate_up_b,
                              lw.experts_down_b, e_begin=ep_rank * El, residual=h if first else None,
                              alpha=cfg.swiglu_alpha, limit=cfg.swiglu_limit, rows_hint=hint)
    if lw.shared_gate_up is not None:
        out = (out.float() + _shared_expert(cfg, lw, x_shared).float()).to(out.dtype)
    if ep > 1:
        out = comm.all_reduce(out)
    return out
