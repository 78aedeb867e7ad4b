"""Hybrid state-space / attention language models on the serving engine.

A model is a flat list of pre-norm residual blocks; the family decides the list (``block_kinds``):

=====  ===============================================================================================
``M``  Mamba2 mixer (``models/mamba2.py``)                       Nemotron-H, Granite-4 hybrid
``m``  first-generation Mamba mixer (``models/mamba1.py``)       Jamba
``L``  Gated DeltaNet mixer (``models/gdn.py``)                  Qwen3-Next
``P``  Mamba2 mixer and attention side by side                   Falcon-H1
``*``  grouped-query attention over the paged KV pool (NoPE or RoPE per family)
``A``  the same with per-head (1 + w) q/k norms and a sigmoid output gate    Qwen3-Next
``-``  plain MLP ``down(relu(up(x))^2)``                         Nemotron-H
``G``  gated (SwiGLU) MLP
``E``  mixture of experts (``models/moe.py``)                    Jamba, Qwen3-Next
=====  ===============================================================================================

Nemotron-H gives one block per layer through ``hybrid_override_pattern`` (``"M-M-M*-..."``); the other
families have a mixer block and an MLP / MoE block per layer. Reference: src/models/nemotron_h.rs,
granitemoehybrid.rs, jamba.rs, falcon_h1.rs, qwen3_next.rs.

Only the attention blocks own KV-pool layers (``num_kv_layers``); the engine sizes its pool from that.
The executor composes existing ones: a recurrent-mixer model (Mamba2 / Mamba / Gated DeltaNet) for the
per-sequence state slots and its mixer, a :class:`DecoderModel` for the attention path. Single GPU.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import recurrent as rops
from .decoder import DecoderModel, LocalComm, StepBatch
from .mamba2 import Mamba2LayerWeights, Mamba2Model, Mamba2Weights, mamba_dims
from .weights import LayerWeights, ModelWeights


@dataclass
class HybridBlock:
    kind: str                                   # "mamba2" | "mamba1" | "attention" | "mlp" | "moe"
    norm: torch.Tensor
    mamba: object | None = None                 # Mamba2LayerWeights or Mamba1LayerWeights
    moe: LayerWeights | None = None             # router + stacked experts (block kind "moe")
    attn: LayerWeights | None = None            # wqkv / wo (+ biases)
    up: torch.Tensor | None = None              # plain MLP [I, H]; gated MLP: [2I, H] (gate rows first)
    down: torch.Tensor | None = None            # [H, I]
    gated: bool = False
    act: str = "silu"                           # activation of a gated MLP block
    up_b: torch.Tensor | None = None            # MLP biases (RecurrentGemma)
    down_b: torch.Tensor | None = None
    out_gate: torch.Tensor | None = None        # gated attention (Qwen3-Next): [Hq * D, H] sigmoid gate projection
    latent_in: torch.Tensor | None = None       # Nemotron-H MoE: optional projections around the routed experts
    latent_out: torch.Tensor | None = None      #   ([latent, H] and [H, latent]); up / down hold the shared expert


@dataclass
class HybridWeights:
    embed: torch.Tensor
    blocks: list
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    layers: list = field(default_factory=list)  # the attention blocks' LayerWeights (= KV-pool layers)


_KINDS = {"M": "mamba2", "m": "mamba1", "L": "gdn", "C": "shortconv", "R": "rglru", "P": "parallel", "*": "attention", "A": "attention", "-": "mlp", "G": "mlp",
          "E": "moe"}   # G: gated MLP, A: attention with an output gate, L: Gated DeltaNet


def block_kinds(cfg: ModelConfig) -> list[str]:
    pat = cfg.extra["hybrid_pattern"]
    per_layer = 2 if cfg.extra.get("hybrid_layout") in ("granite", "jamba", "qwen3_next", "falcon_h1", "lfm2",
                                                             "recurrent_gemma") else 1
    if len(pat) != cfg.num_hidden_layers * per_layer:
        raise ValueError(f"hybrid pattern has {len(pat)} entries for {cfg.num_hidden_layers} layers")
    try:
        return [_KINDS[c] for c in pat]
    except KeyError as e:
        raise ValueError(f"unknown block kind {e.args[0]!r} in hybrid pattern {pat!r}") from None


def random_hybrid_weights(cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16, device="cpu", std: float = 0.02):
    from .mamba2 import random_mamba2_weights

    g = torch.Generator().manual_seed(seed + 1)
    r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype).to(device)  # noqa: E731
    H, I = cfg.hidden_size, cfg.intermediate_size
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    kinds = block_kinds(cfg)
    mw = random_mamba2_weights(cfg, seed=seed, dtype=dtype, device=device, std=std)   # one per layer; mamba ones are used
    one = lambda: torch.ones(H, dtype=dtype, device=device)  # noqa: E731
    blocks, attn_layers = [], []
    for i, k in enumerate(kinds):
        if k == "mamba2":
            blocks.append(HybridBlock(k, one(), mamba=mw.layers[i]))
        elif k == "attention":
            lw = LayerWeights(ln1=one(), ln2=one(), wqkv=r((Hq + 2 * Hkv) * D, H), wo=r(H, Hq * D))
            attn_layers.append(lw)
            blocks.append(HybridBlock(k, lw.ln1, attn=lw))
        else:
            blocks.append(HybridBlock(k, one(), up=r(I, H), down=r(H, I)))
    return HybridWeights(embed=mw.embed, blocks=blocks, final_norm=mw.final_norm, lm_head=mw.lm_head,
                         layers=attn_layers)


def load_hybrid_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """Nemotron-H checkpoint names: ``backbone.layers.N.norm.weight`` and ``backbone.layers.N.mixer.*``
    with ``in_proj / conv1d / A_log / D / dt_bias / norm / out_proj`` (Mamba2), ``q_proj / k_proj /
    v_proj / o_proj`` (attention) or ``up_proj / down_proj`` (+ ``gate_proj``) (MLP). Quantized
    projections are dequantised at load."""
    from ..loading.checkpoint import TensorSource, _Getter

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = mamba_dims(cfg)
    pre = "backbone." if any(k.startswith("backbone.") for k in src.keys()) else "model."

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    blocks, attn_layers = [], []
    for i, kind in enumerate(block_kinds(cfg)):
        p = f"{pre}layers.{i}."
        m = p + "mixer."
        norm = need(g.vec(p + "norm.weight"), p + "norm.weight")
        if kind == "mamba2":
            cw = need(g.vec(m + "conv1d.weight"), m + "conv1d.weight")
            cw = cw.reshape(d["conv_dim"], d["K"]) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
            cb = g.vec(m + "conv1d.bias")
            lw = Mamba2LayerWeights(
                norm=norm, in_proj=need(g.mat(m + "in_proj"), m + "in_proj"), conv_w=cw.float(),
                conv_b=None if cb is None else cb.float().to(device),
                dt_bias=need(g.vec(m + "dt_bias"), m + "dt_bias").float(),
                A_log=need(g.vec(m + "A_log"), m + "A_log").float(), D=need(g.vec(m + "D"), m + "D").float(),
                gnorm=need(g.vec(m + "norm.weight"), m + "norm.weight"),
                out_proj=need(g.mat(m + "out_proj"), m + "out_proj"))
            blocks.append(HybridBlock(kind, norm, mamba=lw))
        elif kind == "attention":
            q, k, v = (need(g.mat(m + n), m + n) for n in ("q_proj", "k_proj", "v_proj"))
            bq, bk, bv = (g.vec(m + n + ".bias") for n in ("q_proj", "k_proj", "v_proj"))
            bo = g.vec(m + "o_proj.bias")
            lw = LayerWeights(ln1=norm, ln2=norm, wqkv=torch.cat([q, k, v], 0).contiguous(),
                              wo=need(g.mat(m + "o_proj"), m + "o_proj"),
                              bqkv=None if bq is None else torch.cat([bq, bk, bv]).to(device),
                              bo=None if bo is None else bo.to(device))
            attn_layers.append(lw)
            blocks.append(HybridBlock(kind, norm, attn=lw))
        elif kind == "moe":
            # plain (non-gated) experts stored stacked [E, I, in] / [E, in, I], fp32 router with a
            # selection bias, one always-on shared expert, optional latent projections
            E = cfg.num_experts
            if src.has(m + "experts.up_proj"):
                ups, downs = src.get(m + "experts.up_proj"), src.get(m + "experts.down_proj")
            else:
                ups = torch.stack([g.mat(f"{m}experts.{e}.up_proj") for e in range(E)])
                downs = torch.stack([g.mat(f"{m}experts.{e}.down_proj") for e in range(E)])
            bias = g.vec(m + "gate.e_score_correction_bias")
            moe = LayerWeights(ln1=norm, ln2=norm, wqkv=None, wo=None, router_w=need(g.mat(m + "gate"), m + "gate"),
                               router_b=None if bias is None else bias.float().to(device),
                               experts_gate_up=ups.to(dtype).to(device).contiguous(),
                               experts_down=downs.to(dtype).to(device).contiguous())
            opt = lambda n: None if g.mat(n) is None else g.mat(n).to(device)  # noqa: E731
            blocks.append(HybridBlock("moe_plain", norm, moe=moe,
                                      up=need(g.mat(m + "shared_experts.up_proj"), m + "shared_experts.up_proj"),
                                      down=need(g.mat(m + "shared_experts.down_proj"), m + "shared_experts.down_proj"),
                                      latent_in=opt(m + "fc1_latent_proj"), latent_out=opt(m + "fc2_latent_proj")))
        else:
            up = need(g.mat(m + "up_proj"), m + "up_proj")
            gate = g.mat(m + "gate_proj")
            blocks.append(HybridBlock(kind, norm, up=up if gate is None else torch.cat([gate.to(device), up], 0).contiguous(),
                                      down=need(g.mat(m + "down_proj"), m + "down_proj"), gated=gate is not None))
    ename = next((pre + n for n in ("embeddings", "embedding", "embed_tokens") if src.has(pre + n + ".weight")),
                 pre + "embeddings")
    embed = need(g.mat(ename), ename)
    head = g.mat("lm_head") if src.has("lm_head.weight") else None
    return HybridWeights(embed=embed, blocks=blocks,
                         final_norm=need(g.vec(pre + "norm_f.weight"), pre + "norm_f.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def load_granite_hybrid_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """Granite 4 hybrid checkpoint: ``model.layers.N.{input_layernorm, mamba.* | self_attn.*,
    post_attention_layernorm, shared_mlp.input_linear / output_linear [, block_sparse_moe.{router.layer,
    input_linear, output_linear}]}``; each layer becomes a mixer block and a gated-MLP block, or a MoE
    block (routed experts plus the shared MLP) when the checkpoint has routed experts."""
    from ..loading.checkpoint import TensorSource, _Getter

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = mamba_dims(cfg)

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    blocks, attn_layers = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = need(g.vec(p + "input_layernorm.weight"), p + "input_layernorm.weight")
        if src.has(p + "mamba.in_proj.weight"):
            m = p + "mamba."
            cw = need(g.vec(m + "conv1d.weight"), m + "conv1d.weight")
            cw = cw.reshape(d["conv_dim"], d["K"]) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
            cb = g.vec(m + "conv1d.bias")
            lw = Mamba2LayerWeights(
                norm=norm, in_proj=need(g.mat(m + "in_proj"), m + "in_proj"), conv_w=cw.float(),
                conv_b=None if cb is None else cb.float().to(device),
                dt_bias=need(g.vec(m + "dt_bias"), m + "dt_bias").float(),
                A_log=need(g.vec(m + "A_log"), m + "A_log").float(), D=need(g.vec(m + "D"), m + "D").float(),
                gnorm=need(g.vec(m + "norm.weight"), m + "norm.weight"),
                out_proj=need(g.mat(m + "out_proj"), m + "out_proj"))
            blocks.append(HybridBlock("mamba2", norm, mamba=lw))
        else:
            a = p + "self_attn."
            q, k, v = (need(g.mat(a + n), a + n) for n in ("q_proj", "k_proj", "v_proj"))
            lw = LayerWeights(ln1=norm, ln2=norm, wqkv=torch.cat([q, k, v], 0).contiguous(),
                              wo=need(g.mat(a + "o_proj"), a + "o_proj"))
            attn_layers.append(lw)
            blocks.append(HybridBlock("attention", norm, attn=lw))
        s = p + "shared_mlp."
        fn = need(g.vec(p + "post_attention_layernorm.weight"), p + "post_attention_layernorm")
        up, down = need(g.mat(s + "input_linear"), s + "input_linear"), need(g.mat(s + "output_linear"), s + "output_linear")
        e = p + "block_sparse_moe."
        if cfg.num_experts and src.has(e + "input_linear.weight"):
            # routed experts stored fused ([E, 2I, H] gate rows first, [E, H, I]) beside the shared MLP
            moe = LayerWeights(ln1=fn, ln2=fn, wqkv=None, wo=None,
                               router_w=need(g.mat(e + "router.layer"), e + "router.layer"),
                               experts_gate_up=src.get(e + "input_linear.weight").to(dtype).to(device).contiguous(),
                               experts_down=src.get(e + "output_linear.weight").to(dtype).to(device).contiguous(),
                               shared_gate_up=up, shared_down=down)
            blocks.append(HybridBlock("moe", fn, moe=moe))
        else:
            blocks.append(HybridBlock("mlp", fn, up=up, down=down, gated=True))
    embed = need(g.mat("model.embed_tokens"), "model.embed_tokens")
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return HybridWeights(embed=embed, blocks=blocks, final_norm=need(g.vec("model.norm.weight"), "model.norm.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def load_jamba_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """Jamba checkpoint: ``model.layers.N.{input_layernorm, mamba.* | self_attn.*, pre_ff_layernorm,
    feed_forward.(gate|up|down)_proj | feed_forward.router + experts.E.*}``; each layer becomes a mixer
    block (first-generation Mamba with norms on dt / B / C, or attention without positional encoding)
    and an MLP or MoE block (reference src/models/jamba.rs)."""
    from ..loading.checkpoint import TensorSource, _Getter, _cat_rows, _stack
    from .mamba1 import Mamba1LayerWeights, mamba1_dims

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = mamba1_dims(cfg)

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    blocks, attn_layers = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = need(g.vec(p + "input_layernorm.weight"), p + "input_layernorm.weight")
        if src.has(p + "mamba.in_proj.weight"):
            m = p + "mamba."
            cw = need(g.vec(m + "conv1d.weight"), m + "conv1d.weight")
            cw = cw.reshape(d["Di"], d["K"]) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
            cb = g.vec(m + "conv1d.bias")
            opt = lambda n: None if g.vec(n) is None else g.vec(n).to(device)  # noqa: E731
            lw = Mamba1LayerWeights(
                norm=norm, in_proj=need(g.mat(m + "in_proj"), m + "in_proj"), in_proj_b=opt(m + "in_proj.bias"),
                conv_w=cw.float(), conv_b=None if cb is None else cb.float().to(device),
                x_proj=need(g.mat(m + "x_proj"), m + "x_proj"), dt_proj=need(g.mat(m + "dt_proj"), m + "dt_proj"),
                dt_proj_b=need(g.vec(m + "dt_proj.bias"), m + "dt_proj.bias"),
                A_log=need(g.vec(m + "A_log"), m + "A_log").float(), D=need(g.vec(m + "D"), m + "D").float(),
                out_proj=need(g.mat(m + "out_proj"), m + "out_proj"), out_proj_b=opt(m + "out_proj.bias"),
                dt_norm=opt(m + "dt_layernorm.weight"), b_norm=opt(m + "b_layernorm.weight"),
                c_norm=opt(m + "c_layernorm.weight"))
            blocks.append(HybridBlock("mamba1", norm, mamba=lw))
        else:
            a = p + "self_attn."
            q, k, v = (need(g.mat(a + n), a + n) for n in ("q_proj", "k_proj", "v_proj"))
            lw = LayerWeights(ln1=norm, ln2=norm, wqkv=torch.cat([q, k, v], 0).contiguous(),
                              wo=need(g.mat(a + "o_proj"), a + "o_proj"))
            attn_layers.append(lw)
            blocks.append(HybridBlock("attention", norm, attn=lw))
        f = p + "feed_forward."
        fn = need(g.vec(p + "pre_ff_layernorm.weight"), p + "pre_ff_layernorm.weight")
        if src.has(f + "router.weight"):
            gus = [_cat_rows([g.mat(f"{f}experts.{e}.gate_proj"), g.mat(f"{f}experts.{e}.up_proj")])
                   for e in range(cfg.num_experts)]
            downs = [g.mat(f"{f}experts.{e}.down_proj") for e in range(cfg.num_experts)]
            moe = LayerWeights(ln1=fn, ln2=fn, wqkv=None, wo=None, router_w=need(g.mat(f + "router"), f + "router"),
                               experts_gate_up=_stack(gus).to(device), experts_down=_stack(downs).to(device))
            blocks.append(HybridBlock("moe", fn, moe=moe))
        else:
            blocks.append(HybridBlock("mlp", fn, up=_cat_rows([need(g.mat(f + "gate_proj"), f + "gate_proj"),
                                                               need(g.mat(f + "up_proj"), f + "up_proj")]),
                                      down=need(g.mat(f + "down_proj"), f + "down_proj"), gated=True))
    embed = need(g.mat("model.embed_tokens"), "model.embed_tokens")
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return HybridWeights(embed=embed, blocks=blocks,
                         final_norm=need(g.vec("model.final_layernorm.weight"), "model.final_layernorm.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def load_lfm2_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """LFM2 checkpoint: ``model.layers.N.{operator_norm, conv.(in_proj, conv, out_proj) | self_attn.(q_proj,
    k_proj, v_proj, out_proj, q_layernorm, k_layernorm), ffn_norm, feed_forward.(w1, w3, w2)}`` and
    ``model.embedding_norm`` as the final norm; each layer becomes a mixer block (gated short conv or
    attention with per-head q/k RMSNorm) and a gated-MLP block (reference src/models/lfm2.rs)."""
    from ..loading.checkpoint import TensorSource, _cat_rows, _Getter
    from .shortconv import ShortConvLayerWeights

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    K, H = int(cfg.extra["shortconv"]["d_conv"]), cfg.hidden_size

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    opt = lambda n: None if g.vec(n) is None else g.vec(n).to(device)  # noqa: E731
    blocks, attn_layers = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = need(g.vec(p + "operator_norm.weight"), p + "operator_norm.weight")
        if src.has(p + "conv.in_proj.weight"):
            c = p + "conv."
            cw = need(g.vec(c + "conv.weight"), c + "conv.weight")
            cw = cw.reshape(H, K) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
            cb = opt(c + "conv.bias")
            lw = ShortConvLayerWeights(norm=norm, in_proj=need(g.mat(c + "in_proj"), c + "in_proj"), conv_w=cw.float(),
                                       out_proj=need(g.mat(c + "out_proj"), c + "out_proj"), in_proj_b=opt(c + "in_proj.bias"),
                                       conv_b=None if cb is None else cb.float(), out_proj_b=opt(c + "out_proj.bias"))
            blocks.append(HybridBlock("shortconv", norm, mamba=lw))
        else:
            a = p + "self_attn."
            q, k, v = (need(g.mat(a + n), a + n) for n in ("q_proj", "k_proj", "v_proj"))
            lw = LayerWeights(ln1=norm, ln2=norm, wqkv=torch.cat([q, k, v], 0).contiguous(),
                              wo=need(g.mat(a + "out_proj"), a + "out_proj"),
                              q_norm=need(g.vec(a + "q_layernorm.weight"), a + "q_layernorm"),
                              k_norm=need(g.vec(a + "k_layernorm.weight"), a + "k_layernorm"))
            attn_layers.append(lw)
            blocks.append(HybridBlock("attention", norm, attn=lw))
        f = p + "feed_forward."
        fn = need(g.vec(p + "ffn_norm.weight"), p + "ffn_norm.weight")
        if src.has(f + "gate.weight"):              # LFM2-MoE: routed experts w1 (gate) / w3 (up) / w2 (down)
            from ..loading.checkpoint import _stack
            gus = [_cat_rows([g.mat(f"{f}experts.{e}.w1"), g.mat(f"{f}experts.{e}.w3")]) for e in range(cfg.num_experts)]
            downs = [g.mat(f"{f}experts.{e}.w2") for e in range(cfg.num_experts)]
            moe = LayerWeights(ln1=fn, ln2=fn, wqkv=None, wo=None, router_w=need(g.mat(f + "gate"), f + "gate"),
                               experts_gate_up=_stack(gus).to(device), experts_down=_stack(downs).to(device))
            if src.has(f + "expert_bias"):
                moe.router_b = src.get(f + "expert_bias").float().reshape(-1).to(device)
            blocks.append(HybridBlock("moe", fn, moe=moe))
            continue
        blocks.append(HybridBlock("mlp", fn,
                                  up=_cat_rows([need(g.mat(f + "w1"), f + "w1"), need(g.mat(f + "w3"), f + "w3")]),
                                  down=need(g.mat(f + "w2"), f + "w2"), gated=True))
    embed = need(g.mat("model.embed_tokens"), "model.embed_tokens")
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return HybridWeights(embed=embed, blocks=blocks,
                         final_norm=need(g.vec("model.embedding_norm.weight"), "model.embedding_norm.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def load_qwen3_next_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """Qwen3-Next checkpoint: ``model.layers.N.{input_layernorm, linear_attn.* | self_attn.*,
    post_attention_layernorm, mlp.(gate + experts.E.* + shared_expert.* + shared_expert_gate | gate_proj ...)}``.
    Layer norms, the final norm and the per-head q/k norms are stored as (weight - 1): one is added
    here. ``q_proj`` carries query and output gate interleaved per head; they are separated."""
    from ..loading.checkpoint import TensorSource, _Getter, _cat_rows, _stack
    from .gdn import GdnLayerWeights, gdn_dims, regroup_ba, regroup_qkvz

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = gdn_dims(cfg)
    Hq, D = cfg.num_attention_heads, cfg.head_dim

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    def plus1(name):
        return (need(g.vec(name), name).float() + 1.0).to(dtype)

    # Qwen3.5 checkpoints keep the language model under ``model.language_model`` and store the
    # linear-attention input projection as four matrices already ordered q | k | v, z, b, a
    root = "model.language_model." if src.has("model.language_model.embed_tokens.weight") else "model."
    blocks, attn_layers = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"{root}layers.{i}."
        norm = plus1(p + "input_layernorm.weight")
        if src.has(p + "linear_attn.out_proj.weight"):
            m = p + "linear_attn."
            cw = need(g.vec(m + "conv1d.weight"), m + "conv1d.weight")
            cw = cw.reshape(d["conv_dim"], d["K"]) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
            if src.has(m + "in_proj_qkvz.weight"):
                in_proj = regroup_qkvz(need(g.mat(m + "in_proj_qkvz"), m + "in_proj_qkvz"), d)
                in_ba = regroup_ba(need(g.mat(m + "in_proj_ba"), m + "in_proj_ba"), d)
            else:
                in_proj = torch.cat([need(g.mat(m + n), m + n) for n in ("in_proj_qkv", "in_proj_z")], 0).contiguous()
                in_ba = torch.cat([need(g.mat(m + n), m + n) for n in ("in_proj_b", "in_proj_a")], 0).contiguous()
            lw = GdnLayerWeights(
                norm=norm, in_proj=in_proj, in_proj_ba=in_ba, conv_w=cw.float(),
                dt_bias=need(g.vec(m + "dt_bias"), m + "dt_bias").float(),
                A_log=need(g.vec(m + "A_log"), m + "A_log").float(),
                gnorm=need(g.vec(m + "norm.weight"), m + "norm.weight"),
                out_proj=need(g.mat(m + "out_proj"), m + "out_proj"))
            blocks.append(HybridBlock("gdn", norm, mamba=lw))
        else:
            a = p + "self_attn."
            qg = need(g.mat(a + "q_proj"), a + "q_proj").view(Hq, 2, D, -1)          # per head: query rows, gate rows
            q, gate = qg[:, 0].reshape(Hq * D, -1), qg[:, 1].reshape(Hq * D, -1).contiguous()
            k, v = need(g.mat(a + "k_proj"), a + "k_proj"), need(g.mat(a + "v_proj"), a + "v_proj")
            lw = LayerWeights(ln1=norm, ln2=norm, wqkv=torch.cat([q, k, v], 0).contiguous(),
                              wo=need(g.mat(a + "o_proj"), a + "o_proj"), q_norm=plus1(a + "q_norm.weight"),
                              k_norm=plus1(a + "k_norm.weight"))
            attn_layers.append(lw)
            blocks.append(HybridBlock("attention", norm, attn=lw, out_gate=gate))
        f = p + "mlp."
        fn = plus1(p + "post_attention_layernorm.weight")
        if src.has(f + "gate.weight"):
            gus = [_cat_rows([g.mat(f"{f}experts.{e}.gate_proj"), g.mat(f"{f}experts.{e}.up_proj")])
                   for e in range(cfg.num_experts)]
            downs = [g.mat(f"{f}experts.{e}.down_proj") for e in range(cfg.num_experts)]
            moe = LayerWeights(ln1=fn, ln2=fn, wqkv=None, wo=None, router_w=need(g.mat(f + "gate"), f + "gate"),
                               experts_gate_up=_stack(gus).to(device), experts_down=_stack(downs).to(device))
            if src.has(f + "shared_expert.gate_proj.weight"):
                moe.shared_gate_up = _cat_rows([g.mat(f + "shared_expert.gate_proj"), g.mat(f + "shared_expert.up_proj")]).to(device)
                moe.shared_down = need(g.mat(f + "shared_expert.down_proj"), f + "shared_expert.down_proj")
                moe.shared_gate = need(g.mat(f + "shared_expert_gate"), f + "shared_expert_gate")
            blocks.append(HybridBlock("moe", fn, moe=moe))
        else:
            blocks.append(HybridBlock("mlp", fn, up=_cat_rows([need(g.mat(f + "gate_proj"), f + "gate_proj"),
                                                               need(g.mat(f + "up_proj"), f + "up_proj")]),
                                      down=need(g.mat(f + "down_proj"), f + "down_proj"), gated=True))
    embed = need(g.mat(root + "embed_tokens"), root + "embed_tokens")
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return HybridWeights(embed=embed, blocks=blocks, final_norm=plus1(root + "norm.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def load_recurrent_gemma_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """RecurrentGemma checkpoint: ``model.layers.N.{temporal_pre_norm, temporal_block.*, channel_pre_norm,
    mlp_block.*}``. Norms are stored as (weight - 1); the RG-LRU gate blocks are stored as
    [heads, in, out] and are transposed to Linear orientation here."""
    from ..loading.checkpoint import TensorSource, _Getter, _cat_rows
    from .rglru import RglruLayerWeights

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    W, K = int(cfg.extra["rglru"]["width"]), int(cfg.extra["rglru"]["d_conv"])

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    def vec(name):
        return need(g.vec(name), name)

    def plus1(name):
        return (vec(name).float() + 1.0).to(dtype)

    blocks, attn_layers = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        t = p + "temporal_block."
        norm = plus1(p + "temporal_pre_norm.weight")
        if src.has(t + "rg_lru.recurrent_param"):
            cw = vec(t + "conv_1d.weight")
            lw = RglruLayerWeights(
                norm=norm, linear_y=need(g.mat(t + "linear_y"), t + "linear_y"), linear_y_b=vec(t + "linear_y.bias"),
                linear_x=need(g.mat(t + "linear_x"), t + "linear_x"), linear_x_b=vec(t + "linear_x.bias"),
                conv_w=cw.reshape(W, K).float(), conv_b=vec(t + "conv_1d.bias").float(),
                gate_in_w=vec(t + "rg_lru.input_gate_weight").transpose(1, 2).contiguous(),
                gate_in_b=vec(t + "rg_lru.input_gate_bias").reshape(-1),
                gate_rec_w=vec(t + "rg_lru.recurrent_gate_weight").transpose(1, 2).contiguous(),
                gate_rec_b=vec(t + "rg_lru.recurrent_gate_bias").reshape(-1),
                decay=vec(t + "rg_lru.recurrent_param").float(),
                out_proj=need(g.mat(t + "linear_out"), t + "linear_out"), out_proj_b=vec(t + "linear_out.bias"))
            blocks.append(HybridBlock("rglru", norm, mamba=lw))
        else:
            bs = [g.vec(t + f"{n}_proj.bias") for n in "qkv"]
            lw = LayerWeights(ln1=norm, ln2=norm,
                              wqkv=_cat_rows([need(g.mat(t + f"{n}_proj"), t + f"{n}_proj") for n in "qkv"]),
                              bqkv=torch.cat(bs).to(device) if all(b is not None for b in bs) else None,
                              wo=need(g.mat(t + "o_proj"), t + "o_proj"), bo=g.vec(t + "o_proj.bias"))
            if lw.bo is not None:
                lw.bo = lw.bo.to(device)
            attn_layers.append(lw)
            blocks.append(HybridBlock("attention", norm, attn=lw))
        m = p + "mlp_block."
        bg, bu = g.vec(m + "gate_proj.bias"), g.vec(m + "up_proj.bias")
        blocks.append(HybridBlock("mlp", plus1(p + "channel_pre_norm.weight"),
                                  up=_cat_rows([need(g.mat(m + "gate_proj"), m + "gate_proj"),
                                                need(g.mat(m + "up_proj"), m + "up_proj")]),
                                  down=need(g.mat(m + "down_proj"), m + "down_proj"), gated=True, act="gelu_tanh",
                                  up_b=torch.cat([bg, bu]).to(device) if bg is not None and bu is not None else None,
                                  down_b=None if g.vec(m + "down_proj.bias") is None else g.vec(m + "down_proj.bias").to(device)))
    for blk in blocks:                      # every tensor a kernel will read lives on the executor's device
        for obj in (blk, blk.mamba, blk.attn):
            if obj is not None:
                for k, v in list(vars(obj).items()):
                    if isinstance(v, torch.Tensor) and v.device != torch.device(device):
                        setattr(obj, k, v.to(device))
    embed = need(g.mat("model.embed_tokens"), "model.embed_tokens")
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return HybridWeights(embed=embed, blocks=blocks, final_norm=plus1("model.final_norm.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def load_falcon_h1_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> HybridWeights:
    """Falcon-H1 checkpoint: ``model.layers.N.{input_layernorm, mamba.*, self_attn.*, pre_ff_layernorm,
    feed_forward.*}``. Every muP multiplier of the config is a constant factor on one projection's
    input or output, so it is multiplied into that projection's weight here and the executor runs
    plain blocks."""
    from ..loading.checkpoint import TensorSource, _Getter, _cat_rows

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = mamba_dims(cfg)
    mup = cfg.extra["falcon_mup"]
    di, gn = d["d_inner"], d["G"] * d["N"]
    seg = torch.cat([torch.full((n,), v) for n, v in zip((di, di, gn, gn, d["heads"]), mup["ssm"])]) * mup["ssm_in"]

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    def scaled(name, factor):
        w = need(g.mat(name), name)
        return w if factor == 1.0 else (w.float() * factor).to(w.dtype)

    blocks, attn_layers = [], []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        norm = need(g.vec(p + "input_layernorm.weight"), p + "input_layernorm.weight")
        m = p + "mamba."
        cw = need(g.vec(m + "conv1d.weight"), m + "conv1d.weight")
        cw = cw.reshape(d["conv_dim"], d["K"]) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
        cb = g.vec(m + "conv1d.bias")
        w_in = need(g.mat(m + "in_proj"), m + "in_proj")
        gn_w = g.vec(m + "norm.weight")
        mw = Mamba2LayerWeights(
            norm=norm, in_proj=(w_in.float() * seg.to(w_in.device).unsqueeze(1)).to(w_in.dtype), conv_w=cw.float(),
            conv_b=None if cb is None else cb.float().to(device),
            dt_bias=need(g.vec(m + "dt_bias"), m + "dt_bias").float(), A_log=need(g.vec(m + "A_log"), m + "A_log").float(),
            D=need(g.vec(m + "D"), m + "D").float(),
            gnorm=torch.ones(di, dtype=dtype, device=device) if gn_w is None else gn_w.to(device),
            out_proj=scaled(m + "out_proj", mup["ssm_out"]))
        a = p + "self_attn."
        q, k, v = (scaled(a + "q_proj", mup["attn_in"]), scaled(a + "k_proj", mup["attn_in"] * mup["key"]),
                   scaled(a + "v_proj", mup["attn_in"]))
        aw = LayerWeights(ln1=norm, ln2=norm, wqkv=torch.cat([q, k, v], 0).contiguous(),
                          wo=scaled(a + "o_proj", mup["attn_out"]))
        attn_layers.append(aw)
        blocks.append(HybridBlock("parallel", norm, mamba=mw, attn=aw))
        f = p + "feed_forward."
        blocks.append(HybridBlock("mlp", need(g.vec(p + "pre_ff_layernorm.weight"), p + "pre_ff_layernorm.weight"),
                                  up=_cat_rows([scaled(f + "gate_proj", mup["gate"]), need(g.mat(f + "up_proj"), f + "up_proj")]),
                                  down=scaled(f + "down_proj", mup["down"]), gated=True))
    embed = need(g.mat("model.embed_tokens"), "model.embed_tokens")
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return HybridWeights(embed=embed, blocks=blocks,
                         final_norm=need(g.vec("model.final_layernorm.weight"), "model.final_layernorm.weight"),
                         lm_head=embed if head is None else head.to(device), layers=attn_layers)


def hybrid_config_dict(cfg: ModelConfig) -> dict:
    d = mamba_dims(cfg)
    return dict(model_type="nemotron_h", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                num_hidden_layers=cfg.num_hidden_layers, hybrid_override_pattern=cfg.extra["hybrid_pattern"],
                mamba_num_heads=d["heads"], mamba_head_dim=d["P"], ssm_state_size=d["N"], conv_kernel=d["K"],
                n_groups=d["G"], intermediate_size=cfg.intermediate_size,
                num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim, layer_norm_epsilon=cfg.rms_norm_eps,
                tie_word_embeddings=cfg.tie_word_embeddings)


def save_hybrid_checkpoint(path, cfg_dict: dict, w: HybridWeights, cfg: ModelConfig) -> None:
    import json
    from pathlib import Path

    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    t = {"backbone.embeddings.weight": w.embed, "backbone.norm_f.weight": w.final_norm}
    if w.lm_head is not w.embed:
        t["lm_head.weight"] = w.lm_head
    for i, blk in enumerate(w.blocks):
        p = f"backbone.layers.{i}."
        m = p + "mixer."
        t[p + "norm.weight"] = blk.norm
        if blk.kind == "mamba2":
            lw = blk.mamba
            t.update({m + "in_proj.weight": lw.in_proj, m + "conv1d.weight": lw.conv_w.unsqueeze(1),
                      m + "dt_bias": lw.dt_bias, m + "A_log": lw.A_log, m + "D": lw.D, m + "norm.weight": lw.gnorm,
                      m + "out_proj.weight": lw.out_proj})
            if lw.conv_b is not None:
                t[m + "conv1d.bias"] = lw.conv_b
        elif blk.kind == "attention":
            q, k, v = blk.attn.wqkv.split([Hq * D, Hkv * D, Hkv * D], 0)
            t.update({m + "q_proj.weight": q, m + "k_proj.weight": k, m + "v_proj.weight": v,
                      m + "o_proj.weight": blk.attn.wo})
        else:
            if blk.gated:
                gate, up = blk.up.chunk(2, 0)
                t[m + "gate_proj.weight"] = gate
            else:
                up = blk.up
            t.update({m + "up_proj.weight": up, m + "down_proj.weight": blk.down})
    save_file({k: v.detach().cpu().contiguous() for k, v in t.items()}, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(cfg_dict))


class HybridModel:
    """Engine-facing executor (``forward`` / ``forward_hidden`` / ``logits`` / ``release_seq``)."""

    recurrent = True

    def __init__(self, cfg: ModelConfig, weights: HybridWeights, max_seqs: int = 256, comm=None, kv_bits: int = 16):
        self.cfg, self.w = cfg, weights
        self.comm = comm or LocalComm()
        assert self.comm.tp_size == 1, "the hybrid executor is single-GPU"
        self.device = weights.final_norm.device
        mamba_layers = [b.mamba for b in weights.blocks if b.kind in ("mamba2", "parallel")]
        mamba1_layers = [b.mamba for b in weights.blocks if b.kind == "mamba1"]
        gdn_layers = [b.mamba for b in weights.blocks if b.kind == "gdn"]
        conv_layers = [b.mamba for b in weights.blocks if b.kind == "shortconv"]
        rglru_layers = [b.mamba for b in weights.blocks if b.kind == "rglru"]
        if rglru_layers:                        # RecurrentGemma: RG-LRU recurrent blocks
            from .rglru import RglruModel
            self.ssm = RglruModel(cfg, Mamba2Weights(weights.embed, rglru_layers, weights.final_norm, weights.lm_head),
                                  max_seqs=max_seqs, comm=self.comm)
        elif conv_layers:                         # LFM2: gated short convolutions
            from .shortconv import ShortConvModel
            self.ssm = ShortConvModel(cfg, Mamba2Weights(weights.embed, conv_layers, weights.final_norm, weights.lm_head),
                                      max_seqs=max_seqs, comm=self.comm)
        elif gdn_layers:                          # Qwen3-Next: Gated DeltaNet mixers
            from .gdn import GdnModel
            self.ssm = GdnModel(cfg, Mamba2Weights(weights.embed, gdn_layers, weights.final_norm, weights.lm_head),
                                max_seqs=max_seqs, comm=self.comm)
        elif mamba1_layers:                     # Jamba: first-generation mixers
            from .mamba1 import Mamba1Model
            self.ssm = Mamba1Model(cfg, Mamba2Weights(weights.embed, mamba1_layers, weights.final_norm, weights.lm_head),
                                   max_seqs=max_seqs, comm=self.comm)
        else:
            self.ssm = Mamba2Model(cfg, Mamba2Weights(weights.embed, mamba_layers, weights.final_norm, weights.lm_head),
                                   max_seqs=max_seqs, comm=self.comm)
        self.attn = DecoderModel(cfg, ModelWeights(weights.embed, weights.layers, weights.final_norm, weights.lm_head),
                                 comm=self.comm, kv_bits=kv_bits)
        self.Hq, self.Hkv, self.D = self.attn.Hq, self.attn.Hkv, self.attn.D
        self.num_kv_layers = len(weights.layers)
        self.layer_range = range(cfg.num_hidden_layers)
        self.I = cfg.intermediate_size

    def release_seq(self, seq_id: int) -> None:
        self.ssm.release_seq(seq_id)

    @torch.inference_mode()
    def forward_hidden(self, b: StepBatch, kv_layers=None, hidden_in: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.cfg
        eps = cfg.rms_norm_eps
        pieces = self.ssm.pieces(b)
        h = hidden_in if hidden_in is not None else ops.embedding(b.token_ids, self.w.embed, cfg.embed_scale)
        mi = ai = 0
        rm = float(cfg.extra.get("residual_multiplier", 1.0))     # Granite: every branch is scaled

        def add(branch_in, w, bias=None):
            if rm == 1.0:
                return ops.linear(branch_in, w, bias=bias, residual=h)
            return (h.float() + ops.linear(branch_in, w, bias=bias).float() * rm).to(h.dtype)

        for blk in self.w.blocks:
            x = ops.rmsnorm(h, blk.norm, eps, 0.0)
            if blk.kind in ("mamba2", "mamba1", "gdn", "shortconv", "rglru"):
                h = add(self.ssm._mixer(mi, blk.mamba, x, pieces), blk.mamba.out_proj,
                        getattr(blk.mamba, "out_proj_b", None))
                mi += 1
            elif blk.kind == "parallel":         # Falcon-H1: Mamba2 mixer and attention side by side
                ym = ops.linear(self.ssm._mixer(mi, blk.mamba, x, pieces), blk.mamba.out_proj)
                ya = ops.linear(self.attn._attention(ai, blk.attn, x, b, kv_layers[ai]), blk.attn.wo, bias=blk.attn.bo)
                h = (h.float() + ym.float() + ya.float()).to(h.dtype)
                mi += 1
                ai += 1
            elif blk.kind == "moe":
                from .moe import moe_forward
                if rm == 1.0:
                    h = moe_forward(cfg, blk.moe, x, h, self.comm)
                else:                            # Granite: (experts + shared MLP) scaled into the stream
                    y = moe_forward(cfg, blk.moe, x, torch.zeros_like(h), self.comm)
                    h = (h.float() + y.float() * rm).to(h.dtype)
            elif blk.kind == "moe_plain":        # Nemotron-H: plain relu^2 experts + shared expert
                from ..ops import moe as moe_ops
                r, lw = cfg.extra["moe_routing"], blk.moe
                ids, wts = moe_ops.route_sigmoid_grouped(x.float() @ lw.router_w.float().t(), cfg.num_experts_per_tok,
                                                         lw.router_b, r["n_group"], r["topk_group"], cfg.norm_topk_prob,
                                                         r["scale"])
                xin = x if blk.latent_in is None else ops.linear(x, blk.latent_in)
                y = moe_ops.moe_experts(xin, ids, wts.to(torch.float32), lw.experts_gate_up, lw.experts_down,
                                        lw.experts_gate_up.shape[1], "relu2", gated=False)
                if blk.latent_out is not None:
                    y = ops.linear(y, blk.latent_out)
                sh = ops.linear(rops.relu2(ops.linear(x, blk.up)), blk.down)
                h = (h.float() + y.float() + sh.float()).to(h.dtype)
            elif blk.kind == "attention":
                a = self.attn._attention(ai, blk.attn, x, b, kv_layers[ai])
                if blk.out_gate is not None:     # Qwen3-Next: sigmoid gate computed from the block input
                    a = (a.float() * torch.sigmoid(ops.linear(x, blk.out_gate).float())).to(a.dtype)
                h = add(a, blk.attn.wo, blk.attn.bo)
                ai += 1
            elif blk.gated:
                h = add(ops.glu_linear(x, blk.up, blk.up.shape[0] // 2, blk.act, bias=blk.up_b), blk.down, blk.down_b)
            else:
                h = add(rops.relu2(ops.linear(x, blk.up)), blk.down)
        return h

    def logits(self, h: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        lg = self.ssm.logits(h, rows)
        ls = self.cfg.extra.get("logits_scaling", 1.0)
        lg = lg if ls == 1.0 else (lg.float() / ls).to(lg.dtype)
        cap = self.cfg.final_logit_softcap
        return lg if cap <= 0 else (torch.tanh(lg.float() / cap) * cap).to(lg.dtype)

    def forward(self, b: StepBatch, kv_layers=None) -> torch.Tensor:
        return self.logits(self.forward_hidden(b, kv_layers), b.logits_rows)
