"""Checkpoint name aliases: families whose tensors are named (or laid out) differently from the
canonical ``model.layers.N.self_attn.q_proj`` scheme are presented to the loader under canonical
names, with the layout fixed on the way (reference src/models/sanitize.rs: weight-name remaps and
re-layouts at load time).

``aliases_for(cfg, keys)`` returns ``{canonical_name: (actual_name, transform | None)}``;
``TensorSource.set_aliases`` makes those names resolvable.
"""
from __future__ import annotations

import re

import torch


def _t(w: torch.Tensor) -> torch.Tensor:
    return w.t().contiguous()


def _neox_qkv(heads: int):
    """GPT-NeoX stores query_key_value per head as [heads, 3, D, ...]; the executor wants all q rows,
    then all k rows, then all v rows."""
    def fix(w: torch.Tensor) -> torch.Tensor:
        rest = w.shape[1:]
        d = w.shape[0] // (3 * heads)
        return w.view(heads, 3, d, *rest).transpose(0, 1).reshape(3 * heads * d, *rest).contiguous()
    return fix


def _grouped_qkv(heads: int, kv_heads: int):
    """InternLM2 stores wqkv per key/value group as [kv_heads, heads / kv_heads + 2, D, ...] (the group's
    query heads, then its key head, then its value head); the executor wants all q rows, k rows, v rows."""
    def fix(w: torch.Tensor) -> torch.Tensor:
        rest = w.shape[1:]
        g = heads // kv_heads
        d = w.shape[0] // (kv_heads * (g + 2))
        v = w.view(kv_heads, g + 2, d, *rest)
        q, k, vv = v[:, :g].reshape(heads * d, *rest), v[:, g].reshape(kv_heads * d, *rest), v[:, g + 1].reshape(kv_heads * d, *rest)
        return torch.cat([q, k, vv], 0).contiguous()
    return fix


def _rules(cfg) -> list[tuple[str, str, object]]:
    mt = cfg.model_type
    if mt == "internlm2":
        L = r"model\.layers\.(\d+)\."
        return [(r"model\.tok_embeddings\.(\w+)", r"model.embed_tokens.\1", None),
                (r"output\.(\w+)", r"lm_head.\1", None),
                (L + r"attention_norm\.(\w+)", r"model.layers.\1.input_layernorm.\2", None),
                (L + r"ffn_norm\.(\w+)", r"model.layers.\1.post_attention_layernorm.\2", None),
                (L + r"attention\.wqkv\.(\w+)", r"model.layers.\1.self_attn.qkv_proj.\2",
                 _grouped_qkv(cfg.num_attention_heads, cfg.num_key_value_heads)),
                (L + r"attention\.wo\.(\w+)", r"model.layers.\1.self_attn.o_proj.\2", None),
                (L + r"feed_forward\.w1\.(\w+)", r"model.layers.\1.mlp.gate_proj.\2", None),
                (L + r"feed_forward\.w3\.(\w+)", r"model.layers.\1.mlp.up_proj.\2", None),
                (L + r"feed_forward\.w2\.(\w+)", r"model.layers.\1.mlp.down_proj.\2", None)]
    if mt == "baichuan":                            # W_pack is already q rows | k rows | v rows
        return [(r"model\.layers\.(\d+)\.self_attn\.W_pack\.(\w+)", r"model.layers.\1.self_attn.qkv_proj.\2", None)]
    if mt == "gpt_neox":
        qkv = _neox_qkv(cfg.num_attention_heads)
        L = r"gpt_neox\.layers\.(\d+)\."
        return [(r"gpt_neox\.embed_in\.(\w+)", r"model.embed_tokens.\1", None),
                (r"gpt_neox\.final_layer_norm\.(\w+)", r"model.norm.\1", None),
                (r"embed_out\.(\w+)", r"lm_head.\1", None),
                (L + r"input_layernorm\.(\w+)", r"model.layers.\1.input_layernorm.\2", None),
                (L + r"post_attention_layernorm\.(\w+)", r"model.layers.\1.post_attention_layernorm.\2", None),
                (L + r"attention\.query_key_value\.(\w+)", r"model.layers.\1.self_attn.qkv_proj.\2", qkv),
                (L + r"attention\.dense\.(\w+)", r"model.layers.\1.self_attn.o_proj.\2", None),
                (L + r"mlp\.dense_h_to_4h\.(\w+)", r"model.layers.\1.mlp.fc1.\2", None),
                (L + r"mlp\.dense_4h_to_h\.(\w+)", r"model.layers.\1.mlp.fc2.\2", None)]
    if mt in ("gpt2", "gpt_bigcode"):
        tr = _t if mt == "gpt2" else None          # GPT-2 keeps Conv1D weights as [in, out]
        L = r"transformer\.h\.(\d+)\."
        return [(r"transformer\.wte\.(\w+)", r"model.embed_tokens.\1", None),
                (r"transformer\.wpe\.(\w+)", r"model.embed_positions.\1", None),
                (r"transformer\.ln_f\.(\w+)", r"model.norm.\1", None),
                (L + r"ln_1\.(\w+)", r"model.layers.\1.input_layernorm.\2", None),
                (L + r"ln_2\.(\w+)", r"model.layers.\1.post_attention_layernorm.\2", None),
                (L + r"attn\.c_attn\.weight", r"model.layers.\1.self_attn.qkv_proj.weight", tr),
                (L + r"attn\.c_attn\.bias", r"model.layers.\1.self_attn.qkv_proj.bias", None),
                (L + r"attn\.c_proj\.weight", r"model.layers.\1.self_attn.o_proj.weight", tr),
                (L + r"attn\.c_proj\.bias", r"model.layers.\1.self_attn.o_proj.bias", None),
                (L + r"mlp\.c_fc\.weight", r"model.layers.\1.mlp.fc1.weight", tr),
                (L + r"mlp\.c_fc\.bias", r"model.layers.\1.mlp.fc1.bias", None),
                (L + r"mlp\.c_proj\.weight", r"model.layers.\1.mlp.fc2.weight", tr),
                (L + r"mlp\.c_proj\.bias", r"model.layers.\1.mlp.fc2.bias", None)]
    if mt in ("llama4", "llama4_text"):
        # ``feed_forward`` is this family's name of the MLP / MoE block; the routed experts are stored
        # as [E, H, 2I] (gate columns, then up columns) and [E, I, H], i.e. transposed Linear weights
        half = lambda which: (lambda w: w[..., : w.shape[-1] // 2].transpose(1, 2).contiguous() if which == 0  # noqa: E731
                              else w[..., w.shape[-1] // 2:].transpose(1, 2).contiguous())
        P = r"(.*layers\.\d+\.)feed_forward\."
        return [(P + r"experts\.gate_up_proj", r"\1mlp.experts.gate_proj.weight", half(0)),
                (P + r"experts\.gate_up_proj", r"\1mlp.experts.up_proj.weight", half(1)),
                (P + r"experts\.down_proj", r"\1mlp.experts.down_proj.weight", lambda w: w.transpose(1, 2).contiguous()),
                (P + r"((?!experts\.).*)", r"\1mlp.\2", None)]
    if mt == "exaone":
        L = r"transformer\.h\.(\d+)\."
        M = r"model.layers.\1."
        return [(r"transformer\.wte\.(\w+)", r"model.embed_tokens.\1", None),
                (r"transformer\.ln_f\.(\w+)", r"model.norm.\1", None),
                (L + r"ln_1\.(\w+)", M + r"input_layernorm.\2", None),
                (L + r"ln_2\.(\w+)", M + r"post_attention_layernorm.\2", None),
                (L + r"attn\.attention\.(q_proj|k_proj|v_proj)\.(\w+)", M + r"self_attn.\2.\3", None),
                (L + r"attn\.attention\.out_proj\.(\w+)", M + r"self_attn.o_proj.\2", None),
                (L + r"mlp\.c_fc_0\.(\w+)", M + r"mlp.gate_proj.\2", None),
                (L + r"mlp\.c_fc_1\.(\w+)", M + r"mlp.up_proj.\2", None),
                (L + r"mlp\.c_proj\.(\w+)", M + r"mlp.down_proj.\2", None)]
    if mt == "dbrx":
        E = cfg.num_experts
        L = r"transformer\.blocks\.(\d+)\."
        M = r"model.layers.\1."
        stacked = lambda w: w.view(E, w.shape[0] // E, w.shape[1]).contiguous()                  # noqa: E731
        stacked_t = lambda w: w.view(E, w.shape[0] // E, w.shape[1]).transpose(1, 2).contiguous()  # noqa: E731
        return [(r"transformer\.wte\.(\w+)", r"model.embed_tokens.\1", None),
                (r"transformer\.norm_f\.(\w+)", r"model.norm.\1", None),
                (L + r"norm_attn_norm\.norm_1\.(\w+)", M + r"input_layernorm.\2", None),
                (L + r"norm_attn_norm\.norm_2\.(\w+)", M + r"post_attention_layernorm.\2", None),
                (L + r"norm_attn_norm\.attn\.Wqkv\.(\w+)", M + r"self_attn.qkv_proj.\2", None),
                (L + r"norm_attn_norm\.attn\.out_proj\.(\w+)", M + r"self_attn.o_proj.\2", None),
                (L + r"ffn\.router\.layer\.(\w+)", M + r"mlp.router.\2", None),
                # original checkpoints: w1 / v1 / w2 stacked as [E * I, H] (w2 is used transposed)
                (L + r"ffn\.experts\.mlp\.w1", M + r"mlp.experts.gate_proj.weight", stacked),
                (L + r"ffn\.experts\.mlp\.v1", M + r"mlp.experts.up_proj.weight", stacked),
                (L + r"ffn\.experts\.mlp\.w2", M + r"mlp.experts.down_proj.weight", stacked_t),
                # converted checkpoints: one Linear per expert and projection
                (L + r"ffn\.experts\.(\d+)\.w1\.(\w+)", M + r"mlp.experts.\2.gate_proj.\3", None),
                (L + r"ffn\.experts\.(\d+)\.v1\.(\w+)", M + r"mlp.experts.\2.up_proj.\3", None),
                (L + r"ffn\.experts\.(\d+)\.w2\.(\w+)", M + r"mlp.experts.\2.down_proj.\3", None)]
    return []


def aliases_for(cfg, keys) -> dict:
    rules = [(re.compile("^" + pat + "$"), rep, fn) for pat, rep, fn in _rules(cfg)]
    out = {}
    if not rules:
        return out
    for k in keys:
        for pat, rep, fn in rules:
            if pat.match(k):                     # (one tensor may be presented under several names)
                out.setdefault(pat.sub(rep, k), (k, fn))
    return out
