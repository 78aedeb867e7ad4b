"""Model configuration: ``config.json`` → one normalised :class:`ModelConfig`.

The reference detects ~190 model types and gives each its own struct
(src/models/detection.rs:787,1236; src/models/registry.rs:1064). Here one record describes the
decoder-only transformer design space (attention variant, norm variant, MLP variant, MoE, RoPE
scaling, sliding windows, sinks, quantization) and model families are entries of
:data:`FAMILIES` that set flags on it.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any


@dataclass
class QuantConfig:
    """Checkpoint weight quantization (MLX formats, src/lib/mlxcel-core/src/layers.rs:1885-1933)."""

    mode: str = "none"  # none | affine | mxfp4 | mxfp8 | nvfp4
    bits: int = 16
    group_size: int = 64
    # per-module overrides: module path -> {"bits":..,"group_size":..,"mode":..} or False (unquantized)
    overrides: dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_dict(d: dict | None) -> "QuantConfig":
        if not d:
            return QuantConfig()
        mode = d.get("mode")
        bits = int(d.get("bits", 4))
        group = int(d.get("group_size", 64))
        if mode is None:
            mode = "affine"
        overrides = {k: v for k, v in d.items()
                     if isinstance(v, (dict, bool)) and k not in ("mode", "bits", "group_size")}
        return QuantConfig(mode=mode, bits=bits, group_size=group, overrides=overrides)

    def for_module(self, path: str) -> "QuantConfig | None":
        """Effective quantization of one module (``None`` = stored unquantized)."""
        ov = self.overrides.get(path)
        if ov is False:
            return None
        if isinstance(ov, dict):
            return QuantConfig(mode=ov.get("mode", self.mode), bits=int(ov.get("bits", self.bits)),
                               group_size=int(ov.get("group_size", self.group_size)))
        if self.mode == "none":
            return None
        return self


@dataclass
class ModelConfig:
    model_type: str = "llama"
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    rms_norm_eps: float = 1e-5
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    # rope
    rope_theta: float = 10000.0
    rope_scaling: dict | None = None
    rope_traditional: bool = False
    partial_rotary_factor: float = 1.0
    # attention variants
    attention_bias: bool = False
    mlp_bias: bool = False
    qk_norm: bool = False               # per-head RMSNorm on q and k (Qwen3, OLMo2-style)
    sliding_window: int = 0
    layer_types: list[str] | None = None  # per layer: "full_attention" | "sliding_attention"
    attention_sinks: bool = False       # gpt-oss per-head sink logits
    attn_logit_softcap: float = 0.0
    final_logit_softcap: float = 0.0
    query_pre_attn_scalar: float | None = None
    # norms / residual layout
    norm_weight_bias: float = 0.0       # 1.0 for Gemma's (1 + w)
    post_norms: bool = False            # Gemma2/3: post-attention and post-ffn norms
    embed_scale: float = 1.0
    # mlp
    hidden_act: str = "silu"            # silu | gelu_tanh | clipped_swiglu
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    # MoE
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    moe_route_mode: str = "topk_softmax"  # topk_softmax (mixtral, gpt-oss) | softmax_topk (qwen-moe)
    norm_topk_prob: bool = True
    shared_expert_intermediate_size: int = 0
    expert_bias: bool = False
    router_bias: bool = False
    # MTP / drafter
    num_nextn_predict_layers: int = 0
    # misc
    bos_token_id: int | None = None
    eos_token_id: Any = None
    quantization: QuantConfig = field(default_factory=QuantConfig)
    dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def rot_dim(self) -> int:
        r = int(self.head_dim * self.partial_rotary_factor)
        return r - (r % 2)

    @property
    def attn_scale(self) -> float:
        if self.query_pre_attn_scalar:
            return 1.0 / math.sqrt(self.query_pre_attn_scalar)
        return 1.0 / math.sqrt(self.head_dim)

    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_window(self, layer: int) -> int:
        """Sliding-window size of a layer (0 = full attention)."""
        if self.layer_types:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else 0
        return self.sliding_window

    def eos_ids(self) -> list[int]:
        e = self.eos_token_id
        if e is None:
            return []
        return [int(x) for x in e] if isinstance(e, (list, tuple)) else [int(e)]

    def kv_bytes_per_token(self, kv_bits: int = 16) -> int:
        per = self.num_key_value_heads * self.head_dim
        if kv_bits == 16:
            b = per * 2
        else:
            b = per * kv_bits // 8 + (per // 64) * 4
        return 2 * b * self.num_hidden_layers

    def param_count(self) -> int:
        h, i, L = self.hidden_size, self.intermediate_size, self.num_hidden_layers
        attn = h * (self.q_size + 2 * self.kv_size) + self.q_size * h
        if self.is_moe:
            mi = self.moe_intermediate_size or i
            mlp = self.num_experts * 3 * h * mi + h * self.num_experts
            if self.shared_expert_intermediate_size:
                mlp += 3 * h * self.shared_expert_intermediate_size
        else:
            mlp = 3 * h * i
        emb = self.vocab_size * h * (1 if self.tie_word_embeddings else 2)
        return L * (attn + mlp + 2 * h) + emb + h

    def to_dict(self) -> dict:
        d = asdict(self)
        return d

    # ------------------------------------------------------------------ construction
    @staticmethod
    def from_dict(raw: dict) -> "ModelConfig":
        raw = dict(raw)
        if "text_config" in raw and isinstance(raw["text_config"], dict):
            # VLM wrappers keep the language model under text_config
            inner = dict(raw["text_config"])
            for k in ("quantization", "quantization_config"):
                if k in raw and k not in inner:
                    inner[k] = raw[k]
            inner.setdefault("model_type", raw.get("model_type", "llama"))
            if "tie_word_embeddings" in raw:
                # the wrapper owns the LM head: its flag says whether the head is the embedding table
                inner["tie_word_embeddings"] = raw["tie_word_embeddings"]
            raw = inner
        mt = raw.get("model_type", "llama")
        fam = FAMILIES.get(mt)
        if fam is None:
            raise ValueError(f"unsupported model_type {mt!r}; supported: {sorted(FAMILIES)}")
        c = ModelConfig(model_type=mt)
        g = raw.get
        c.vocab_size = int(g("vocab_size", c.vocab_size))
        c.hidden_size = int(g("hidden_size", g("n_embd", c.hidden_size)))
        c.num_hidden_layers = int(g("num_hidden_layers", g("n_layer", c.num_hidden_layers)))
        c.num_attention_heads = int(g("num_attention_heads", g("n_head", c.num_attention_heads)))
        c.num_key_value_heads = int(g("num_key_value_heads", c.num_attention_heads))
        c.head_dim = int(g("head_dim") or c.hidden_size // c.num_attention_heads)
        c.intermediate_size = int(g("intermediate_size", g("ffn_dim", 4 * c.hidden_size)))
        c.rms_norm_eps = float(g("rms_norm_eps", g("layer_norm_epsilon", 1e-5)))
        c.max_position_embeddings = int(g("max_position_embeddings", 8192))
        c.tie_word_embeddings = bool(g("tie_word_embeddings", False))
        c.rope_theta = float(g("rope_theta", 10000.0))
        c.rope_scaling = g("rope_scaling")
        rp = g("rope_parameters")
        if isinstance(rp, dict):
            # transformers >= 5 layout: theta and scaling in one record, or one record per layer type
            if "full_attention" in rp or "sliding_attention" in rp:
                loc = rp.get("sliding_attention") or {}
                if loc.get("rope_theta") is not None:
                    c.extra["rope_local_theta"] = float(loc["rope_theta"])
                rp = rp.get("full_attention") or {}
            if rp.get("rope_theta") is not None:
                c.rope_theta = float(rp["rope_theta"])
            if rp.get("rope_type", rp.get("type", "default")) not in (None, "default"):
                c.rope_scaling = rp
            if rp.get("partial_rotary_factor") is not None and "partial_rotary_factor" not in raw:
                raw["partial_rotary_factor"] = rp["partial_rotary_factor"]
        if g("rope_local_base_freq") is not None:
            c.extra["rope_local_theta"] = float(g("rope_local_base_freq"))
        c.rope_traditional = bool(g("rope_traditional", False))
        c.partial_rotary_factor = float(g("partial_rotary_factor", 1.0))
        c.attention_bias = bool(g("attention_bias", g("qkv_bias", False)))
        c.mlp_bias = bool(g("mlp_bias", False))
        c.sliding_window = int(g("sliding_window") or 0)
        c.layer_types = g("layer_types")
        c.hidden_act = {"silu": "silu", "swish": "silu", "gelu_pytorch_tanh": "gelu_tanh",
                        "gelu_tanh": "gelu_tanh", "gelu": "gelu_tanh"}.get(
                            g("hidden_act", g("hidden_activation", "silu")), "silu")
        c.extra["act_raw"] = str(g("hidden_act", g("hidden_activation", g("activation_function", "silu"))))
        c.num_experts = int(g("num_local_experts", g("num_experts", g("n_routed_experts", 0))) or 0)
        c.num_experts_per_tok = int(g("num_experts_per_tok", g("experts_per_token", 0)) or 0)
        c.moe_intermediate_size = int(g("moe_intermediate_size", 0) or 0)
        c.norm_topk_prob = bool(g("norm_topk_prob", True))
        c.shared_expert_intermediate_size = int(g("shared_expert_intermediate_size", 0) or 0)
        c.num_nextn_predict_layers = int(g("num_nextn_predict_layers", g("mtp_num_hidden_layers", 0)) or 0)
        c.bos_token_id = g("bos_token_id")
        c.eos_token_id = g("eos_token_id")
        c.attn_logit_softcap = float(g("attn_logit_softcapping") or 0.0)
        c.final_logit_softcap = float(g("final_logit_softcapping") or 0.0)
        c.query_pre_attn_scalar = g("query_pre_attn_scalar")
        qc = g("quantization") or g("quantization_config")
        if isinstance(g("quantization_config"), dict) and g("quantization_config").get("quant_method"):
            qc = g("quantization_config")
        if isinstance(qc, dict) and qc.get("quant_method") in ("fp8", "compressed-tensors", "fbgemm_fp8", "modelopt"):
            # FP8 checkpoints: stored as float8 + scales, widened to bf16 at load (no packed groups)
            if qc.get("weight_block_size"):
                c.extra["fp8_block_size"] = tuple(int(x) for x in qc["weight_block_size"])
            qc = None
        c.quantization = QuantConfig.from_dict(qc)
        c.dtype = str(g("torch_dtype", g("dtype", "bfloat16")))
        rs = c.rope_scaling
        if rs and rs.get("rope_type", rs.get("type")) == "dynamic" and not rs.get("original_max_position_embeddings"):
            c.rope_scaling = dict(rs, original_max_position_embeddings=int(g("max_position_embeddings", 0) or 0))
        fam(c, raw)
        if c.is_moe and not c.moe_intermediate_size:
            c.moe_intermediate_size = c.intermediate_size
        if c.layer_types is not None and len(c.layer_types) != c.num_hidden_layers:
            raise ValueError("layer_types length does not match num_hidden_layers")
        if c.num_attention_heads % c.num_key_value_heads:
            raise ValueError("num_attention_heads must be a multiple of num_key_value_heads")
        return c

    @staticmethod
    def from_path(path: str | Path, overrides: dict | None = None) -> "ModelConfig":
        """``overrides``: keys replaced in ``config.json`` before it is interpreted (the ``--rope-*`` and
        ``--override-kv`` options; reference src/cli/rope.rs). RoPE keys also replace their copies inside
        ``rope_parameters`` when the checkpoint uses that spelling."""
        p = Path(path)
        if p.is_dir():
            p = p / "config.json"
        raw = json.loads(p.read_text())
        if overrides:
            raw = apply_config_overrides(raw, overrides)
        return ModelConfig.from_dict(raw)


def apply_config_overrides(raw: dict, overrides: dict) -> dict:
    raw = json.loads(json.dumps(raw))
    tgt = raw.get("text_config") if isinstance(raw.get("text_config"), dict) else raw
    for k, v in overrides.items():
        tgt[k] = v
        rp = tgt.get("rope_parameters")
        if isinstance(rp, dict) and k in ("rope_theta", "rope_scaling"):
            flat = all(not isinstance(x, dict) for x in rp.values())
            for d in ([rp] if flat else [x for x in rp.values() if isinstance(x, dict)]):
                if k == "rope_theta":
                    d["rope_theta"] = v
                elif v is None:
                    for kk in [kk for kk in d if kk not in ("rope_theta", "partial_rotary_factor")]:
                        d.pop(kk)
                    d["rope_type"] = "default"
                else:
                    d.update(v)
    return raw


# ----------------------------------------------------------------------------- families
def _plain(c: ModelConfig, raw: dict) -> None:
    pass


def _qwen2(c: ModelConfig, raw: dict) -> None:
    c.attention_bias = True
    if not raw.get("use_sliding_window", False):
        c.sliding_window = 0


def _qwen2_vl(c: ModelConfig, raw: dict) -> None:
    """Language model of Qwen2-VL / Qwen2.5-VL: Qwen2 blocks with multimodal rotary positions (each
    rotary frequency belongs to the temporal, height or width section)."""
    _qwen2(c, raw)
    for rec in (raw.get("rope_parameters"), raw.get("rope_scaling")):
        if isinstance(rec, dict) and rec.get("mrope_section"):
            c.extra["mrope_section"] = [int(x) for x in rec["mrope_section"]]
    rs = c.rope_scaling
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) in ("mrope", "default", None):
        c.rope_scaling = None                 # "mrope" names the position layout, not a frequency scaling


def _qwen3_vl(c: ModelConfig, raw: dict) -> None:
    """Language model of Qwen3-VL: Qwen3 blocks (per-head q/k norm) with interleaved multimodal rotary
    positions; visual features of intermediate tower depths are added to the first layers' outputs
    (DeepStack, carried with the media rows)."""
    _qwen3(c, raw)
    for rec in (raw.get("rope_parameters"), raw.get("rope_scaling")):
        if isinstance(rec, dict) and rec.get("mrope_section"):
            c.extra["mrope_section"] = [int(x) for x in rec["mrope_section"]]
            c.extra["mrope_interleaved"] = bool(rec.get("mrope_interleaved", True))
    rs = c.rope_scaling
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) in ("mrope", "default", None):
        c.rope_scaling = None


def _qwen3_vl_moe(c: ModelConfig, raw: dict) -> None:
    """Language model of Qwen3-VL-MoE: the Qwen3-MoE blocks under Qwen3-VL's positions and DeepStack."""
    _qwen3_vl(c, raw)
    c.moe_route_mode = "softmax_topk"
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", True))


def _qwen3(c: ModelConfig, raw: dict) -> None:
    c.qk_norm = True
    c.sliding_window = 0 if not raw.get("use_sliding_window", False) else c.sliding_window


def _qwen_moe(c: ModelConfig, raw: dict) -> None:
    if c.model_type.startswith("qwen3"):
        _qwen3(c, raw)
    else:
        _qwen2(c, raw)
    c.moe_route_mode = "softmax_topk"
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", False))


def _mixtral(c: ModelConfig, raw: dict) -> None:
    c.moe_route_mode = "topk_softmax"
    c.moe_intermediate_size = c.intermediate_size


def _gemma(c: ModelConfig, raw: dict) -> None:
    c.norm_weight_bias = 1.0
    c.embed_scale = math.sqrt(c.hidden_size)
    c.hidden_act = "gelu_tanh"
    c.tie_word_embeddings = True


def _gemma2(c: ModelConfig, raw: dict) -> None:
    _gemma(c, raw)
    c.post_norms = True
    n = c.num_hidden_layers
    if c.layer_types is None and c.sliding_window:
        c.layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n)]


def _gemma3(c: ModelConfig, raw: dict) -> None:
    _gemma(c, raw)
    c.post_norms = True
    c.qk_norm = True
    n = c.num_hidden_layers
    pat = int(raw.get("sliding_window_pattern", 6) or 6)
    if c.layer_types is None and c.sliding_window:
        c.layer_types = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention" for i in range(n)]


def _gpt_oss(c: ModelConfig, raw: dict) -> None:
    c.attention_sinks = True
    c.attention_bias = True
    c.hidden_act = "clipped_swiglu"
    c.swiglu_limit = float(raw.get("swiglu_limit", 7.0))
    c.moe_route_mode = "topk_softmax"
    c.expert_bias = True
    c.router_bias = True
    c.moe_intermediate_size = c.intermediate_size
    if c.layer_types is None and c.sliding_window:
        c.layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention"
                         for i in range(c.num_hidden_layers)]


def _phi3(c: ModelConfig, raw: dict) -> None:
    # fused qkv_proj / gate_up_proj names are handled by the weight-name sanitizer; the long-context
    # variants keep the lengths that longrope needs beside (not inside) the scaling block
    rs = c.rope_scaling
    if rs and rs.get("rope_type", rs.get("type")) in ("longrope", "su"):
        rs = dict(rs)
        rs.setdefault("original_max_position_embeddings", raw.get("original_max_position_embeddings"))
        rs.setdefault("max_position_embeddings", raw.get("max_position_embeddings"))
        c.rope_scaling = rs


def _olmo2(c: ModelConfig, raw: dict) -> None:
    c.qk_norm = True
    c.extra["qk_norm_full"] = True   # norm over the whole projection, not per head
    c.extra["post_norm_only"] = True  # norms after attention / mlp instead of before


def _plain_act(c: ModelConfig) -> str:
    """Activation of a non-gated MLP from the checkpoint's spelling."""
    a = c.extra.get("act_raw", "gelu")
    return {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh",
            "relu2": "relu2", "silu": "silu", "swish": "silu"}.get(a, "gelu")


def _starcoder2(c: ModelConfig, raw: dict) -> None:
    """LayerNorm with bias, biased projections, plain MLP c_fc -> GELU(tanh) -> c_proj
    (reference src/models/starcoder2.rs)."""
    c.extra["norm"] = "layernorm"
    c.extra["mlp"] = "plain"
    c.rms_norm_eps = float(raw.get("norm_epsilon", 1e-5))
    c.attention_bias = c.mlp_bias = bool(raw.get("use_bias", True))
    c.hidden_act = _plain_act(c)
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))
    c.layer_types = None                         # one window for every layer (sliding_window, may be null)


def _stablelm(c: ModelConfig, raw: dict) -> None:
    """LayerNorm with bias, partial rotary embedding, gated SiLU MLP (reference src/models/stablelm.rs)."""
    c.extra["norm"] = "layernorm"
    c.rms_norm_eps = float(raw.get("layer_norm_eps", 1e-5))
    c.attention_bias = bool(raw.get("use_qkv_bias", False))
    c.extra["parallel_block"] = bool(raw.get("use_parallel_residual", False))
    if raw.get("qk_layernorm"):
        raise ValueError("stablelm with per-head q/k LayerNorm is not supported")


def _cohere(c: ModelConfig, raw: dict) -> None:
    """Bias-free LayerNorm, attention and MLP in parallel from one normed input, interleaved RoPE,
    logits multiplied by logit_scale (reference src/models/cohere.rs)."""
    c.extra["norm"] = "layernorm"
    c.extra["parallel_block"] = True
    c.rms_norm_eps = float(raw.get("layer_norm_eps", 1e-5))
    c.rope_traditional = True
    c.extra["logits_scaling"] = 1.0 / float(raw.get("logit_scale", 0.0625))
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))
    if raw.get("use_qk_norm"):
        raise ValueError("cohere with q/k LayerNorm is not supported")


def _interleaved_rope(c: ModelConfig, raw: dict) -> None:
    """Llama layout with RoPE on interleaved pairs (Helium, ERNIE 4.5)."""
    c.rope_traditional = True


def _smollm3(c: ModelConfig, raw: dict) -> None:
    """Llama layout where every ``no_rope_layer_interval``-th layer has no positional encoding
    (``no_rope_layers[i] == 0``; reference src/models/smollm3.rs)."""
    flags = raw.get("no_rope_layers")
    if flags is None:
        iv = int(raw.get("no_rope_layer_interval", 4))
        flags = [int((i + 1) % iv != 0) for i in range(c.num_hidden_layers)]
    c.extra["nope_layers"] = [i for i, f in enumerate(flags) if not f]
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))


def _exaone4(c: ModelConfig, raw: dict) -> None:
    """Norms after attention / MLP only, per-head q/k RMSNorm, and (hybrid models) no positional
    encoding on the full-attention layers (reference src/models/exaone4.rs)."""
    c.qk_norm = True
    c.extra["post_norm_only"] = True
    if c.sliding_window and c.layer_types:
        c.extra["nope_layers"] = [i for i, t in enumerate(c.layer_types) if t != "sliding_attention"]


def _apertus(c: ModelConfig, raw: dict) -> None:
    """Per-head q/k RMSNorm, plain MLP up -> xIELU -> down with learned per-layer activation
    parameters (reference src/models/apertus.rs)."""
    c.qk_norm = True
    c.extra["mlp"] = "plain"
    c.hidden_act = "xielu"


def _minicpm(c: ModelConfig, raw: dict) -> None:
    """Llama layout with scaled embeddings, depth-scaled residual branches and width-scaled logits
    (reference src/models/minicpm.rs)."""
    c.embed_scale = float(raw.get("scale_emb", 1.0))
    c.extra["residual_multiplier"] = float(raw.get("scale_depth", 1.0)) / math.sqrt(c.num_hidden_layers)
    c.extra["logits_scaling"] = c.hidden_size / float(raw.get("dim_model_base", c.hidden_size))


def _phi(c: ModelConfig, raw: dict) -> None:
    """Phi-1 / Phi-2: one LayerNorm feeding attention and a plain GELU MLP in parallel, partial rotary
    embedding, biases everywhere including the LM head (reference src/models/phi.rs)."""
    c.extra["norm"] = "layernorm"
    c.extra["parallel_block"] = True
    c.extra["mlp"] = "plain"
    c.hidden_act = _plain_act(c)
    c.rms_norm_eps = float(raw.get("layer_norm_eps", 1e-5))
    c.attention_bias = c.mlp_bias = True
    if raw.get("qk_layernorm"):
        raise ValueError("phi with q/k LayerNorm is not supported")


def _gpt_neox(c: ModelConfig, raw: dict) -> None:
    """GPT-NeoX / Pythia: LayerNorm with bias, attention and MLP in parallel from two norms of the
    same stream, rotary embedding on a quarter of each head, plain GELU MLP, fused per-head qkv
    (reference src/models/gpt_neox.rs; re-layout in loading/aliases.py)."""
    c.extra["norm"] = "layernorm"
    c.extra["mlp"] = "plain"
    c.extra["parallel_block"] = bool(raw.get("use_parallel_residual", True))
    c.hidden_act = _plain_act(c)
    c.rms_norm_eps = float(raw.get("layer_norm_eps", 1e-5))
    c.attention_bias = c.mlp_bias = True
    c.num_key_value_heads = c.num_attention_heads
    c.head_dim = c.hidden_size // c.num_attention_heads
    if "partial_rotary_factor" not in raw and not (raw.get("rope_parameters") or {}).get("partial_rotary_factor"):
        c.partial_rotary_factor = float(raw.get("rotary_pct", 0.25))


def _gpt2(c: ModelConfig, raw: dict) -> None:
    """GPT-2 and GPT-BigCode (StarCoder-1, SantaCoder): learned absolute positions, LayerNorm with
    bias, plain GELU MLP, fused c_attn (multi-query in BigCode) (reference src/models/gpt2.rs,
    gpt_bigcode.rs)."""
    c.extra["norm"] = "layernorm"
    c.extra["mlp"] = "plain"
    c.hidden_act = _plain_act(c)
    c.intermediate_size = int(raw.get("n_inner") or 4 * c.hidden_size)
    c.rms_norm_eps = float(raw.get("layer_norm_epsilon", 1e-5))
    c.attention_bias = c.mlp_bias = True
    c.partial_rotary_factor = 0.0
    c.max_position_embeddings = int(raw.get("n_positions", c.max_position_embeddings))
    c.num_key_value_heads = 1 if raw.get("multi_query", c.model_type == "gpt_bigcode") and c.model_type == "gpt_bigcode" \
        else c.num_attention_heads
    c.head_dim = c.hidden_size // c.num_attention_heads
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))
    if raw.get("scale_attn_by_inverse_layer_idx"):
        raise ValueError("gpt2 with scale_attn_by_inverse_layer_idx is not supported")


def _olmo1(c: ModelConfig, raw: dict) -> None:
    """OLMo-1: LayerNorm without parameters, otherwise the Llama layout (reference src/models/olmo.rs)."""
    c.extra["norm"] = "layernorm"
    c.extra["norm_no_params"] = True
    c.rms_norm_eps = 1e-5
    if raw.get("clip_qkv"):
        raise ValueError("olmo with clip_qkv is not supported")


def _granitemoehybrid(c: ModelConfig, raw: dict) -> None:
    """Granite 4 hybrid: every layer is a Mamba2 or an attention mixer followed by a gated shared
    MLP (plus top-k routed experts when ``num_local_experts > 0``), with Granite's embedding / residual / attention / logit multipliers; attention carries RoPE
    only when ``position_embedding_type == "rope"`` (reference src/models/granitemoehybrid.rs).
    Runs on the hybrid executor as the block pattern ``MG`` / ``*G`` per layer."""
    _granite(c, raw)
    c.num_experts = int(raw.get("num_local_experts", 0) or 0)
    if c.num_experts:
        c.moe_route_mode = "topk_softmax"
        c.moe_intermediate_size = c.intermediate_size
        c.num_experts_per_tok = int(raw.get("num_experts_per_tok", c.num_experts_per_tok or 2))
    P = int(raw.get("mamba_d_head", 64))
    heads = int(raw.get("mamba_n_heads", raw.get("mamba_expand", 2) * c.hidden_size // P))
    lim = raw.get("time_step_limit") or (0.0, float("inf"))
    c.extra["mamba"] = dict(d_inner=heads * P, head_dim=P, n_groups=int(raw.get("mamba_n_groups", 1)),
                            d_state=int(raw.get("mamba_d_state", 128)), d_conv=int(raw.get("mamba_d_conv", 4)),
                            time_step_limit=(_num(lim[0]), _num(lim[1])), norm_groups=1)
    types = raw.get("layer_types") or ["mamba"] * c.num_hidden_layers
    c.extra["hybrid_pattern"] = "".join(("M" if t == "mamba" else "*") + ("E" if c.num_experts else "G") for t in types)
    c.extra["hybrid_layout"] = "granite"
    c.extra["mlp_size"] = int(raw.get("shared_intermediate_size", c.intermediate_size))
    c.layer_types = None
    if raw.get("position_embedding_type") != "rope":
        c.partial_rotary_factor = 0.0


def _qwen3_next(c: ModelConfig, raw: dict) -> None:
    """Qwen3-Next: Gated DeltaNet layers and gated full-attention layers (per-head (1 + w) q/k norms,
    rotary embedding on a quarter of each head, sigmoid output gate), each followed by a MoE with a
    gated shared expert (or a dense MLP); norms are stored as (weight - 1)
    (reference src/models/qwen3_next.rs). Runs on the hybrid executor as ``L`` / ``A`` + ``E`` / ``G``.
    Qwen3.5 (dense) and Qwen3.5-MoE language models are the same stack with the linear-attention input
    projection stored as four matrices (reference src/models/qwen3_5.rs)."""
    n = c.num_hidden_layers
    types = raw.get("layer_types")
    if not types:
        iv = int(raw.get("full_attention_interval", 4))
        types = ["full_attention" if (i + 1) % iv == 0 else "linear_attention" for i in range(n)]
    c.num_experts = int(raw.get("num_experts", 0) or 0)
    c.moe_route_mode = "softmax_topk"
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", True))
    step = int(raw.get("decoder_sparse_step", 1) or 1)
    dense = set(raw.get("mlp_only_layers") or [])
    pat = ""
    for i, t in enumerate(types):
        pat += "A" if t == "full_attention" else "L"
        pat += "E" if (c.num_experts > 0 and i not in dense and (i + 1) % step == 0) else "G"
    c.extra["hybrid_pattern"], c.extra["hybrid_layout"] = pat, "qwen3_next"
    c.extra["gdn"] = dict(k_heads=int(raw.get("linear_num_key_heads", 16)), v_heads=int(raw.get("linear_num_value_heads", 32)),
                          k_dim=int(raw.get("linear_key_head_dim", 128)), v_dim=int(raw.get("linear_value_head_dim", 128)),
                          d_conv=int(raw.get("linear_conv_kernel_dim", 4)))
    c.qk_norm = True
    if "partial_rotary_factor" not in raw and not (raw.get("rope_parameters") or {}).get("partial_rotary_factor"):
        c.partial_rotary_factor = 0.25
    c.layer_types = None
    c.sliding_window = 0


def _falcon_h1(c: ModelConfig, raw: dict) -> None:
    """Falcon-H1: every layer runs a Mamba2 mixer and rotary attention in parallel on the same normed
    input, then a gated MLP; the muP multipliers of the checkpoint (embedding, mixer input / per-segment
    / output, attention input / key / output, MLP gate / down, LM head) are folded into the weights at
    load (reference src/models/falcon_h1.rs). Runs on the hybrid executor as ``P`` + ``G`` per layer."""
    hs = c.hidden_size
    P = int(raw.get("mamba_d_head", 64))
    d_inner = int(raw.get("mamba_d_ssm") or raw.get("mamba_expand", 2) * hs)
    G = int(raw.get("mamba_n_groups", 1))
    lim = raw.get("time_step_limit") or (0.0, float("inf"))
    mode = "none"
    if raw.get("mamba_rms_norm", False):
        mode = "norm_then_gate" if raw.get("mamba_norm_before_gate", True) else "gate_then_norm"
    c.extra["mamba"] = dict(d_inner=d_inner, head_dim=P, n_groups=G, d_state=int(raw.get("mamba_d_state", 128)),
                            d_conv=int(raw.get("mamba_d_conv", 4)), time_step_limit=(_num(lim[0]), _num(lim[1])),
                            norm_groups=G, gate_mode=mode)
    c.extra["hybrid_pattern"], c.extra["hybrid_layout"] = "PG" * c.num_hidden_layers, "falcon_h1"
    c.embed_scale = float(raw.get("embedding_multiplier", 1.0))
    c.extra["logits_scaling"] = 1.0 / float(raw.get("lm_head_multiplier", 1.0))
    sm = raw.get("ssm_multipliers") or [1.0] * 5
    mm = raw.get("mlp_multipliers") or [1.0, 1.0]
    c.extra["falcon_mup"] = dict(ssm_in=float(raw.get("ssm_in_multiplier", 1.0)), ssm=[float(v) for v in sm],
                                 ssm_out=float(raw.get("ssm_out_multiplier", 1.0)),
                                 attn_in=float(raw.get("attention_in_multiplier", 1.0)),
                                 key=float(raw.get("key_multiplier", 1.0)),
                                 attn_out=float(raw.get("attention_out_multiplier", 1.0)),
                                 gate=float(mm[0]), down=float(mm[1]))
    c.layer_types = None
    c.sliding_window = 0


def _jamba(c: ModelConfig, raw: dict) -> None:
    """Jamba: first-generation Mamba mixers (with RMSNorm on dt / B / C) and attention without
    positional encoding, interleaved by ``attn_layer_period / offset``; every layer ends in a gated
    MLP or, every ``expert_layer_period``-th, a softmax top-k MoE (reference src/models/jamba.rs).
    Runs on the hybrid executor as the block pattern ``m`` / ``*`` + ``G`` / ``E`` per layer."""
    n = c.num_hidden_layers
    ap, ao = int(raw.get("attn_layer_period", 8)), int(raw.get("attn_layer_offset", 4))
    ep, eo = int(raw.get("expert_layer_period", 2)), int(raw.get("expert_layer_offset", 1))
    c.num_experts = int(raw.get("num_experts", 0) or 0)
    c.moe_intermediate_size = c.intermediate_size
    c.moe_route_mode, c.norm_topk_prob = "softmax_topk", False
    pat = ""
    for i in range(n):
        pat += "*" if i % ap == ao else "m"
        pat += "E" if (c.num_experts > 1 and i % ep == eo) else "G"
    c.extra["hybrid_pattern"], c.extra["hybrid_layout"] = pat, "jamba"
    hs = c.hidden_size
    rank = raw.get("mamba_dt_rank", "auto")
    c.extra["mamba1"] = dict(d_inner=int(raw.get("mamba_expand", 2)) * hs, d_state=int(raw.get("mamba_d_state", 16)),
                             d_conv=int(raw.get("mamba_d_conv", 4)),
                             dt_rank=math.ceil(hs / 16) if rank in ("auto", None, 0) else int(rank))
    c.partial_rotary_factor = 0.0
    c.layer_types = None
    c.sliding_window = 0


def _granitemoe(c: ModelConfig, raw: dict) -> None:
    _granite(c, raw)
    c.moe_route_mode = "topk_softmax"
    c.moe_intermediate_size = c.intermediate_size


def _granitemoeshared(c: ModelConfig, raw: dict) -> None:
    """GraniteMoE with an always-on shared gated MLP beside the routed experts (reference src/models/granitemoe*.rs)."""
    _granitemoe(c, raw)
    c.shared_expert_intermediate_size = int(raw.get("shared_intermediate_size", 0) or 0)


def _deepseek_routing(c: ModelConfig, raw: dict) -> None:
    """Sigmoid scores + correction bias + group-limited top-k + scaled weights, shared experts always
    on, the first ``first_k_dense_replace`` layers dense (DeepSeek-V3 routing; reference
    src/models/switch_layers.rs group-limited masks, src/models/glm4_moe.rs)."""
    c.moe_route_mode = "sigmoid_group"
    c.num_experts = int(raw.get("n_routed_experts", c.num_experts) or 0)
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", True))
    c.extra["moe_routing"] = dict(n_group=int(raw.get("n_group", 1) or 1), topk_group=int(raw.get("topk_group", 1) or 1),
                                  scale=float(raw.get("routed_scaling_factor", 1.0)))
    c.extra["first_k_dense"] = int(raw.get("first_k_dense_replace", 0) or 0)
    c.shared_expert_intermediate_size = c.moe_intermediate_size * int(raw.get("n_shared_experts", 0) or 0)
    c.router_bias = True                         # the correction bias travels in router_b


def _yarn_mscale(factor: float, m: float) -> float:
    return 1.0 if factor <= 1 or not m else 0.1 * m * math.log(factor) + 1.0


def _deepseek_mla(c: ModelConfig, raw: dict) -> None:
    """Multi-head latent attention geometry. The paged pool stores expanded per-head keys and values
    padded to one head size (64 / 128 / 256), see ``DecoderModel._attention_mla``."""
    nope, rope_d, vd = int(raw["qk_nope_head_dim"]), int(raw["qk_rope_head_dim"]), int(raw["v_head_dim"])
    qk = nope + rope_d
    big = max(qk, vd)
    if big > 256:
        raise ValueError("MLA head dimensions above 256 are not supported")
    c.extra["mla"] = dict(q_lora_rank=raw.get("q_lora_rank"), kv_lora_rank=int(raw["kv_lora_rank"]), nope=nope,
                          rope=rope_d, v=vd, interleave=bool(raw.get("rope_interleave", True)))
    c.head_dim = 64 if big <= 64 else 128 if big <= 128 else 256
    c.num_key_value_heads = c.num_attention_heads
    scale = qk ** -0.5
    rs = c.rope_scaling
    if rs and rs.get("rope_type", rs.get("type")) == "yarn":
        f = float(rs.get("factor", 1.0))
        if rs.get("mscale_all_dim"):
            scale *= _yarn_mscale(f, float(rs["mscale_all_dim"])) ** 2
            if rs.get("mscale") and rs.get("attention_factor") is None:
                rs = dict(rs)
                rs["attention_factor"] = _yarn_mscale(f, float(rs["mscale"])) / _yarn_mscale(f, float(rs["mscale_all_dim"]))
                c.rope_scaling = rs
    c.query_pre_attn_scalar = 1.0 / (scale * scale)


def _deepseek_v3(c: ModelConfig, raw: dict) -> None:
    """DeepSeek-V3 / R1 (and Kimi-K2 with the same layout): multi-head latent attention + sigmoid
    group-limited routing with shared experts (reference src/models/deepseek_v3.rs)."""
    _deepseek_routing(c, raw)
    _deepseek_mla(c, raw)


def _glm_moe_dsa(c: ModelConfig, raw: dict) -> None:
    """GLM-5 / DeepSeek-V3.2 layout: the DeepSeek-V3 model (latent attention, sigmoid group-limited
    routing) with half-split rotary pairs and a sparse-attention indexer that keeps the ``index_topk``
    best keys of every query. Contexts are served up to ``index_topk`` tokens, where the selection
    keeps every key and attention is dense; the indexer itself is not built
    (reference src/models/glm_moe_dsa.rs, deepseek_v32.rs)."""
    raw = dict(raw)
    raw.setdefault("rope_interleave", False)
    _deepseek_v3(c, raw)
    topk = int(raw.get("index_topk", 2048) or 2048)
    c.extra["dsa_index_topk"] = topk
    c.max_position_embeddings = min(c.max_position_embeddings, topk)


def _deepseek_v2(c: ModelConfig, raw: dict) -> None:
    """DeepSeek-V2 / V2-Lite: multi-head latent attention, softmax routing (greedy or limited to the
    groups with the best single score), weights not normalised, shared experts
    (reference src/models/deepseek_v2.rs)."""
    _deepseek_routing(c, raw)
    c.router_bias = False
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", False))
    r = c.extra["moe_routing"]
    r.update(score="softmax", group_score="max")
    if raw.get("topk_method", "greedy") == "greedy":
        r.update(n_group=1, topk_group=1)
    _deepseek_mla(c, raw)


def _glm4_moe(c: ModelConfig, raw: dict) -> None:
    """GLM-4.5 / 4.6: half-rotary GQA attention with biased q/k/v and optional per-head q/k norm,
    DeepSeek-V3 style MoE (reference src/models/glm4_moe.rs)."""
    _deepseek_routing(c, raw)
    if "partial_rotary_factor" not in raw and not (raw.get("rope_parameters") or {}).get("partial_rotary_factor"):
        c.partial_rotary_factor = 0.5
    c.attention_bias = bool(raw.get("attention_bias", False))
    c.qk_norm = bool(raw.get("use_qk_norm", False))


def _ernie4_5_moe(c: ModelConfig, raw: dict) -> None:
    """ERNIE 4.5 MoE: interleaved RoPE, softmax routing with a selection bias, shared experts, dense
    layers before ``moe_layer_start_index`` (reference src/models/ernie4_5_moe.rs)."""
    c.rope_traditional = True
    c.moe_route_mode = "sigmoid_group"
    c.num_experts = int(raw.get("moe_num_experts", 0) or 0)
    c.num_experts_per_tok = int(raw.get("moe_k", 2))
    c.moe_intermediate_size = int(raw.get("moe_intermediate_size", c.intermediate_size))
    c.norm_topk_prob = True
    c.extra["moe_routing"] = dict(n_group=1, topk_group=1, scale=1.0, score="softmax",
                                  norm_min=float(raw.get("moe_norm_min", 1e-12)))
    c.extra["first_k_dense"] = int(raw.get("moe_layer_start_index", 0) or 0)
    if int(raw.get("moe_layer_interval", 1) or 1) != 1:
        raise ValueError("ernie4_5_moe with moe_layer_interval != 1 is not supported")
    c.shared_expert_intermediate_size = c.moe_intermediate_size * int(raw.get("moe_num_shared_experts", 0) or 0)
    c.router_bias = True
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))


def _dots1(c: ModelConfig, raw: dict) -> None:
    """dots.llm1: Qwen3-style attention (per-head q/k norm) with DeepSeek-V3 style MoE
    (reference src/models/dots1.rs)."""
    _deepseek_routing(c, raw)
    c.qk_norm = True


def _phimoe(c: ModelConfig, raw: dict) -> None:
    """Phi-3.5-MoE: LayerNorm with bias, biased attention projections and LM head, top-2 SparseMixer
    routing (reference src/models/phimoe.rs)."""
    c.extra["norm"] = "layernorm"
    c.attention_bias = True
    c.moe_route_mode = "sparsemixer"
    c.num_experts_per_tok = 2
    c.moe_intermediate_size = c.intermediate_size
    c.extra["router_jitter"] = float(raw.get("router_jitter_noise", 0.01))


def _bitnet(c: ModelConfig, raw: dict) -> None:
    """BitNet b1.58: the Llama layout with an RMSNorm of the attention output in front of ``o_proj``
    (``attn_sub_norm``), one of ``relu(gate)^2 * up`` in front of ``down_proj`` (``ffn_sub_norm``), and
    every projection stored as ternary weights packed four to a byte with one scale
    (reference src/models/bitnet.rs). The packed projections are expanded to bf16 at load (their
    values are exactly representable) and run on the dense GEMMs; like the reference's
    ``bitlinear_matmul`` the activations are not quantized."""
    c.hidden_act = "relu2"
    c.extra["sub_norms"] = True
    qc = raw.get("quantization_config") or {}
    # packed scales divide the output unless the checkpoint was written by the "autobitlinear" class
    c.extra["bitlinear_invert_scale"] = (qc.get("linear_class") or "bitlinear") != "autobitlinear"
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))


def _llama4(c: ModelConfig, raw: dict) -> None:
    """Llama 4 language model (Scout / Maverick): interleaved (pairwise) rotary embedding on most
    layers and none on every ``no_rope_layer_interval``-th, weightless per-head RMS ("L2") norm of q
    and k on the rotary layers, a position-dependent query temperature on the others, and MoE layers
    (``moe_layers``) whose router takes the sigmoid of the top-1 logit and scales the expert's INPUT
    with it, beside an always-on shared expert; the other layers are dense MLPs of
    ``intermediate_size_mlp`` (reference src/models/llama4.rs, llama4_helpers.rs). The rotary layers
    attend inside chunks of ``attention_chunk_size`` tokens; contexts are served up to that size,
    where chunked and full attention coincide."""
    c.num_experts = int(raw.get("num_local_experts", 16))
    c.num_experts_per_tok = int(raw.get("num_experts_per_tok", 1))
    if c.num_experts_per_tok != 1:
        raise ValueError("llama4: only top-1 routing is supported (the router score scales the expert input)")
    c.moe_intermediate_size = int(raw.get("intermediate_size", 8192))
    c.intermediate_size = int(raw.get("intermediate_size_mlp", 16384))
    c.moe_route_mode = "sigmoid_input"
    c.rope_traditional = True
    flags = raw.get("no_rope_layers")
    if not flags:
        iv = int(raw.get("no_rope_layer_interval", 4))
        flags = [int((i + 1) % iv != 0) for i in range(c.num_hidden_layers)]
    c.extra["nope_layers"] = [i for i, f in enumerate(flags) if not f]
    if raw.get("use_qk_norm", True):
        c.qk_norm = True
        c.extra["qk_norm_no_params"] = True
        c.extra["qk_norm_rope_layers_only"] = True
    if raw.get("attn_temperature_tuning", True):
        c.extra["nope_query_temperature"] = (float(raw.get("attn_scale", 0.1)), float(raw.get("floor_scale", 8192)))
    chunk = raw.get("attention_chunk_size")
    if chunk:
        c.extra["attention_chunk_size"] = int(chunk)
        c.max_position_embeddings = min(c.max_position_embeddings, int(chunk))
    c.sliding_window = 0
    c.layer_types = None


def _dbrx(c: ModelConfig, raw: dict) -> None:
    """DBRX: bias-free LayerNorm, one fused ``Wqkv`` whose output is clamped to +-clip_qkv, rotary GQA
    attention, top-k of 16 gated experts with softmax over all experts renormalised over the chosen
    ones (= softmax over the k logits) (reference src/models/dbrx.rs). The config nests its fields under
    ``attn_config`` / ``ffn_config`` and uses the MPT names."""
    a, f = raw.get("attn_config") or {}, raw.get("ffn_config") or {}
    c.hidden_size = int(raw.get("d_model", c.hidden_size))
    c.num_attention_heads = int(raw.get("n_heads", c.num_attention_heads))
    c.num_hidden_layers = int(raw.get("n_layers", c.num_hidden_layers))
    c.num_key_value_heads = int(a.get("kv_n_heads", c.num_attention_heads))
    c.head_dim = c.hidden_size // c.num_attention_heads
    c.max_position_embeddings = int(raw.get("max_seq_len", c.max_position_embeddings))
    c.rope_theta = float(a.get("rope_theta", 10000.0))
    c.rms_norm_eps = 1e-5
    c.extra["norm"] = "layernorm"
    if a.get("clip_qkv"):
        c.extra["clip_qkv"] = float(a["clip_qkv"])
    c.num_experts = int(f.get("moe_num_experts", 16))
    c.num_experts_per_tok = int(f.get("moe_top_k", 4))
    c.intermediate_size = c.moe_intermediate_size = int(f.get("ffn_hidden_size", 4 * c.hidden_size))
    c.hidden_act = (f.get("ffn_act_fn") or {}).get("name", "silu")
    c.moe_route_mode = "topk_softmax"
    if f.get("moe_normalize_expert_weights") not in (1, 1.0):
        raise ValueError("dbrx: only moe_normalize_expert_weights = 1 is supported")
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", False))


def _hunyuan_dense(c: ModelConfig, raw: dict) -> None:
    """Hunyuan dense: Llama layout with per-head q/k RMSNorm applied after the rotary embedding
    (reference src/models/hunyuan_v1_dense.rs)."""
    c.qk_norm = True
    c.extra["qk_norm_after_rope"] = True
    rs = c.rope_scaling or {}
    if rs.get("alpha") and rs.get("rope_type", rs.get("type")) in ("dynamic", None):
        # NTK-alpha scaling: the base grows by alpha^(D / (D - 2))
        c.rope_theta = c.rope_theta * float(rs["alpha"]) ** (c.head_dim / (c.head_dim - 2))


def _hunyuan_moe(c: ModelConfig, raw: dict) -> None:
    """Hunyuan MoE (Hunyuan-A13B): the dense layout plus softmax top-k experts (renormalised) and an
    always-on shared MLP (reference src/models/hunyuan_moe.rs)."""
    _hunyuan_dense(c, raw)
    c.moe_route_mode, c.norm_topk_prob = "softmax_topk", True
    k = raw.get("moe_topk", 2)
    c.num_experts_per_tok = int(k[0] if isinstance(k, (list, tuple)) else k)
    c.moe_intermediate_size = c.intermediate_size
    c.shared_expert_intermediate_size = c.intermediate_size


def _arcee(c: ModelConfig, raw: dict) -> None:
    """Llama layout with a plain MLP up -> relu^2 -> down (reference src/models/arcee.rs)."""
    c.extra["mlp"] = "plain"
    c.hidden_act = "relu2"


def _ministral3(c: ModelConfig, raw: dict) -> None:
    """Ministral 3: the Mistral layout with YaRN frequencies and a position-dependent query scale
    ``1 + beta * log(1 + floor(pos / original_max_position))`` (reference src/models/ministral3.rs)."""
    rp = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
    if rp.get("llama_4_scaling_beta"):
        c.extra["llama4_attn_scale"] = (float(rp["llama_4_scaling_beta"]),
                                        int(rp.get("original_max_position_embeddings") or c.max_position_embeddings))


def _recurrent_gemma(c: ModelConfig, raw: dict) -> None:
    """RecurrentGemma (Griffin): residual blocks whose temporal mixer is an RG-LRU recurrent block or
    local multi-query attention (``block_types`` repeated over the layers), each followed by a gated
    tanh-GELU MLP with biases; Gemma conventions elsewhere ((1 + w) norms, sqrt(hidden) embedding
    scale, tied head, logit soft cap) (reference src/models/recurrent_gemma.rs). Runs on the hybrid
    executor as ``R`` / ``*`` + ``G``."""
    n = c.num_hidden_layers
    types = list(raw.get("block_types") or ("recurrent", "recurrent", "attention"))
    kinds = (types * n)[:n]
    c.extra["hybrid_pattern"] = "".join(("R" if k == "recurrent" else "*") + "G" for k in kinds)
    c.extra["hybrid_layout"] = "recurrent_gemma"
    c.extra["rglru"] = dict(width=int(raw.get("lru_width") or c.hidden_size), heads=c.num_attention_heads,
                            d_conv=int(raw.get("conv1d_width", 4)))
    c.num_key_value_heads = int(raw.get("num_key_value_heads") or 1)
    c.head_dim = int(raw.get("head_dim") or c.hidden_size // c.num_attention_heads)
    c.partial_rotary_factor = float(raw.get("partial_rotary_factor", 0.5))
    c.sliding_window = int(raw.get("attention_window_size", 2048))
    c.layer_types = None
    c.intermediate_size = int(raw.get("intermediate_size", 3 * c.hidden_size)) // 2     # the config counts gate + up
    c.hidden_act = "gelu_tanh"
    c.embed_scale = math.sqrt(c.hidden_size)
    c.final_logit_softcap = float(raw.get("logits_soft_cap", 30.0) or 0.0)
    c.rms_norm_eps = float(raw.get("rms_norm_eps", 1e-6))
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))
    c.attention_bias = bool(raw.get("attention_bias", False))


def _exaone(c: ModelConfig, raw: dict) -> None:
    """EXAONE 3.x: the Llama architecture under GPT-2 style names (``transformer.h.N.attn.attention.*``,
    ``mlp.c_fc_0 / c_fc_1 / c_proj``, ``ln_1 / ln_2``, ``wte``, ``ln_f``), presented to the loader
    through aliases (reference src/models/exaone.rs)."""
    c.num_hidden_layers = int(raw.get("num_layers", c.num_hidden_layers))
    c.rms_norm_eps = float(raw.get("layer_norm_epsilon", raw.get("rms_norm_eps", 1e-5)))
    c.hidden_act = "silu"


def _telechat3(c: ModelConfig, raw: dict) -> None:
    """TeleChat3: the Llama decoder with YaRN frequencies (its config spells the type
    ``telechat3-yarn``) and optional biases on q / k / v / o (reference src/models/telechat3.rs)."""
    rs = c.rope_scaling
    if rs and str(rs.get("rope_type", rs.get("type", ""))).endswith("yarn"):
        rs = dict(rs)
        rs["rope_type"] = "yarn"
        rs.pop("type", None)
        c.rope_scaling = rs
    c.attention_bias = bool(raw.get("attention_bias", False))


def _deepseek_v1(c: ModelConfig, raw: dict) -> None:
    """DeepSeek-MoE (v1): Llama attention; MoE layers with softmax top-k routing (weights not
    normalised unless the config says so, scaled by ``routed_scaling_factor``), always-on shared
    experts, the first ``first_k_dense_replace`` layers dense (reference src/models/deepseek.rs)."""
    if int(raw.get("moe_layer_freq", 1) or 1) != 1:
        raise ValueError("deepseek with moe_layer_freq != 1 is not supported")
    _deepseek_routing(c, raw)
    c.router_bias = False
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", False))
    c.extra["moe_routing"].update(score="softmax", group_score="max", n_group=1, topk_group=1)


def _afmoe(c: ModelConfig, raw: dict) -> None:
    """Arcee AFM MoE (Trinity): norms before and after both the attention and the MLP / MoE block,
    per-head q/k RMSNorm, rotary embedding on the sliding-window layers only, a sigmoid output gate on
    the attention (``gate_proj``), sigmoid router with a selection bias, normalised and scaled
    weights, shared experts, ``num_dense_layers`` dense layers first, optional muP input scaling
    (reference src/models/afmoe.rs)."""
    n = c.num_hidden_layers
    c.post_norms = True
    c.extra["post_norm_names"] = ("post_attention_layernorm", "pre_mlp_layernorm", "post_mlp_layernorm")
    c.qk_norm = True
    if c.layer_types is None:
        every = int(raw.get("global_attn_every_n_layers", 4) or 4)
        c.layer_types = ["full_attention" if (i + 1) % every == 0 else "sliding_attention" for i in range(n)]
    c.extra["nope_layers"] = [i for i, t in enumerate(c.layer_types) if t != "sliding_attention"]
    c.extra["attn_output_gate"] = True
    c.num_experts = int(raw.get("num_experts", 0) or 0)
    c.moe_route_mode = "sigmoid_group"
    c.norm_topk_prob = True
    c.extra["moe_routing"] = dict(n_group=1, topk_group=1, scale=float(raw.get("route_scale", 1.0) or 1.0), norm_min=1e-20)
    c.extra["first_k_dense"] = int(raw.get("num_dense_layers", 0) or 0)
    c.shared_expert_intermediate_size = c.moe_intermediate_size * int(raw.get("num_shared_experts", 0) or 0)
    c.router_bias = True
    if raw.get("mup_enabled"):
        c.embed_scale = math.sqrt(c.hidden_size)


def _mistral4(c: ModelConfig, raw: dict) -> None:
    """Mistral 4 (Mistral Small 4 / Large 3 line): multi-head latent attention with the Ministral-3
    position-dependent query scale and no YaRN factor in the softmax scale, softmax router limited to
    the best groups (sum of each group's two best scores), normalised and scaled weights, shared
    experts, dense layers first; experts stored fused as [E, 2I, H] / [E, H, I]
    (reference src/models/mistral4.rs)."""
    _deepseek_routing(c, raw)
    c.router_bias = False
    c.extra["moe_routing"].update(score="softmax", group_score="top2sum", norm_min=1e-20)
    _deepseek_mla(c, raw)
    qk = int(raw["qk_nope_head_dim"]) + int(raw["qk_rope_head_dim"])
    c.query_pre_attn_scalar = float(qk)                 # plain 1 / sqrt(qk): no mscale^2 factor here
    _ministral3(c, raw)


def _nanochat(c: ModelConfig, raw: dict) -> None:
    """nanochat: RMSNorm without gains everywhere (blocks, final, and per-head q/k norms applied AFTER the
    rotary embedding), plain MLP fc1 -> relu^2 -> fc2, logit soft cap (reference src/models/nanochat.rs)."""
    c.extra["norm_no_params"] = True
    c.qk_norm = True
    c.extra["qk_norm_after_rope"] = True
    c.extra["qk_norm_no_params"] = True
    c.extra["rope_negate"] = True          # its rotate_half is (x2, -x1)
    c.extra["embed_norm"] = True           # the embeddings are normalised before the first block
    c.extra["mlp"] = "plain"
    c.hidden_act = "relu2"


def _glm(c: ModelConfig, raw: dict) -> None:
    """GLM-4 (2024): interleaved RoPE on half of each head, biased q/k/v, fused gate_up projection
    (reference src/models/glm4.rs)."""
    c.rope_traditional = True
    if "partial_rotary_factor" not in raw and not (raw.get("rope_parameters") or {}).get("partial_rotary_factor"):
        c.partial_rotary_factor = 0.5
    c.attention_bias = bool(raw.get("attention_bias", True))


def _glm4(c: ModelConfig, raw: dict) -> None:
    """GLM-4-0414: the GLM layout plus norms after attention and after the MLP (sandwich)."""
    _glm(c, raw)
    c.post_norms = True
    c.extra["post_norm_names"] = ("post_self_attn_layernorm", "post_attention_layernorm", "post_mlp_layernorm")


def _glm4v(c: ModelConfig, raw: dict) -> None:
    """Language model of GLM-4.1V / GLM-4.5V dense: GLM-4-0414 blocks whose rotary half-heads take
    multimodal positions (temporal / height / width sections, pairs of adjacent columns)."""
    _glm4(c, raw)
    for rec in (raw.get("rope_parameters"), raw.get("rope_scaling")):
        if isinstance(rec, dict) and rec.get("mrope_section"):
            c.extra["mrope_section"] = [int(x) for x in rec["mrope_section"]]
    rs = c.rope_scaling
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) in ("mrope", "default", None):
        c.rope_scaling = None


def _glm_ocr(c: ModelConfig, raw: dict) -> None:
    """Language model of GLM-OCR: the GLM-4V one without biases on q / k / v."""
    _glm4v(c, raw)
    c.attention_bias = False


def _paddleocr_vl(c: ModelConfig, raw: dict) -> None:
    """Language model of PaddleOCR-VL: Llama-layout blocks (optional projection biases) with multimodal
    rotary positions in half-split pairs."""
    c.attention_bias = bool(raw.get("use_bias", False))
    c.mlp_bias = bool(raw.get("use_bias", False))
    for rec in (raw.get("rope_parameters"), raw.get("rope_scaling")):
        if isinstance(rec, dict) and rec.get("mrope_section"):
            c.extra["mrope_section"] = [int(x) for x in rec["mrope_section"]]
    rs = c.rope_scaling
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) in ("mrope", "default", None):
        c.rope_scaling = None


def _glm4v_moe(c: ModelConfig, raw: dict) -> None:
    """Language model of GLM-4.5V: GLM-4.5 MoE blocks (half-split rotary pairs on half of each head) with
    multimodal rotary positions."""
    _glm4_moe(c, raw)
    for rec in (raw.get("rope_parameters"), raw.get("rope_scaling")):
        if isinstance(rec, dict) and rec.get("mrope_section"):
            c.extra["mrope_section"] = [int(x) for x in rec["mrope_section"]]
    rs = c.rope_scaling
    if isinstance(rs, dict) and rs.get("rope_type", rs.get("type")) in ("mrope", "default", None):
        c.rope_scaling = None


def _cohere2(c: ModelConfig, raw: dict) -> None:
    """Cohere layout with sliding-window layers that rotate and full-attention layers without
    positional encoding (reference src/models/cohere2.rs)."""
    _cohere(c, raw)
    if c.layer_types is None and c.sliding_window:
        pat = int(raw.get("sliding_window_pattern", 4) or 4)
        c.layer_types = ["full_attention" if (i + 1) % pat == 0 else "sliding_attention"
                         for i in range(c.num_hidden_layers)]
    if c.layer_types:
        c.extra["nope_layers"] = [i for i, t in enumerate(c.layer_types) if t != "sliding_attention"]


def _nemotron(c: ModelConfig, raw: dict) -> None:
    """Nemotron-4 / Minitron: LayerNorm stored as (weight - 1) with bias, partial rotary embedding,
    plain MLP up -> relu^2 -> down (reference src/models/nemotron.rs)."""
    c.extra["norm"] = "layernorm"
    c.extra["norm_plus_one"] = True
    c.extra["mlp"] = "plain"
    c.hidden_act = "relu2"
    c.rms_norm_eps = float(raw.get("norm_eps", 1e-5))
    if "partial_rotary_factor" not in raw and not (raw.get("rope_parameters") or {}).get("partial_rotary_factor"):
        c.partial_rotary_factor = 0.5


def _olmoe(c: ModelConfig, raw: dict) -> None:
    _qwen_moe(c, raw)
    c.attention_bias = False
    c.qk_norm = True
    c.extra["qk_norm_full"] = True
    c.norm_topk_prob = bool(raw.get("norm_topk_prob", False))


def _granite(c: ModelConfig, raw: dict) -> None:
    c.embed_scale = float(raw.get("embedding_multiplier", 1.0))
    c.extra["residual_multiplier"] = float(raw.get("residual_multiplier", 1.0))
    c.extra["logits_scaling"] = float(raw.get("logits_scaling", 1.0))
    if raw.get("attention_multiplier"):
        c.query_pre_attn_scalar = 1.0 / float(raw["attention_multiplier"]) ** 2


def _num(v) -> float:
    """A JSON number, or HF's spelling of a non-finite one (``{"__float__": "Infinity"}``, ``"inf"``)."""
    if isinstance(v, dict):
        v = v.get("__float__", "inf")
    return float(v)


def _mamba1(c: ModelConfig, raw: dict) -> None:
    """First-generation Mamba (HF ``MambaConfig``; reference src/models/mamba.rs). No layer has attention:
    the attention geometry is the minimum the block pool accepts."""
    hs = c.hidden_size
    d_inner = int(raw.get("intermediate_size") or raw.get("expand", 2) * hs)
    rank = raw.get("time_step_rank", "auto")
    c.extra["mamba1"] = dict(d_inner=d_inner, d_state=int(raw.get("state_size", 16)),
                             d_conv=int(raw.get("conv_kernel", 4)),
                             dt_rank=math.ceil(hs / 16) if rank in ("auto", None, 0) else int(rank))
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))
    c.num_attention_heads = c.num_key_value_heads = 1
    c.head_dim = 16
    c.intermediate_size = d_inner


def _mamba2(c: ModelConfig, raw: dict) -> None:
    """Pure state-space model (HF ``Mamba2Config``; reference src/models/mamba2.rs:40-76). The
    attention geometry is reduced to the minimum the block pool accepts: no layer has attention."""
    hs = c.hidden_size
    P = int(raw.get("head_dim", 64))
    d_inner = int(raw.get("intermediate_size") or raw.get("expand", 2) * hs)
    if raw.get("num_heads"):
        d_inner = int(raw["num_heads"]) * P
    lim = raw.get("time_step_limit") or (0.0, float("inf"))
    c.extra["mamba"] = dict(d_inner=d_inner, head_dim=P, n_groups=int(raw.get("n_groups", 1)),
                            d_state=int(raw.get("state_size", raw.get("ssm_state_size", 128))),
                            d_conv=int(raw.get("conv_kernel", raw.get("d_conv", 4))),
                            time_step_limit=(_num(lim[0]), _num(lim[1])),
                            use_bias=bool(raw.get("use_bias", False)),
                            use_conv_bias=bool(raw.get("use_conv_bias", True)))
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", True))
    c.num_attention_heads = c.num_key_value_heads = 1
    c.head_dim = 16
    c.intermediate_size = d_inner


def _nemotron_h(c: ModelConfig, raw: dict) -> None:
    """Hybrid Mamba2 / attention / MLP stack chosen per layer by ``hybrid_override_pattern``
    (reference src/models/nemotron_h.rs). Attention has no positional encoding; the Mamba2 gated
    norm is applied per B/C group; the MLP is ``down(relu(up(x))^2)``; ``E`` blocks are a mixture of such
    plain experts (sigmoid scores, selection bias, group-limited top-k, scaled weights) plus one shared
    expert, optionally between two latent projections."""
    hs = c.hidden_size
    P = int(raw.get("mamba_head_dim", 64))
    heads = int(raw.get("mamba_num_heads", raw.get("expand", 2) * hs // P))
    G = int(raw.get("n_groups", raw.get("mamba_n_groups", 8)))
    lim = raw.get("time_step_limit") or raw.get("mamba_dt_limit") or (0.0, float("inf"))
    c.extra["mamba"] = dict(d_inner=heads * P, head_dim=P, n_groups=G,
                            d_state=int(raw.get("ssm_state_size", 128)),
                            d_conv=int(raw.get("conv_kernel", raw.get("mamba_d_conv", 4))),
                            time_step_limit=(_num(lim[0]), _num(lim[1])), norm_groups=G,
                            use_conv_bias=bool(raw.get("use_conv_bias", True)))
    pat = raw.get("hybrid_override_pattern")
    if not pat and raw.get("layers_block_type"):      # newer spelling: one word per layer
        names = {"mamba": "M", "attention": "*", "mlp": "-", "moe": "E"}
        pat = "".join(names.get(t, "?") for t in raw["layers_block_type"])
    if not pat:
        raise ValueError("nemotron_h config needs hybrid_override_pattern or layers_block_type")
    c.extra["hybrid_pattern"] = str(pat)
    c.num_hidden_layers = len(pat)
    if "E" in pat:                               # MoE blocks: DeepSeek-V3 style routing over plain relu^2 experts
        c.num_experts = int(raw.get("n_routed_experts", 0) or 0)
        c.num_experts_per_tok = int(raw.get("num_experts_per_tok", 2))
        c.moe_intermediate_size = int(raw.get("moe_intermediate_size", c.intermediate_size))
        c.norm_topk_prob = bool(raw.get("norm_topk_prob", True))
        c.extra["moe_routing"] = dict(n_group=int(raw.get("n_group", 1) or 1), topk_group=int(raw.get("topk_group", 1) or 1),
                                      scale=float(raw.get("routed_scaling_factor", 1.0)))
    c.partial_rotary_factor = 0.0
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", False))
    c.hidden_act = "relu2"


def _vaultgemma(c: ModelConfig, raw: dict) -> None:
    """VaultGemma: the Gemma-2 block (soft-capped logits, alternating sliding / full attention,
    (1 + w) norms) without the two post-norms (reference src/models/vaultgemma.rs)."""
    _gemma(c, raw)
    n = c.num_hidden_layers
    if c.layer_types is None and c.sliding_window:
        c.layer_types = ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n)]


def _solar_open(c: ModelConfig, raw: dict) -> None:
    """Solar Open: the GLM-4.5 MoE (sigmoid scores, selection bias, group-limited top-k, shared
    experts) in every layer, full-rotary GQA attention without biases or q/k norms."""
    _deepseek_routing(c, raw)
    c.extra["first_k_dense"] = 0
    c.attention_bias = False


def _minimax_m2(c: ModelConfig, raw: dict) -> None:
    """MiniMax-M2: q/k RMSNorm over the whole projection, partial rotary, sigmoid router scores with a
    selection bias, top-k weights normalised to one, no shared experts (reference
    src/models/minimax.rs)."""
    c.qk_norm = True
    c.extra["qk_norm_full"] = True
    c.moe_route_mode = "sigmoid_group"
    c.num_experts = int(raw.get("num_local_experts", raw.get("num_experts", 0)) or 0)
    c.moe_intermediate_size = c.intermediate_size
    c.norm_topk_prob = True
    c.extra["moe_routing"] = dict(n_group=1, topk_group=1, scale=1.0, norm_min=0.0)
    c.router_bias = True


def _exaone_moe(c: ModelConfig, raw: dict) -> None:
    """K-EXAONE: pre-norm blocks with the EXAONE-4 attention (per-head q/k RMSNorm, no positional
    encoding on the full-attention layers of hybrid models) and DeepSeek-V3 style MoE layers after
    ``first_k_dense_replace`` dense ones (reference src/models/exaone_moe.rs)."""
    raw = dict(raw)
    raw.setdefault("n_routed_experts", raw.get("num_experts", 0))
    raw.setdefault("n_shared_experts", raw.get("num_shared_experts", 0))
    _deepseek_routing(c, raw)
    c.qk_norm = True
    if c.sliding_window and c.layer_types:
        c.extra["nope_layers"] = [i for i, t in enumerate(c.layer_types) if t != "sliding_attention"]


def _lfm2(c: ModelConfig, raw: dict) -> None:
    """LFM2: every layer is a gated short convolution or a GQA attention layer (per-head q/k RMSNorm,
    full rotary) followed by a SwiGLU MLP (reference src/models/lfm2.rs). Runs on the hybrid executor
    as ``CG`` / ``*G`` per layer."""
    c.rms_norm_eps = float(raw.get("norm_eps", raw.get("block_norm_eps", 1e-5)))
    c.qk_norm = True
    c.tie_word_embeddings = bool(raw.get("tie_word_embeddings", raw.get("tie_embedding", True)))
    types = raw.get("layer_types")
    if not types:
        full = set(raw.get("full_attn_idxs") or [])
        types = ["full_attention" if i in full else "conv" for i in range(c.num_hidden_layers)]
    c.extra["shortconv"] = dict(d_conv=int(raw.get("conv_L_cache", 3)), bias=bool(raw.get("conv_bias", False)))
    # LFM2-MoE: the feed-forward of the layers behind the first num_dense_layers is a sparse MoE
    # (sigmoid scores + selection bias, top-k, normalised and scaled weights)
    c.num_experts = int(raw.get("num_experts", 0) or 0) if c.model_type == "lfm2_moe" else 0
    dense = int(raw.get("num_dense_layers", 0) or 0) if c.num_experts else len(types)
    if c.num_experts:
        c.moe_route_mode = "sigmoid_group"
        c.norm_topk_prob = bool(raw.get("norm_topk_prob", True))
        c.moe_intermediate_size = int(raw.get("moe_intermediate_size", c.intermediate_size))
        c.extra["moe_routing"] = dict(n_group=1, topk_group=1, scale=float(raw.get("routed_scaling_factor", 1.0)), norm_min=1e-6)
        c.router_bias = bool(raw.get("use_expert_bias", True))
    c.extra["hybrid_pattern"] = "".join(("*" if t == "full_attention" else "C") + ("G" if i < dense else "E")
                                        for i, t in enumerate(types))
    c.extra["hybrid_layout"] = "lfm2"
    c.layer_types = None


def _baichuan(c: ModelConfig, raw: dict) -> None:
    """Baichuan (7B layout): Llama block with q, k, v fused in ``W_pack`` (reference src/models/baichuan.rs).
    The 13B models replace RoPE by ALiBi, which no attention kernel here implements."""
    if raw.get("alibi") or (c.hidden_size >= 5120 and "rope_theta" not in raw and raw.get("model_max_length")):
        raise ValueError("baichuan checkpoints with ALiBi attention are not supported")
    c.num_key_value_heads = c.num_attention_heads


FAMILIES = {
    "llama": _plain, "mistral": _plain, "ministral": _plain, "smollm3": _smollm3, "seed_oss": _plain,
    "helium": _interleaved_rope, "internlm3": _plain, "exaone4": _exaone4, "hunyuan_v1_dense": _hunyuan_dense,
    "hunyuan_v1_moe": _hunyuan_moe,
    "ernie4_5": _interleaved_rope, "apertus": _apertus, "minicpm": _minicpm, "mimo": _qwen2, "yi": _plain,
    "qwen2": _qwen2, "qwen2_vl": _qwen2_vl, "qwen2_vl_text": _qwen2_vl, "qwen2_5_vl": _qwen2_vl,
    "qwen2_5_vl_text": _qwen2_vl, "qwen3_vl": _qwen3_vl, "qwen3_vl_text": _qwen3_vl, "qwen3_vl_moe": _qwen3_vl_moe, "qwen3_vl_moe_text": _qwen3_vl_moe, "qwen3": _qwen3, "qwen2_moe": _qwen_moe, "qwen3_moe": _qwen_moe,
    "mixtral": _mixtral, "phimoe": _phimoe, "olmoe": _olmoe,
    "gemma": _gemma, "gemma2": _gemma2, "gemma3_text": _gemma3, "gemma3": _gemma3,
    "gpt_oss": _gpt_oss, "phi3": _phi3, "olmo2": _olmo2, "olmo3": _olmo2,
    "mamba": _mamba1, "mamba2": _mamba2, "nemotron_h": _nemotron_h, "granite": _granite, "starcoder2": _starcoder2, "stablelm": _stablelm, "cohere": _cohere,
    "deepseek_v2": _deepseek_v2, "deepseek_v3": _deepseek_v3, "kimi_k2": _deepseek_v3, "glm4_moe": _glm4_moe, "dots1": _dots1, "ernie4_5_moe": _ernie4_5_moe,
    "gpt_neox": _gpt_neox, "gpt2": _gpt2, "gpt_bigcode": _gpt2, "phi": _phi, "olmo": _olmo1, "granitemoe": _granitemoe, "granitemoehybrid": _granitemoehybrid, "jamba": _jamba, "bitnet": _bitnet, "lfm2_moe": _lfm2, "exaone": _exaone, "telechat3": _telechat3, "deepseek": _deepseek_v1, "recurrent_gemma": _recurrent_gemma, "glm_moe_dsa": _glm_moe_dsa, "deepseek_v32": _glm_moe_dsa, "mistral4": _mistral4, "afmoe": _afmoe, "dbrx": _dbrx, "llama4": _llama4, "llama4_text": _llama4, "qwen3_next": _qwen3_next, "qwen3_5": _qwen3_next, "qwen3_5_text": _qwen3_next, "qwen3_5_moe": _qwen3_next, "qwen3_5_moe_text": _qwen3_next, "falcon_h1": _falcon_h1, "cohere2": _cohere2, "arcee": _arcee, "glm": _glm, "glm4": _glm4, "glm4v": _glm4v, "glm4v_text": _glm4v, "glm4v_moe": _glm4v_moe, "glm4v_moe_text": _glm4v_moe, "cohere2_vision": _cohere2, "paddleocr_vl": _paddleocr_vl, "glm_ocr": _glm_ocr, "glm_ocr_text": _glm_ocr, "paddleocr_vl_text": _paddleocr_vl, "nemotron": _nemotron,
    "ministral3": _ministral3, "granitemoeshared": _granitemoeshared, "nanochat": _nanochat, "code_llama": _plain, "cwm": _plain, "glm4_moe_lite": _deepseek_v3,
    "vaultgemma": _vaultgemma, "solar_open": _solar_open, "minimax_m2": _minimax_m2, "exaone_moe": _exaone_moe, "lfm2": _lfm2, "internlm2": _plain, "baichuan": _baichuan,
}


# ----------------------------------------------------------------------------- presets
def preset(name: str) -> ModelConfig:
    """Architectures named by the benchmark configurations (random-init, synthetic runs)."""
    if name == "tiny-llama":
        return ModelConfig.from_dict(dict(
            model_type="llama", num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, intermediate_size=688, rms_norm_eps=1e-5,
            rope_theta=10000.0, vocab_size=1024, tie_word_embeddings=True,
            max_position_embeddings=2048))
    if name == "llama-3.1-8b":
        return ModelConfig.from_dict(dict(
            model_type="llama", num_hidden_layers=32, hidden_size=4096, num_attention_heads=32,
            num_key_value_heads=8, head_dim=128, intermediate_size=14336, vocab_size=128256,
            rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=131072,
            rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0,
                              high_freq_factor=4.0, original_max_position_embeddings=8192)))
    if name == "qwen3-32b":
        return ModelConfig.from_dict(dict(
            model_type="qwen3", num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
            num_key_value_heads=8, head_dim=128, intermediate_size=25600, vocab_size=151936,
            rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960))
    if name == "gpt-oss-120b":
        return ModelConfig.from_dict(dict(
            model_type="gpt_oss", num_hidden_layers=36, hidden_size=2880, num_attention_heads=64,
            num_key_value_heads=8, head_dim=64, intermediate_size=2880, vocab_size=201088,
            num_local_experts=128, num_experts_per_tok=4, sliding_window=128, rms_norm_eps=1e-5,
            rope_theta=150000.0, max_position_embeddings=131072,
            rope_scaling=dict(rope_type="yarn", factor=32.0, beta_fast=32.0, beta_slow=1.0,
                              original_max_position_embeddings=4096, truncate=False)))
    if name == "tiny-moe":
        return ModelConfig.from_dict(dict(
            model_type="mixtral", num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1024,
            num_local_experts=8, num_experts_per_tok=2, max_position_embeddings=2048))
    if name == "tiny-gpt-oss":
        return ModelConfig.from_dict(dict(
            model_type="gpt_oss", num_hidden_layers=4, hidden_size=256, num_attention_heads=8,
            num_key_value_heads=2, head_dim=64, intermediate_size=256, vocab_size=1024,
            num_local_experts=8, num_experts_per_tok=2, sliding_window=32,
            max_position_embeddings=4096))
    if name == "tiny-qwen3":
        return ModelConfig.from_dict(dict(
            model_type="qwen3", num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
            num_key_value_heads=2, head_dim=64, intermediate_size=512, vocab_size=1024,
            rms_norm_eps=1e-6, max_position_embeddings=2048))
    if name == "tiny-mamba":
        return ModelConfig.from_dict(dict(
            model_type="mamba", num_hidden_layers=2, hidden_size=128, state_size=16, conv_kernel=4, expand=2,
            vocab_size=1024, layer_norm_epsilon=1e-5))
    if name == "tiny-mamba2":
        return ModelConfig.from_dict(dict(
            model_type="mamba2", num_hidden_layers=2, hidden_size=128, num_heads=8, head_dim=32,
            state_size=32, conv_kernel=4, n_groups=1, expand=2, vocab_size=1024, layer_norm_epsilon=1e-5))
    if name == "tiny-nemotron-h":
        return ModelConfig.from_dict(dict(
            model_type="nemotron_h", hidden_size=128, hybrid_override_pattern="M-M*-M-", mamba_num_heads=8,
            mamba_head_dim=32, ssm_state_size=32, conv_kernel=4, n_groups=2, intermediate_size=256,
            num_attention_heads=4, num_key_value_heads=2, head_dim=64, vocab_size=1024, layer_norm_epsilon=1e-5))
    if name == "mamba2-2.7b":
        return ModelConfig.from_dict(dict(
            model_type="mamba2", num_hidden_layers=64, hidden_size=2560, num_heads=80, head_dim=64,
            state_size=128, conv_kernel=4, n_groups=1, expand=2, vocab_size=50288, layer_norm_epsilon=1e-5))
    raise KeyError(name)
