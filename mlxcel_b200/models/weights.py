"""Weight containers of the decoder executor.

``LayerWeights`` holds one transformer block in the fused layout the kernels want
(qkv rows concatenated, gate rows followed by up rows); ``ModelWeights`` the whole model.
Tensors are either bf16 ``torch.Tensor`` or :class:`QuantizedTensor` (MLX affine / mxfp4 /
mxfp8 packed data kept as stored in the checkpoint).
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..config import ModelConfig


@dataclass
class QuantizedTensor:
    """MLX quantized matrix ``[out, in]`` (or stacked ``[E, out, in]``) as stored on disk
    (src/lib/mlxcel-core/src/layers.rs:2322-2522): ``packed`` uint32 ``[.., out, in*bits/32]``,
    ``scales`` ``[.., out, in/group]`` (bf16 for affine, uint8 e8m0 for mxfp4/mxfp8),
    ``biases`` (affine only)."""

    packed: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor | None
    bits: int
    group_size: int
    mode: str  # affine | mxfp4 | mxfp8

    @property
    def shape(self):
        *lead, out, pk = self.packed.shape
        return (*lead, out, pk * 32 // self.bits)

    def to(self, device):
        return QuantizedTensor(self.packed.to(device), self.scales.to(device),
                               None if self.biases is None else self.biases.to(device),
                               self.bits, self.group_size, self.mode)

    def nbytes(self) -> int:
        n = self.packed.numel() * 4 + self.scales.numel() * self.scales.element_size()
        if self.biases is not None:
            n += self.biases.numel() * self.biases.element_size()
        return n


Weight = "torch.Tensor | QuantizedTensor"


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    wqkv: object
    wo: object
    bqkv: torch.Tensor | None = None
    bo: torch.Tensor | None = None
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    sinks: torch.Tensor | None = None            # fp32 [Hq_local]
    post_attn_norm: torch.Tensor | None = None   # Gemma2/3
    post_mlp_norm: torch.Tensor | None = None
    ln1_b: torch.Tensor | None = None            # LayerNorm families: norm biases
    ln2_b: torch.Tensor | None = None
    mla: dict | None = None                      # multi-head latent attention projections (DeepSeek)
    act_params: tuple | None = None              # xIELU: (alpha_p, alpha_n, beta, eps) of this layer
    attn_gate: object | None = None              # AFMoE: sigmoid gate on the attention output, [Hq * D, H]
    attn_sub_norm: torch.Tensor | None = None    # BitNet: RMSNorm of the attention output before o_proj
    ffn_sub_norm: torch.Tensor | None = None     # BitNet: RMSNorm of act(gate) * up before down_proj
    # dense MLP
    w_gate_up: object | None = None
    w_down: object | None = None
    b_gate_up: torch.Tensor | None = None
    b_down: torch.Tensor | None = None
    # MoE
    router_w: torch.Tensor | None = None         # [E, H] bf16
    router_b: torch.Tensor | None = None
    experts_gate_up: object | None = None        # [E_local, 2I, H]
    experts_down: object | None = None           # [E_local, H, I]
    experts_gate_up_b: torch.Tensor | None = None
    experts_down_b: torch.Tensor | None = None
    shared_gate_up: object | None = None
    shared_down: object | None = None
    shared_gate: torch.Tensor | None = None      # qwen2-moe shared-expert gate [1, H]


@dataclass
class ModelWeights:
    embed: torch.Tensor
    layers: list[LayerWeights]
    final_norm: torch.Tensor
    lm_head: object
    extra: dict = field(default_factory=dict)

    def nbytes(self) -> int:
        total = 0

        def add(x):
            nonlocal total
            if isinstance(x, torch.Tensor):
                total += x.numel() * x.element_size()
            elif isinstance(x, QuantizedTensor):
                total += x.nbytes()

        add(self.embed)
        add(self.final_norm)
        if self.lm_head is not self.embed:
            add(self.lm_head)
        for l in self.layers:
            for v in vars(l).values():
                add(v)
        return total


def _randn(shape, std, gen, dtype, device):
    # Generated on the target device in bf16-sized pieces to keep peak memory low.
    t = torch.empty(shape, dtype=dtype, device=device)
    t.normal_(0.0, std, generator=gen)
    return t


def random_weights(cfg: ModelConfig, *, seed: int = 0, dtype=torch.bfloat16, device="cpu",
                   tp_rank: int = 0, tp_size: int = 1, ep_rank: int = 0, ep_size: int = 1,
                   layers: range | None = None, std: float = 0.02,
                   vocab_parallel: bool = False, layer_hook=None) -> ModelWeights:
    """Random-init N(0, std) weights of the architecture, already sharded for (tp, ep, pp).

    Every rank draws from its own generator stream (seed, rank) directly at shard shape: the
    synthetic benchmarks need the architecture's shapes and byte counts, not rank-consistent values.
    Use :func:`mlxcel_b200.loading.shard.shard_weights` on a full model when values must agree
    across ranks (parity tests do)."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)   # sharded tensors: one stream per rank
    gen.manual_seed(seed * 1000003 + tp_rank * 101 + ep_rank + 1)
    shared = torch.Generator(device=dev)  # replicated tensors: the same stream on every rank
    shared.manual_seed(seed * 1000003)
    H, D = cfg.hidden_size, cfg.head_dim
    Hq, Hkv = cfg.num_attention_heads // tp_size, max(1, cfg.num_key_value_heads // tp_size)
    I = cfg.intermediate_size // tp_size
    V = cfg.vocab_size
    ones = lambda n: torch.ones(n, dtype=dtype, device=dev) - cfg.norm_weight_bias  # noqa: E731
    Vl = V // tp_size if vocab_parallel else V
    # The embedding table stays replicated (a gather needs no collective); only the LM head is
    # vocab-parallel.
    embed = _randn((V, H), std, shared, dtype, dev)
    lws = []
    for li in (layers if layers is not None else range(cfg.num_hidden_layers)):
        if cfg.extra.get("mla"):
            if tp_size != 1:
                raise NotImplementedError("tensor-parallel multi-head latent attention")
            m = cfg.extra["mla"]
            qk = m["nope"] + m["rope"]
            mla = dict(kv_a=_randn((m["kv_lora_rank"] + m["rope"], H), std, gen, dtype, dev),
                       kv_a_norm=torch.ones(m["kv_lora_rank"], dtype=dtype, device=dev),
                       kv_b=_randn((Hq * (m["nope"] + m["v"]), m["kv_lora_rank"]), std, gen, dtype, dev))
            if m.get("q_lora_rank"):
                mla.update(q_a=_randn((m["q_lora_rank"], H), std, gen, dtype, dev),
                           q_a_norm=torch.ones(m["q_lora_rank"], dtype=dtype, device=dev),
                           q_b=_randn((Hq * qk, m["q_lora_rank"]), std, gen, dtype, dev))
            else:
                mla["q"] = _randn((Hq * qk, H), std, gen, dtype, dev)
            lw = LayerWeights(ln1=ones(H), ln2=ones(H), wqkv=None, wo=_randn((H, Hq * m["v"]), std, gen, dtype, dev),
                              mla=mla)
        else:
            lw = LayerWeights(ln1=ones(H), ln2=ones(H),
                              wqkv=_randn(((Hq + 2 * Hkv) * D, H), std, gen, dtype, dev),
                              wo=_randn((H, Hq * D), std, gen, dtype, dev))
        if cfg.attention_bias and lw.mla is None:
            lw.bqkv = _randn(((Hq + 2 * Hkv) * D,), std, gen, dtype, dev)
            if cfg.model_type == "gpt_oss":
                lw.bo = _randn((H,), std, shared, dtype, dev)
        if cfg.qk_norm:
            full = cfg.extra.get("qk_norm_full")              # OLMo-2 / OLMoE: one norm over the projection
            lw.q_norm, lw.k_norm = (ones(Hq * D), ones(Hkv * D)) if full else (ones(D), ones(D))
        if cfg.extra.get("norm") == "layernorm" and not cfg.extra.get("norm_no_params") \
                and cfg.model_type not in ("cohere", "cohere2"):
            lw.ln1_b, lw.ln2_b = _randn((H,), std, shared, dtype, dev), _randn((H,), std, shared, dtype, dev)
        if cfg.extra.get("post_norm_only"):
            lw.post_attn_norm, lw.post_mlp_norm = ones(H), ones(H)
        if cfg.attention_sinks:
            lw.sinks = torch.randn(Hq, generator=gen, device=dev, dtype=torch.float32)
        if cfg.post_norms:
            lw.post_attn_norm, lw.post_mlp_norm = ones(H), ones(H)
        if cfg.is_moe and li >= cfg.extra.get("first_k_dense", 0):
            E = cfg.num_experts
            El = E // ep_size
            mi = cfg.moe_intermediate_size // tp_size
            lw.router_w = _randn((E, H), std, shared, dtype, dev)
            if cfg.router_bias:
                lw.router_b = _randn((E,), std, shared, dtype, dev)
                if cfg.moe_route_mode == "sigmoid_group":          # selection bias, kept in fp32
                    lw.router_b = lw.router_b.float() * 5
            lw.experts_gate_up = _randn((El, 2 * mi, H), std, gen, dtype, dev)
            lw.experts_down = _randn((El, H, mi), std, gen, dtype, dev)
            if cfg.expert_bias:
                lw.experts_gate_up_b = _randn((El, 2 * mi), std, gen, dtype, dev)
                lw.experts_down_b = _randn((El, H), std, gen, dtype, dev)
                if tp_size > 1 and ep_size == 1:
                    lw.experts_down_b = _randn((El, H), std, shared, dtype, dev)
            if cfg.shared_expert_intermediate_size:
                si = cfg.shared_expert_intermediate_size // tp_size
                lw.shared_gate_up = _randn((2 * si, H), std, gen, dtype, dev)
                lw.shared_down = _randn((H, si), std, gen, dtype, dev)
                if cfg.moe_route_mode != "sigmoid_group":          # Qwen2-MoE gates its shared expert
                    lw.shared_gate = _randn((1, H), std, shared, dtype, dev)
        else:
            rows = I if cfg.extra.get("mlp") == "plain" else 2 * I     # plain MLP: fc only, no gate
            lw.w_gate_up = _randn((rows, H), std, gen, dtype, dev)
            lw.w_down = _randn((H, I), std, gen, dtype, dev)
            if cfg.mlp_bias:
                lw.b_gate_up = _randn((rows,), std, gen, dtype, dev)
                lw.b_down = _randn((H,), std, shared, dtype, dev)
            if cfg.hidden_act == "xielu":
                lw.act_params = (0.8, 0.8, 0.5, -1e-6)
        if layer_hook is not None:
            layer_hook(lw)        # e.g. quantize this layer before the next one is drawn (peak memory)
        lws.append(lw)
    if cfg.tie_word_embeddings:
        lm_head = embed[tp_rank * Vl:(tp_rank + 1) * Vl] if vocab_parallel else embed
    else:
        lm_head = _randn((Vl, H), std, gen, dtype, dev)
    return ModelWeights(embed=embed, layers=lws, final_norm=ones(H), lm_head=lm_head)
