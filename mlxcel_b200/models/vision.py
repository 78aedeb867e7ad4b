"""Vision towers and connectors for vision-language checkpoints.

A vision-language model here is three parts: a **tower** that turns pixels into patch states, a
**connector** that maps those states into the language model's embedding space, and the ordinary
decoder, which receives the connector's rows in place of the embeddings of the image placeholder
tokens (``StepBatch.embeds``). The reference keeps one encoder file per family under src/vision/
(encoders, connectors) and glues them in src/multimodal/; here one parametrised ViT covers the
CLIP and SigLIP layouts and `Qwen2VisionTower` the Qwen2-VL / Qwen2.5-VL layout (2-D rotary
positions, patch merger).

Towers:
  * CLIP (`clip_vision_model`): conv patch embedding without bias, class token, learned positions,
    pre-LayerNorm, pre-norm blocks with quick-GELU. LLaVA takes the states of layer -2 and drops the
    class token (`vision_feature_layer`, `vision_feature_select_strategy`).
  * SigLIP (`siglip_vision_model`): conv patch embedding with bias, no class token, tanh-GELU,
    post-LayerNorm after the last block.

Connectors: `llava` (linear, GELU, linear), `pixel_shuffle` (Idefics3 / SmolVLM: fold s x s
neighbouring patches into the channel dimension, then one linear), `gemma3` (average pool to a
fixed token grid, RMSNorm, linear).

Projections run through ``ops.linear`` (the tcgen05 GEMM on a GPU); the attention of a tower is one
non-causal softmax(QK^T)V per image through PyTorch's ``scaled_dot_product_attention``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import recurrent as rops


def _act(x: torch.Tensor, kind: str) -> torch.Tensor:
    if kind == "quick_gelu":
        v = x.float()
        return (v * torch.sigmoid(1.702 * v)).to(x.dtype)
    return rops.activation(x, kind)


_ACT_NAMES = {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh",
              "quick_gelu": "quick_gelu", "silu": "silu"}


@dataclass
class VisionConfig:
    kind: str = "clip"                 # clip | siglip
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    intermediate: int = 4096
    patch: int = 14
    image_size: int = 336
    eps: float = 1e-5
    act: str = "quick_gelu"
    channels: int = 3
    feature_layer: int = -1            # which hidden state feeds the connector (-1 = last, LLaVA: -2)
    drop_cls: bool = True
    extra: dict = field(default_factory=dict)

    @staticmethod
    def from_dict(v: dict, wrapper: dict | None = None) -> "VisionConfig":
        wrapper = wrapper or {}
        mt = v.get("model_type", "clip_vision_model")
        kind = "siglip" if any(t in mt for t in ("siglip", "idefics3", "smolvlm")) else "clip"
        c = VisionConfig(kind=kind, hidden=int(v.get("hidden_size", 768)), layers=int(v.get("num_hidden_layers", 12)),
                         heads=int(v.get("num_attention_heads", 12)), intermediate=int(v.get("intermediate_size", 3072)),
                         patch=int(v.get("patch_size", 14)), image_size=int(v.get("image_size", 224)),
                         eps=float(v.get("layer_norm_eps", 1e-5 if kind == "clip" else 1e-6)),
                         act=_ACT_NAMES.get(v.get("hidden_act", "quick_gelu" if kind == "clip" else "gelu_pytorch_tanh"), "gelu"),
                         channels=int(v.get("num_channels", 3)))
        fl = wrapper.get("vision_feature_layer", -1)
        c.feature_layer = int(fl if not isinstance(fl, list) else fl[-1])
        c.drop_cls = wrapper.get("vision_feature_select_strategy", "default") == "default"
        return c

    @property
    def grid(self) -> int:
        return self.image_size // self.patch


class ViTTower:
    """CLIP / SigLIP vision transformer. ``tensors`` maps names below the tower's prefix
    (``embeddings.patch_embedding.weight`` ...) to tensors."""

    def __init__(self, cfg: VisionConfig, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.cfg, self.dtype, self.device = cfg, dtype, torch.device(device)

        def t(name, required=True):
            if name not in tensors:
                if required:
                    raise KeyError(f"vision tower tensor {name!r} is missing")
                return None
            return tensors[name].to(dtype).to(self.device).contiguous()

        e = "embeddings."
        pw = t(e + "patch_embedding.weight")                     # [hidden, C, p, p]
        pw = pw.reshape(pw.shape[0], -1)                          # one GEMM over unfolded patches
        self.k_pad = (-pw.shape[1]) % 8                           # the GEMM's TMA rows need 16-byte strides
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.patch_b = t(e + "patch_embedding.bias", False)
        self.cls = t(e + "class_embedding", False)
        self.pos = t(e + "position_embedding.weight")
        pre = "pre_layrnorm" if "pre_layrnorm.weight" in tensors else "pre_layernorm"
        self.pre_ln = (t(pre + ".weight", False), t(pre + ".bias", False))
        self.post_ln = (t("post_layernorm.weight", False), t("post_layernorm.bias", False))
        self.blocks = []
        for i in range(cfg.layers):
            p = f"encoder.layers.{i}."
            a = p + "self_attn."
            wqkv = torch.cat([t(a + "q_proj.weight"), t(a + "k_proj.weight"), t(a + "v_proj.weight")]).contiguous()
            bqkv = torch.cat([t(a + "q_proj.bias"), t(a + "k_proj.bias"), t(a + "v_proj.bias")]).contiguous()
            self.blocks.append(dict(
                ln1=(t(p + "layer_norm1.weight"), t(p + "layer_norm1.bias")), wqkv=wqkv, bqkv=bqkv,
                wo=t(a + "out_proj.weight"), bo=t(a + "out_proj.bias"),
                ln2=(t(p + "layer_norm2.weight"), t(p + "layer_norm2.bias")),
                w1=t(p + "mlp.fc1.weight"), b1=t(p + "mlp.fc1.bias"), w2=t(p + "mlp.fc2.weight"), b2=t(p + "mlp.fc2.bias")))

    @property
    def tokens_per_image(self) -> int:
        return self.cfg.grid ** 2

    def _positions(self, gh: int, gw: int) -> torch.Tensor:
        """Learned position table for a gh x gw patch grid (bicubic interpolation of the square table
        when the grid differs from the one trained on)."""
        g = self.cfg.grid
        n_cls = 0 if self.cls is None else 1
        if (gh, gw) == (g, g):
            return self.pos
        grid = self.pos[n_cls:].float().reshape(1, g, g, -1).permute(0, 3, 1, 2)
        grid = F.interpolate(grid, size=(gh, gw), mode="bicubic", align_corners=False)
        grid = grid.permute(0, 2, 3, 1).reshape(gh * gw, -1).to(self.pos.dtype)
        return torch.cat([self.pos[:n_cls], grid]) if n_cls else grid

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels`` [N, C, H, W] (already normalised). Returns the selected hidden state
        [N, tokens, hidden] without the class token when the wrapper drops it."""
        c = self.cfg
        N, C, H, W = pixels.shape
        p = c.patch
        gh, gw = H // p, W // p
        x = pixels.to(self.device, self.dtype)
        # unfold into [N * gh * gw, C * p * p] rows in the conv weight's (C, p, p) order
        x = x.reshape(N, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5).reshape(N * gh * gw, C * p * p)
        x = F.pad(x, (0, self.k_pad)).contiguous()
        h = ops.linear(x, self.patch_w, bias=self.patch_b).view(N, gh * gw, c.hidden)
        if self.cls is not None:
            h = torch.cat([self.cls.view(1, 1, -1).expand(N, 1, -1), h], dim=1)
        h = (h.float() + self._positions(gh, gw).float()).to(self.dtype)
        T = h.shape[1]
        h = h.reshape(N * T, c.hidden).contiguous()
        if self.pre_ln[0] is not None:
            h = rops.layernorm(h, *self.pre_ln, c.eps)
        want = c.feature_layer if c.feature_layer >= 0 else c.layers + 1 + c.feature_layer   # index into hidden_states
        D = c.hidden // c.heads
        for li, b in enumerate(self.blocks):
            if li == want:
                break
            y = rops.layernorm(h, *b["ln1"], c.eps)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(N, T, 3, c.heads, D)
            q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(N * T, c.hidden).contiguous()
            h = ops.linear(a, b["wo"], bias=b["bo"], residual=h)
            y = rops.layernorm(h, *b["ln2"], c.eps)
            u = _act(ops.linear(y, b["w1"], bias=b["b1"]), c.act)
            h = ops.linear(u, b["w2"], bias=b["b2"], residual=h)
        if want == c.layers and self.post_ln[0] is not None and c.kind == "siglip":
            h = rops.layernorm(h, *self.post_ln, c.eps)
        h = h.view(N, T, c.hidden)
        if self.cls is not None and c.drop_cls:
            h = h[:, 1:]
        return h


# ----------------------------------------------------------------------------- connectors
class LlavaConnector:
    """``linear_2(gelu(linear_1(x)))`` (LLaVA-1.5 `multi_modal_projector`)."""

    def __init__(self, tensors: dict, act: str = "gelu", dtype=torch.bfloat16, device="cpu"):
        t = lambda n: tensors[n].to(dtype).to(device).contiguous() if n in tensors else None  # noqa: E731
        self.w1, self.b1, self.w2, self.b2 = t("linear_1.weight"), t("linear_1.bias"), t("linear_2.weight"), t("linear_2.bias")
        self.act = _ACT_NAMES.get(act, "gelu")

    def tokens_out(self, tokens_in: int) -> int:
        return tokens_in

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N, T, H = x.shape
        u = _act(ops.linear(x.reshape(N * T, H).contiguous(), self.w1, bias=self.b1), self.act)
        return ops.linear(u, self.w2, bias=self.b2).view(N, T, -1)


class PixelShuffleConnector:
    """Idefics3 / SmolVLM: an s x s block of neighbouring patches becomes one token with s*s*hidden
    channels, then one bias-free linear (`connector.modality_projection.proj`)."""

    def __init__(self, tensors: dict, scale: int, dtype=torch.bfloat16, device="cpu"):
        self.s = int(scale)
        self.w = tensors["modality_projection.proj.weight"].to(dtype).to(device).contiguous()

    def tokens_out(self, tokens_in: int) -> int:
        return tokens_in // (self.s * self.s)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N, T, H = x.shape
        g, s = int(math.isqrt(T)), self.s
        x = x.view(N, g, g // s, s * H).permute(0, 2, 1, 3)                    # [N, g/s (w), g (h), s*H]
        x = x.reshape(N, g // s, g // s, s * s * H).permute(0, 2, 1, 3)        # [N, g/s (h), g/s (w), s*s*H]
        x = x.reshape(N * (T // (s * s)), s * s * H).contiguous()
        return ops.linear(x, self.w).view(N, T // (s * s), -1)


class Gemma3Connector:
    """Average-pool the patch grid to ``mm_tokens_per_image`` tokens, Gemma RMSNorm (gain 1 + w), then
    the input projection matrix (stored [vision_hidden, text_hidden])."""

    def __init__(self, tensors: dict, tokens_per_image: int, eps: float, dtype=torch.bfloat16, device="cpu"):
        self.out_grid = int(math.isqrt(tokens_per_image))
        self.norm = tensors["mm_soft_emb_norm.weight"].to(dtype).to(device).contiguous()
        self.w = tensors["mm_input_projection_weight"].to(dtype).to(device).t().contiguous()     # -> [text, vision]
        self.eps = eps

    def tokens_out(self, tokens_in: int) -> int:
        return self.out_grid ** 2

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N, T, H = x.shape
        g = int(math.isqrt(T))
        k = g // self.out_grid
        y = F.avg_pool2d(x.float().transpose(1, 2).reshape(N, H, g, g), k, k).flatten(2).transpose(1, 2)
        y = y.reshape(N * self.out_grid ** 2, H).to(x.dtype).contiguous()
        y = ops.rmsnorm(y, self.norm, self.eps, 1.0)
        return ops.linear(y, self.w).view(N, self.out_grid ** 2, -1)
