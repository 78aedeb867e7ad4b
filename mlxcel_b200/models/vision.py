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


# ----------------------------------------------------------------------------- InternViT (InternVL)
class InternViTTower:
    """InternVL's vision transformer (transformers `InternVLVisionModel`; the reference's
    src/vision/encoders/internvl.rs): conv patch embedding with bias, class token, learned positions
    (bicubic interpolation off the trained grid), pre-norm blocks whose two branches are scaled per
    channel (``lambda_1`` / ``lambda_2``), LayerNorm or RMSNorm per ``norm_type``, optional RMSNorm of
    q and k over the whole embedding width, a final LayerNorm on the last state. ``tensors`` maps
    names below ``vision_tower.``."""

    def __init__(self, v: dict, tensors: dict, feature_layer: int = -1, drop_cls: bool = True,
                 dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        first = lambda x: int(x[0] if isinstance(x, (list, tuple)) else x)  # noqa: E731
        self.hidden, self.layers, self.heads = int(v["hidden_size"]), int(v["num_hidden_layers"]), int(v["num_attention_heads"])
        self.patch, self.image_size = first(v.get("patch_size", 14)), first(v.get("image_size", 448))
        self.eps = float(v.get("layer_norm_eps", 1e-6))
        self.rms = v.get("norm_type", "layer_norm") == "rms_norm"
        self.act = _ACT_NAMES.get(v.get("hidden_act", "gelu"), "gelu")
        self.feature_layer, self.drop_cls = int(feature_layer), bool(drop_cls)

        def t(name, required=True):
            if name not in tensors:
                if required:
                    raise KeyError(f"vision tower tensor {name!r} is missing")
                return None
            return tensors[name].to(dtype).to(self.device).contiguous()

        pw = t("embeddings.patch_embeddings.projection.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.patch_b = t("embeddings.patch_embeddings.projection.bias")
        self.cls = t("embeddings.cls_token").view(1, 1, -1)
        pos = t("embeddings.position_embeddings", False)
        self.pos = None if pos is None else pos.view(-1, self.hidden)
        self.final_ln = (t("layernorm.weight", False), t("layernorm.bias", False))
        self.blocks = []
        for i in range(self.layers):
            p = f"encoder.layer.{i}."
            a = p + "attention."
            wqkv = torch.cat([t(a + "q_proj.weight"), t(a + "k_proj.weight"), t(a + "v_proj.weight")]).contiguous()
            bq = t(a + "q_proj.bias", False)
            bqkv = None if bq is None else torch.cat([bq, t(a + "k_proj.bias"), t(a + "v_proj.bias")]).contiguous()
            self.blocks.append(dict(
                n1=(t(p + "layernorm_before.weight"), t(p + "layernorm_before.bias", False)),
                n2=(t(p + "layernorm_after.weight"), t(p + "layernorm_after.bias", False)),
                wqkv=wqkv, bqkv=bqkv, qn=t(a + "q_norm.weight", False), kn=t(a + "k_norm.weight", False),
                wo=t(a + "projection_layer.weight"), bo=t(a + "projection_layer.bias", False),
                l1=t(p + "lambda_1"), l2=t(p + "lambda_2"),
                w1=t(p + "mlp.fc1.weight"), b1=t(p + "mlp.fc1.bias"), w2=t(p + "mlp.fc2.weight"), b2=t(p + "mlp.fc2.bias")))

    @property
    def tokens_per_image(self) -> int:
        return (self.image_size // self.patch) ** 2

    def _norm(self, x, wb):
        return ops.rmsnorm(x, wb[0], self.eps) if self.rms else rops.layernorm(x, wb[0], wb[1], self.eps)

    def _positions(self, gh: int, gw: int) -> torch.Tensor:
        g = int(math.isqrt(self.pos.shape[0] - 1))
        if (gh, gw) == (g, g):
            return self.pos
        grid = self.pos[1:].float().reshape(1, g, g, -1).permute(0, 3, 1, 2)
        grid = F.interpolate(grid, size=(gh, gw), mode="bicubic", align_corners=False)
        return torch.cat([self.pos[:1], grid.permute(0, 2, 3, 1).reshape(gh * gw, -1).to(self.pos.dtype)])

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        N, C, H, W = pixels.shape
        p, hid = self.patch, self.hidden
        gh, gw = H // p, W // p
        x = pixels.to(self.device, self.dtype).reshape(N, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5)
        x = F.pad(x.reshape(N * gh * gw, C * p * p), (0, self.k_pad)).contiguous()
        h = ops.linear(x, self.patch_w, bias=self.patch_b).view(N, gh * gw, hid)
        h = torch.cat([self.cls.expand(N, 1, -1), h], dim=1)
        if self.pos is not None:
            h = (h.float() + self._positions(gh, gw).float()).to(self.dtype)
        T = h.shape[1]
        h = h.reshape(N * T, hid).contiguous()
        want = self.feature_layer if self.feature_layer >= 0 else self.layers + 1 + self.feature_layer
        D = hid // self.heads
        for li, b in enumerate(self.blocks):
            if li == want:
                break
            y = self._norm(h, b["n1"])
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"])
            q, k, v = qkv[:, :hid], qkv[:, hid:2 * hid], qkv[:, 2 * hid:]
            if b["qn"] is not None:
                q, k = ops.rmsnorm(q.contiguous(), b["qn"], self.eps), ops.rmsnorm(k.contiguous(), b["kn"], self.eps)
            q, k, v = (z.reshape(N, T, self.heads, D).transpose(1, 2) for z in (q, k, v))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(N * T, hid).contiguous()
            a = ops.linear(a, b["wo"], bias=b["bo"])
            h = (h.float() + b["l1"].float() * a.float()).to(self.dtype)
            y = self._norm(h, b["n2"])
            u = ops.linear(_act(ops.linear(y, b["w1"], bias=b["b1"]), self.act), b["w2"], bias=b["b2"])
            h = (h.float() + b["l2"].float() * u.float()).to(self.dtype)
        if want == self.layers and self.final_ln[0] is not None:
            h = rops.layernorm(h, *self.final_ln, self.eps)
        h = h.view(N, T, hid)
        return h[:, 1:] if self.drop_cls else h


class InternVLConnector:
    """Pixel shuffle by ``downsample_ratio`` (0.5: a 2 x 2 block of patches becomes one token with four
    times the channels), LayerNorm, linear, activation, linear (`InternVLMultiModalProjector`)."""

    def __init__(self, tensors: dict, ratio: float = 0.5, act: str = "gelu", dtype=torch.bfloat16, device="cpu"):
        t = lambda n: tensors[n].to(dtype).to(device).contiguous()  # noqa: E731
        self.s = int(round(1 / ratio))
        self.ln = (t("layer_norm.weight"), t("layer_norm.bias"))
        self.w1, self.b1, self.w2, self.b2 = t("linear_1.weight"), t("linear_1.bias"), t("linear_2.weight"), t("linear_2.bias")
        self.act = _ACT_NAMES.get(act, "gelu")

    def tokens_out(self, tokens_in: int) -> int:
        return tokens_in // (self.s * self.s)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N, T, H = x.shape
        g, s = int(math.isqrt(T)), self.s
        x = x.reshape(N, g, g // s, s * H).permute(0, 2, 1, 3)
        x = x.reshape(N, g // s, g // s, s * s * H).permute(0, 2, 1, 3)
        x = x.reshape(N * (T // (s * s)), s * s * H).contiguous()
        y = rops.layernorm(x, *self.ln, 1e-5)
        u = _act(ops.linear(y, self.w1, bias=self.b1), self.act)
        return ops.linear(u, self.w2, bias=self.b2).view(N, T // (s * s), -1)


class Cohere2VisionConnector:
    """Command A Vision / Aya Vision layout: pixel shuffle by ``downsample_factor``, one biased linear to
    twice the gated width, ``silu(gate) * x`` over its two halves (the gate is the second half), one
    biased linear (`Cohere2VisionMultiModalProjector`)."""

    def __init__(self, tensors: dict, factor: int = 2, dtype=torch.bfloat16, device="cpu"):
        t = lambda n: tensors[n].to(dtype).to(device).contiguous()  # noqa: E731
        self.s = int(factor)
        self.w1, self.b1, self.w2, self.b2 = t("linear_1.weight"), t("linear_1.bias"), t("linear_2.weight"), t("linear_2.bias")

    def tokens_out(self, tokens_in: int) -> int:
        return tokens_in // (self.s * self.s)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        N, T, H = x.shape
        g, s = int(math.isqrt(T)), self.s
        x = x.reshape(N, g, g // s, s * H).permute(0, 2, 1, 3)
        x = x.reshape(N, g // s, g // s, s * s * H).permute(0, 2, 1, 3)
        x = x.reshape(N * (T // (s * s)), s * s * H).contiguous()
        u = ops.linear(x, self.w1, bias=self.b1)
        half = u.shape[1] // 2
        u = (_act(u[:, half:].contiguous(), "silu").float() * u[:, :half].float()).to(x.dtype).contiguous()
        return ops.linear(u, self.w2, bias=self.b2).view(N, T // (s * s), -1)


# ----------------------------------------------------------------------------- Pixtral (Mistral3)
class PixtralTower:
    """Pixtral's vision transformer (transformers `PixtralVisionModel`; the reference's
    src/vision/encoders/pixtral.rs): bias-free conv patch embedding, RMSNorm before the blocks,
    pre-norm blocks with bias-free attention under 2-D rotary positions (half of each head's
    frequency pairs turn with the patch row, half with the column) and a gated SiLU MLP. Images keep
    their own sizes; each is attended on its own. ``tensors`` maps names below ``vision_tower.``."""

    def __init__(self, v: dict, tensors: dict, feature_layer: int = -1, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.hidden, self.layers, self.heads = int(v["hidden_size"]), int(v["num_hidden_layers"]), int(v["num_attention_heads"])
        self.patch, self.image_size = int(v.get("patch_size", 16)), int(v.get("image_size", 1024))
        self.D = int(v.get("head_dim") or self.hidden // self.heads)
        rp = v.get("rope_parameters") or {}
        self.theta = float(rp.get("rope_theta", v.get("rope_theta", 10000.0)))
        self.act = _ACT_NAMES.get(v.get("hidden_act", "silu"), "silu")
        self.feature_layer = int(feature_layer)
        t = lambda n: tensors[n].to(dtype).to(self.device).contiguous()  # noqa: E731
        pw = t("patch_conv.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.ln_pre = t("ln_pre.weight")
        self.blocks = []
        for i in range(self.layers):
            p = f"transformer.layers.{i}."
            a = p + "attention."
            self.blocks.append(dict(
                n1=t(p + "attention_norm.weight"), n2=t(p + "ffn_norm.weight"),
                wqkv=torch.cat([t(a + "q_proj.weight"), t(a + "k_proj.weight"), t(a + "v_proj.weight")]).contiguous(),
                wo=t(a + "o_proj.weight"),
                wgu=torch.cat([t(p + "feed_forward.gate_proj.weight"), t(p + "feed_forward.up_proj.weight")]).contiguous(),
                wd=t(p + "feed_forward.down_proj.weight")))
        f = 1.0 / (self.theta ** (torch.arange(0, self.D, 2, dtype=torch.float32) / self.D))
        self._fh, self._fw = f[0::2].to(self.device), f[1::2].to(self.device)

    def _rot(self, gh: int, gw: int):
        r = torch.arange(gh, device=self.device, dtype=torch.float32)
        c = torch.arange(gw, device=self.device, dtype=torch.float32)
        ang = torch.cat([(r[:, None] * self._fh)[:, None, :].expand(gh, gw, -1),
                         (c[:, None] * self._fw)[None, :, :].expand(gh, gw, -1)], dim=-1).reshape(gh * gw, -1)
        ang = torch.cat([ang, ang], dim=-1)                       # [T, D], rotate-half layout
        return ang.cos(), ang.sin()

    def forward_one(self, pixels: torch.Tensor) -> torch.Tensor:
        """``pixels`` [C, H, W] with H and W multiples of the patch size → [gh * gw, hidden]."""
        C, H, W = pixels.shape
        p, hid, D = self.patch, self.hidden, self.D
        gh, gw = H // p, W // p
        T = gh * gw
        x = pixels.to(self.device, self.dtype).reshape(C, gh, p, gw, p).permute(1, 3, 0, 2, 4).reshape(T, C * p * p)
        h = ops.linear(F.pad(x, (0, self.k_pad)).contiguous(), self.patch_w)
        h = ops.rmsnorm(h, self.ln_pre, 1e-5)
        cos, sin = self._rot(gh, gw)
        want = self.feature_layer if self.feature_layer >= 0 else self.layers + 1 + self.feature_layer
        inter = self.blocks[0]["wd"].shape[1]
        for li, b in enumerate(self.blocks):
            if li == want:
                break
            y = ops.rmsnorm(h, b["n1"], 1e-5)
            qkv = ops.linear(y, b["wqkv"]).view(T, 3, self.heads, D).float()
            q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
            half = lambda z: torch.cat([-z[..., D // 2:], z[..., :D // 2]], dim=-1)  # noqa: E731
            q = q * cos[:, None] + half(q) * sin[:, None]
            k = k * cos[:, None] + half(k) * sin[:, None]
            q, k, v = (z.to(self.dtype).transpose(0, 1).unsqueeze(0) for z in (q, k, v))
            a = F.scaled_dot_product_attention(q, k, v)[0].transpose(0, 1).reshape(T, self.heads * D).contiguous()
            h = ops.linear(a, b["wo"], residual=h)
            y = ops.rmsnorm(h, b["n2"], 1e-5)
            gu = ops.linear(y, b["wgu"])
            u = (_act(gu[:, :inter].contiguous(), self.act).float() * gu[:, inter:].float()).to(self.dtype)
            h = ops.linear(u, b["wd"], residual=h)
        return h


class Mistral3Connector:
    """RMSNorm, merge of every ``s x s`` block of patches through one bias-free linear (the block's
    channels are laid out channel-major, the order of `torch.nn.functional.unfold`), then linear,
    activation, linear (`Mistral3MultiModalProjector`)."""

    def __init__(self, tensors: dict, merge: int, eps: float, act: str = "gelu", dtype=torch.bfloat16, device="cpu"):
        t = lambda n: tensors[n].to(dtype).to(device).contiguous() if n in tensors else None  # noqa: E731
        self.s, self.eps = int(merge), float(eps)
        self.norm, self.wm = t("norm.weight"), t("patch_merger.merging_layer.weight")
        self.w1, self.b1, self.w2, self.b2 = t("linear_1.weight"), t("linear_1.bias"), t("linear_2.weight"), t("linear_2.bias")
        self.act = _ACT_NAMES.get(act, "gelu")

    def forward_one(self, x: torch.Tensor, gh: int, gw: int) -> torch.Tensor:
        """[gh * gw, hidden] → [(gh / s) * (gw / s), text_hidden]."""
        s, H = self.s, x.shape[1]
        y = ops.rmsnorm(x.contiguous(), self.norm, self.eps)
        y = y.view(gh // s, s, gw // s, s, H).permute(0, 2, 4, 1, 3).reshape((gh // s) * (gw // s), H * s * s).contiguous()
        y = ops.linear(y, self.wm)
        u = _act(ops.linear(y, self.w1, bias=self.b1), self.act)
        return ops.linear(u, self.w2, bias=self.b2)
