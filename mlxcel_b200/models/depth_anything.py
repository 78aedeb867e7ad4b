"""Dense prediction: DINOv2 backbone and the Depth Anything depth estimator built on it.

The reference keeps a DINOv2 encoder (src/vision/encoders/dinov2*.rs) and dense-prediction models
on ViT backbones (src/vision/dense/: depth, segmentation). Here `Dinov2Backbone` is the plain
transformer (class token, learned positions interpolated bicubically to the image's patch grid,
pre-norm blocks with per-channel layer scale, MLP or SwiGLU feed-forward; its linears run through
``ops.linear``, the tcgen05 GEMM on a GPU) returning the hidden states of chosen depths, and
`DepthAnything` is the DPT-style decoder on four of them: per-level 1x1 projection and resize
(transposed / strided convolution), 3x3 convolution to the fusion width, top-down fusion with
pre-activation residual units and bilinear upsampling, and a three-convolution head that ends in
ReLU (relative depth) or sigmoid x max_depth (metric). The convolutions are library calls
(``torch.nn.functional.conv2d``): they are a small part of the work next to the backbone.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..ops import recurrent as rops


class Dinov2Backbone:
    def __init__(self, cfg: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.hidden, self.layers, self.heads = int(cfg["hidden_size"]), int(cfg["num_hidden_layers"]), int(cfg["num_attention_heads"])
        self.patch, self.eps = int(cfg.get("patch_size", 14)), float(cfg.get("layer_norm_eps", 1e-6))
        self.swiglu = bool(cfg.get("use_swiglu_ffn", False))
        self.apply_ln = bool(cfg.get("apply_layernorm", True))
        names = ["stem"] + [f"stage{i}" for i in range(1, self.layers + 1)]
        want = cfg.get("out_features") or ([names[i] for i in cfg["out_indices"]] if cfg.get("out_indices") else [names[-1]])
        self.out_stages = [names.index(n) for n in want]

        def t(n):
            return tensors[n].to(dtype).to(self.device).contiguous()

        pw = t("embeddings.patch_embeddings.projection.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.patch_b = t("embeddings.patch_embeddings.projection.bias")
        self.cls = t("embeddings.cls_token").view(1, 1, -1)
        self.pos = t("embeddings.position_embeddings").view(-1, self.hidden)
        self.final_ln = (t("layernorm.weight"), t("layernorm.bias"))
        self.blocks = []
        for i in range(self.layers):
            p = f"encoder.layer.{i}."
            a = p + "attention.attention."
            b = dict(n1=(t(p + "norm1.weight"), t(p + "norm1.bias")), n2=(t(p + "norm2.weight"), t(p + "norm2.bias")),
                     wqkv=torch.cat([t(a + "query.weight"), t(a + "key.weight"), t(a + "value.weight")]).contiguous(),
                     bqkv=torch.cat([t(a + "query.bias"), t(a + "key.bias"), t(a + "value.bias")]).contiguous(),
                     wo=t(p + "attention.output.dense.weight"), bo=t(p + "attention.output.dense.bias"),
                     l1=t(p + "layer_scale1.lambda1"), l2=t(p + "layer_scale2.lambda1"))
            if self.swiglu:
                b.update(w1=t(p + "mlp.weights_in.weight"), b1=t(p + "mlp.weights_in.bias"),
                         w2=t(p + "mlp.weights_out.weight"), b2=t(p + "mlp.weights_out.bias"))
            else:
                b.update(w1=t(p + "mlp.fc1.weight"), b1=t(p + "mlp.fc1.bias"), w2=t(p + "mlp.fc2.weight"), b2=t(p + "mlp.fc2.bias"))
            self.blocks.append(b)

    def _positions(self, gh: int, gw: int) -> torch.Tensor:
        g = int(math.isqrt(self.pos.shape[0] - 1))
        if (gh, gw) == (g, g):
            return self.pos.float()
        grid = self.pos[1:].float().reshape(1, g, g, -1).permute(0, 3, 1, 2)
        grid = F.interpolate(grid, size=(gh, gw), mode="bicubic", align_corners=False)
        return torch.cat([self.pos[:1].float(), grid.permute(0, 2, 3, 1).reshape(gh * gw, -1)])

    @torch.no_grad()
    def forward(self, pixels: torch.Tensor) -> list[torch.Tensor]:
        """[N, 3, H, W] (H, W multiples of the patch size) → the chosen stages' states [N, 1 + gh * gw, hidden]
        (with the final LayerNorm when the checkpoint applies it to its features)."""
        N, C, H, W = pixels.shape
        p, hid = self.patch, self.hidden
        gh, gw = H // p, W // p
        x = pixels.to(self.device, self.dtype).reshape(N, C, gh, p, gw, p).permute(0, 2, 4, 1, 3, 5)
        x = F.pad(x.reshape(N * gh * gw, C * p * p), (0, self.k_pad)).contiguous()
        h = ops.linear(x, self.patch_w, bias=self.patch_b).view(N, gh * gw, hid)
        h = torch.cat([self.cls.expand(N, 1, -1), h], dim=1)
        h = (h.float() + self._positions(gh, gw)).to(self.dtype)
        T, D = h.shape[1], hid // self.heads
        h = h.reshape(N * T, hid).contiguous()
        outs = []

        def emit(stage):
            if stage in self.out_stages:
                y = rops.layernorm(h, *self.final_ln, self.eps) if self.apply_ln else h
                outs.append(y.view(N, T, hid))
        emit(0)
        for li, b in enumerate(self.blocks):
            y = rops.layernorm(h, *b["n1"], self.eps)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(N, T, 3, self.heads, D)
            q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
            a = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(N * T, hid).contiguous()
            a = ops.linear(a, b["wo"], bias=b["bo"])
            h = (h.float() + b["l1"].float() * a.float()).to(self.dtype)
            y = rops.layernorm(h, *b["n2"], self.eps)
            u = ops.linear(y, b["w1"], bias=b["b1"])
            if self.swiglu:
                half = u.shape[1] // 2
                u = (rops.activation(u[:, :half].contiguous(), "silu").float() * u[:, half:].float()).to(self.dtype).contiguous()
            else:
                u = rops.activation(u, "gelu")
            u = ops.linear(u, b["w2"], bias=b["b2"])
            h = (h.float() + b["l2"].float() * u.float()).to(self.dtype)
            emit(li + 1)
        return outs

    def embed(self, pixels: torch.Tensor) -> torch.Tensor:
        """Image embedding: the class token of the last stage after the final LayerNorm, [N, hidden]."""
        keep, keep_ln = self.out_stages, self.apply_ln
        self.out_stages, self.apply_ln = [self.layers], True
        try:
            return self.forward(pixels)[0][:, 0]
        finally:
            self.out_stages, self.apply_ln = keep, keep_ln


class DepthAnything:
    def __init__(self, raw: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        bc = dict(raw["backbone_config"])
        self.backbone = Dinov2Backbone(bc, {k[len("backbone."):]: v for k, v in tensors.items() if k.startswith("backbone.")},
                                       dtype, device)
        self.patch = int(raw.get("patch_size", bc.get("patch_size", 14)))
        self.factors = [float(f) for f in raw.get("reassemble_factors", [4, 2, 1, 0.5])]
        self.head_in = int(raw.get("head_in_index", -1))
        self.metric = raw.get("depth_estimation_type", "relative") == "metric"
        self.max_depth = float(raw.get("max_depth") or 1.0)
        t = lambda n: tensors[n].to(dtype).to(self.device).contiguous() if n in tensors else None  # noqa: E731
        n = len(self.factors)
        self.reassemble = [dict(pw=t(f"neck.reassemble_stage.layers.{i}.projection.weight"), pb=t(f"neck.reassemble_stage.layers.{i}.projection.bias"),
                                rw=t(f"neck.reassemble_stage.layers.{i}.resize.weight"), rb=t(f"neck.reassemble_stage.layers.{i}.resize.bias"))
                           for i in range(n)]
        self.convs = [t(f"neck.convs.{i}.weight") for i in range(n)]

        def unit(p):
            return dict(w1=t(p + "convolution1.weight"), b1=t(p + "convolution1.bias"), w2=t(p + "convolution2.weight"), b2=t(p + "convolution2.bias"))
        self.fusion = [dict(pw=t(f"neck.fusion_stage.layers.{i}.projection.weight"), pb=t(f"neck.fusion_stage.layers.{i}.projection.bias"),
                            r1=unit(f"neck.fusion_stage.layers.{i}.residual_layer1."), r2=unit(f"neck.fusion_stage.layers.{i}.residual_layer2."))
                       for i in range(n)]
        self.head = {k: t(f"head.{k}") for k in ("conv1.weight", "conv1.bias", "conv2.weight", "conv2.bias", "conv3.weight", "conv3.bias")}

    @staticmethod
    def from_pretrained(path: str | Path, dtype=torch.bfloat16, device="cpu") -> "DepthAnything":
        from ..loading.checkpoint import TensorSource
        path = Path(path)
        raw = json.loads((path / "config.json").read_text())
        if raw.get("model_type") != "depth_anything":
            raise ValueError(f"not a depth_anything checkpoint: model_type {raw.get('model_type')!r}")
        src = TensorSource(path)
        m = DepthAnything(raw, {k: src.get(k) for k in src.keys()}, dtype, device)
        f = path / "preprocessor_config.json"
        m.pre = json.loads(f.read_text()) if f.exists() else {}
        return m

    @staticmethod
    def _unit(x, u):
        y = F.conv2d(F.relu(x), u["w1"], u["b1"], padding=1)
        return x + F.conv2d(F.relu(y), u["w2"], u["b2"], padding=1)

    @torch.no_grad()
    def predict(self, pixels: torch.Tensor) -> torch.Tensor:
        """[N, 3, H, W] normalised pixels → depth [N, H, W] (fp32)."""
        N, _, H, W = pixels.shape
        gh, gw = H // self.patch, W // self.patch
        feats = []
        for hs, ra, factor, cw in zip(self.backbone.forward(pixels), self.reassemble, self.factors, self.convs):
            x = hs[:, 1:].reshape(N, gh, gw, -1).permute(0, 3, 1, 2).contiguous()
            x = F.conv2d(x, ra["pw"], ra["pb"])
            if factor > 1:
                x = F.conv_transpose2d(x, ra["rw"], ra["rb"], stride=int(factor))
            elif factor < 1:
                x = F.conv2d(x, ra["rw"], ra["rb"], stride=int(round(1 / factor)), padding=1)
            feats.append(F.conv2d(x, cw, None, padding=1))
        feats = feats[::-1]
        fused, out = None, []
        for i, (x, fl) in enumerate(zip(feats, self.fusion)):
            size = feats[i + 1].shape[2:] if i != len(feats) - 1 else None
            if fused is None:
                y = x
            else:
                r = x if x.shape == fused.shape else F.interpolate(x, size=fused.shape[2:], mode="bilinear", align_corners=False)
                y = fused + self._unit(r, fl["r1"])
            y = self._unit(y, fl["r2"])
            y = F.interpolate(y, size=tuple(size), mode="bilinear", align_corners=True) if size is not None else \
                F.interpolate(y, scale_factor=2, mode="bilinear", align_corners=True)
            fused = F.conv2d(y, fl["pw"], fl["pb"])
            out.append(fused)
        h = self.head
        d = F.conv2d(out[self.head_in], h["conv1.weight"], h["conv1.bias"], padding=1)
        d = F.interpolate(d, (gh * self.patch, gw * self.patch), mode="bilinear", align_corners=True)
        d = F.relu(F.conv2d(d, h["conv2.weight"], h["conv2.bias"], padding=1))
        d = F.conv2d(d, h["conv3.weight"], h["conv3.bias"])
        d = (torch.sigmoid(d.float()) if self.metric else F.relu(d.float())) * self.max_depth
        return d[:, 0]

    def estimate(self, image, short_side: int = 518) -> np.ndarray:
        """A PIL image → depth map at the image's own size (float32 [H, W])."""
        from PIL import Image
        pre = getattr(self, "pre", {})
        mean = np.asarray(pre.get("image_mean", [0.485, 0.456, 0.406]), dtype=np.float32)
        std = np.asarray(pre.get("image_std", [0.229, 0.224, 0.225]), dtype=np.float32)
        w, h = image.size
        s = short_side / min(w, h)
        nw, nh = max(self.patch, round(w * s / self.patch) * self.patch), max(self.patch, round(h * s / self.patch) * self.patch)
        a = np.asarray(image.convert("RGB").resize((nw, nh), Image.Resampling.BICUBIC), dtype=np.float32) / 255.0
        px = torch.from_numpy(np.ascontiguousarray(((a - mean) / std).transpose(2, 0, 1)))[None]
        d = self.predict(px)
        d = F.interpolate(d[:, None], size=(h, w), mode="bicubic", align_corners=False)[0, 0]
        return d.cpu().numpy()
