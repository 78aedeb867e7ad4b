"""Qwen2-VL vision side: dynamic-resolution processor, vision transformer with 2-D rotary positions,
patch merger, and the 3-D rotary positions of the language model's prompt
(reference: src/vision/encoders/qwen2_vl*.rs, src/vision/processors/qwen2_vl*.rs, src/models/qwen2_vl.rs).

An image is resized so both sides are multiples of ``patch * merge`` (28) inside a pixel budget, cut
into 14 x 14 patches (the single frame is repeated over the temporal patch of 2), and the patches
are ordered merge-window by merge-window so that every 2 x 2 neighbourhood is contiguous: the merger
then folds 4 consecutive rows into one language-model token. The language model sees, per image, a
grid of (h/2) x (w/2) tokens whose rotary positions are (t, row, col) offsets from the running text
position; text after the image continues at ``max(position) + 1``.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..ops import recurrent as rops
from .vlm import VisionLanguage, _sub


def smart_resize(h: int, w: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280):
    """Both sides multiples of ``factor``, area within [min_pixels, max_pixels], aspect ratio kept."""
    if max(h, w) / min(h, w) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    hb = max(factor, round(h / factor) * factor)
    wb = max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt((h * w) / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb = math.ceil(h * beta / factor) * factor
        wb = math.ceil(w * beta / factor) * factor
    return hb, wb


class Qwen2ImageProcessor:
    def __init__(self, cfg: dict | None = None, patch: int = 14, merge: int = 2, temporal: int = 2):
        cfg = dict(cfg or {})
        self.patch = int(cfg.get("patch_size", patch))
        self.merge = int(cfg.get("merge_size", merge))
        self.temporal = int(cfg.get("temporal_patch_size", temporal))
        size = cfg.get("size") or {}
        self.min_pixels = int(cfg.get("min_pixels", size.get("shortest_edge", 56 * 56)))
        self.max_pixels = int(cfg.get("max_pixels", size.get("longest_edge", 28 * 28 * 1280)))
        self.mean = np.asarray(cfg.get("image_mean", [0.48145466, 0.4578275, 0.40821073]), dtype=np.float32)
        self.std = np.asarray(cfg.get("image_std", [0.26862954, 0.26130258, 0.27577711]), dtype=np.float32)

    def __call__(self, images: list):
        """PIL images → (patch rows float32 [sum gh*gw, C * temporal * patch * patch], grids [(1, gh, gw)])."""
        from PIL import Image
        p, m, tp = self.patch, self.merge, self.temporal
        rows, grids = [], []
        for img in images:
            w, h = img.size
            nh, nw = smart_resize(h, w, p * m, self.min_pixels, self.max_pixels)
            a = np.asarray(img.resize((nw, nh), Image.Resampling.BICUBIC), dtype=np.float32) / 255.0
            a = ((a - self.mean) / self.std).transpose(2, 0, 1)                 # [C, H, W]
            a = np.repeat(a[None], tp, axis=0)                                  # the frame fills the temporal patch
            gh, gw = nh // p, nw // p
            C = a.shape[1]
            x = a.reshape(1, tp, C, gh // m, m, p, gw // m, m, p)
            x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)                          # [1, gh/m, gw/m, m, m, C, tp, p, p]
            rows.append(torch.from_numpy(np.ascontiguousarray(x.reshape(gh * gw, C * tp * p * p))))
            grids.append((1, gh, gw))
        return torch.cat(rows), grids


class Qwen2VisionTower:
    """Patch embedding → blocks (LayerNorm, attention with 2-D rotary positions restricted to the
    image, quick-GELU MLP) → merger (LayerNorm, fold merge^2 rows, two linears with GELU)."""

    def __init__(self, vc: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.depth, self.dim, self.heads = int(vc["depth"]), int(vc["embed_dim"]), int(vc["num_heads"])
        self.patch, self.merge = int(vc.get("patch_size", 14)), int(vc.get("spatial_merge_size", 2))
        self.act = {"quick_gelu": "quick_gelu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh"}.get(
            vc.get("hidden_act", "quick_gelu"), "quick_gelu")

        def t(n):
            return tensors[n].to(dtype).to(self.device).contiguous()

        pw = t("patch_embed.proj.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8                  # the GEMM's TMA rows need 16-byte strides
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.blocks = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            self.blocks.append({k: t(b + n) for k, n in dict(
                n1w="norm1.weight", n1b="norm1.bias", wqkv="attn.qkv.weight", bqkv="attn.qkv.bias",
                wo="attn.proj.weight", bo="attn.proj.bias", n2w="norm2.weight", n2b="norm2.bias",
                w1="mlp.fc1.weight", b1="mlp.fc1.bias", w2="mlp.fc2.weight", b2="mlp.fc2.bias").items()})
        self.ln_q = (t("merger.ln_q.weight"), t("merger.ln_q.bias"))
        self.m1 = (t("merger.mlp.0.weight"), t("merger.mlp.0.bias"))
        self.m2 = (t("merger.mlp.2.weight"), t("merger.mlp.2.bias"))
        D = self.dim // self.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32) / (D // 2)))

    def _rot_angles(self, grids) -> torch.Tensor:
        """[rows, D/2] rotary angles: the first D/4 frequencies turn with the patch's row, the rest with
        its column, rows listed in merge-window order."""
        m, out = self.merge, []
        for t_, gh, gw in grids:
            hp = torch.arange(gh)[:, None].expand(gh, gw).reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(gw)[None, :].expand(gh, gw).reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).flatten()
            ang = torch.cat([hp[:, None].float() * self.inv_freq[None], wp[:, None].float() * self.inv_freq[None]], dim=1)
            out.append(ang.repeat(t_, 1))
        return torch.cat(out)

    @torch.no_grad()
    def forward(self, rows: torch.Tensor, grids) -> torch.Tensor:
        """``rows`` [R, C*tp*p*p] → [R / merge^2, text_hidden]."""
        from ..models.vision import _act
        x = ops.linear(F.pad(rows.to(self.device, self.dtype), (0, self.k_pad)).contiguous(), self.patch_w)
        R, H, D = x.shape[0], self.heads, self.dim // self.heads
        ang = self._rot_angles(grids).to(self.device)
        cos = torch.cat([ang.cos(), ang.cos()], dim=1)[:, None, :]       # [R, 1, D]
        sin = torch.cat([ang.sin(), ang.sin()], dim=1)[:, None, :]
        sizes = [t_ * gh * gw for t_, gh, gw in grids]

        def rot(v):            # [R, H, D] float32
            half = D // 2
            return v * cos + torch.cat([-v[..., half:], v[..., :half]], dim=-1) * sin
        for b in self.blocks:
            y = rops.layernorm(x, b["n1w"], b["n1b"], 1e-6)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(R, 3, H, D)
            q, k, v = rot(qkv[:, 0].float()), rot(qkv[:, 1].float()), qkv[:, 2].float()
            outs, o0 = [], 0
            for n in sizes:                                    # attention never crosses images
                qi, ki, vi = (z[o0:o0 + n].transpose(0, 1)[None] for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qi, ki, vi)[0].transpose(0, 1).reshape(n, H * D))
                o0 += n
            a = torch.cat(outs).to(self.dtype).contiguous()
            x = ops.linear(a, b["wo"], bias=b["bo"], residual=x)
            y = rops.layernorm(x, b["n2w"], b["n2b"], 1e-6)
            x = ops.linear(_act(ops.linear(y, b["w1"], bias=b["b1"]), self.act), b["w2"], bias=b["b2"], residual=x)
        y = rops.layernorm(x, *self.ln_q, 1e-6).view(R // self.merge ** 2, self.dim * self.merge ** 2).contiguous()
        y = rops.activation(ops.linear(y, *self.m1), "gelu")
        return ops.linear(y, *self.m2)


class Qwen25VisionTower:
    """Qwen2.5-VL tower: the Qwen2-VL layout with RMSNorm, a SwiGLU MLP and *windowed* attention. The
    merged-token groups (merge x merge patches) of an image are reordered window by window
    (``window_size`` pixels per side); most blocks attend inside a window, the blocks listed in
    ``fullatt_block_indexes`` over the whole image; the merger's output is put back into raster
    order (reference: src/vision/encoders/qwen2_5_vl*.rs)."""

    def __init__(self, vc: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.depth, self.dim, self.heads = int(vc["depth"]), int(vc["hidden_size"]), int(vc["num_heads"])
        self.patch, self.merge = int(vc.get("patch_size", 14)), int(vc.get("spatial_merge_size", 2))
        self.window = int(vc.get("window_size", 112))
        self.full_blocks = set(int(i) for i in vc.get("fullatt_block_indexes", [7, 15, 23, 31]))
        self.act = {"silu": "silu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh"}.get(vc.get("hidden_act", "silu"), "silu")

        def t(n):
            return tensors[n].to(dtype).to(self.device).contiguous()

        pw = t("patch_embed.proj.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.blocks = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            blk = {k: t(b + n) for k, n in dict(
                n1="norm1.weight", wqkv="attn.qkv.weight", bqkv="attn.qkv.bias", wo="attn.proj.weight", bo="attn.proj.bias",
                n2="norm2.weight", wd="mlp.down_proj.weight", bd="mlp.down_proj.bias").items()}
            blk["wgu"] = torch.cat([t(b + "mlp.gate_proj.weight"), t(b + "mlp.up_proj.weight")]).contiguous()
            blk["bgu"] = torch.cat([t(b + "mlp.gate_proj.bias"), t(b + "mlp.up_proj.bias")]).contiguous()
            self.blocks.append(blk)
        self.ln_q = t("merger.ln_q.weight")
        self.m1 = (t("merger.mlp.0.weight"), t("merger.mlp.0.bias"))
        self.m2 = (t("merger.mlp.2.weight"), t("merger.mlp.2.bias"))
        D = self.dim // self.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32) / (D // 2)))

    _rot_angles = Qwen2VisionTower._rot_angles

    def _windows(self, grids):
        """Order of the merged-token groups (window by window) and the group count of every window."""
        ws = self.window // self.merge // self.patch
        order, sizes, base = [], [], 0
        for t_, gh, gw in grids:
            lh, lw = gh // self.merge, gw // self.merge
            idx = torch.arange(t_ * lh * lw).reshape(t_, lh, lw)
            for ti in range(t_):
                for r0 in range(0, lh, ws):
                    for c0 in range(0, lw, ws):
                        win = idx[ti, r0:r0 + ws, c0:c0 + ws].reshape(-1)
                        order.append(win + base)
                        sizes.append(int(win.numel()))
            base += t_ * lh * lw
        return torch.cat(order), sizes

    @torch.no_grad()
    def forward(self, rows: torch.Tensor, grids) -> torch.Tensor:
        from ..models.vision import _act
        x = ops.linear(F.pad(rows.to(self.device, self.dtype), (0, self.k_pad)).contiguous(), self.patch_w)
        R, H, D = x.shape[0], self.heads, self.dim // self.heads
        unit = self.merge ** 2
        order, win_groups = self._windows(grids)
        order = order.to(self.device)
        x = x.view(R // unit, unit, self.dim)[order].reshape(R, self.dim).contiguous()
        ang = self._rot_angles(grids).to(self.device).view(R // unit, unit, -1)[order].reshape(R, -1)
        cos = torch.cat([ang.cos(), ang.cos()], dim=1)[:, None, :]
        sin = torch.cat([ang.sin(), ang.sin()], dim=1)[:, None, :]
        full_sizes = [gh * gw for t_, gh, gw in grids for _ in range(t_)]
        win_sizes = [g * unit for g in win_groups]

        def rot(v):
            half = D // 2
            return v * cos + torch.cat([-v[..., half:], v[..., :half]], dim=-1) * sin
        for li, b in enumerate(self.blocks):
            y = ops.rmsnorm(x, b["n1"], 1e-6, 0.0)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(R, 3, H, D)
            q, k, v = rot(qkv[:, 0].float()), rot(qkv[:, 1].float()), qkv[:, 2].float()
            outs, o0 = [], 0
            for n in (full_sizes if li in self.full_blocks else win_sizes):
                qi, ki, vi = (z[o0:o0 + n].transpose(0, 1)[None] for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qi, ki, vi)[0].transpose(0, 1).reshape(n, H * D))
                o0 += n
            a = torch.cat(outs).to(self.dtype).contiguous()
            x = ops.linear(a, b["wo"], bias=b["bo"], residual=x)
            y = ops.rmsnorm(x, b["n2"], 1e-6, 0.0)
            gu = ops.linear(y, b["wgu"], bias=b["bgu"])
            inter = gu.shape[1] // 2
            u = (_act(gu[:, :inter].contiguous(), self.act).float() * gu[:, inter:].float()).to(self.dtype)
            x = ops.linear(u.contiguous(), b["wd"], bias=b["bd"], residual=x)
        y = ops.rmsnorm(x, self.ln_q, 1e-6, 0.0).view(R // unit, self.dim * unit).contiguous()
        y = ops.linear(rops.activation(ops.linear(y, *self.m1), "gelu"), *self.m2)
        return y[torch.argsort(order)]


class Qwen3VisionTower(Qwen2VisionTower):
    """Qwen3-VL tower: biased patch embedding plus a learned position table interpolated bilinearly to
    the image's patch grid, full attention per image with the same 2-D rotary positions, tanh-GELU
    MLPs, a merger that norms before folding, and DeepStack mergers (norm after folding) over the
    outputs of ``deepstack_visual_indexes``. ``forward`` returns [R / merge^2, (1 + n_deep) * text_hidden]:
    the merged tokens followed by one feature block per DeepStack level, which the engine adds to the
    first language-model layers' outputs at the image rows (reference: src/vision/encoders/qwen3_vl*.rs)."""

    def __init__(self, vc: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.depth, self.dim, self.heads = int(vc["depth"]), int(vc["hidden_size"]), int(vc["num_heads"])
        self.patch, self.merge = int(vc.get("patch_size", 16)), int(vc.get("spatial_merge_size", 2))
        self.act = {"gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh", "quick_gelu": "quick_gelu"}.get(
            vc.get("hidden_act", "gelu_pytorch_tanh"), "gelu_tanh")
        self.deep_idx = [int(i) for i in vc.get("deepstack_visual_indexes", ())]

        def t(n):
            return tensors[n].to(dtype).to(self.device).contiguous()

        pw = t("patch_embed.proj.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.patch_b = t("patch_embed.proj.bias")
        self.pos_table = t("pos_embed.weight")
        self.side = int(round(self.pos_table.shape[0] ** 0.5))
        self.blocks = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            self.blocks.append({k: t(b + n) for k, n in dict(
                n1w="norm1.weight", n1b="norm1.bias", wqkv="attn.qkv.weight", bqkv="attn.qkv.bias",
                wo="attn.proj.weight", bo="attn.proj.bias", n2w="norm2.weight", n2b="norm2.bias",
                w1="mlp.linear_fc1.weight", b1="mlp.linear_fc1.bias", w2="mlp.linear_fc2.weight", b2="mlp.linear_fc2.bias").items()})

        def merger(p):
            return dict(nw=t(p + "norm.weight"), nb=t(p + "norm.bias"), w1=t(p + "linear_fc1.weight"), b1=t(p + "linear_fc1.bias"),
                        w2=t(p + "linear_fc2.weight"), b2=t(p + "linear_fc2.bias"))
        self.merger = merger("merger.")
        self.deep_mergers = [merger(f"deepstack_merger_list.{j}.") for j in range(len(self.deep_idx))]
        D = self.dim // self.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32) / (D // 2)))

    def _pos_embed(self, grids) -> torch.Tensor:
        """The learned side x side table read bilinearly at each image's gh x gw patch centres, rows in
        merge-window order (fp32)."""
        tab, n, m = self.pos_table.float(), self.side, self.merge
        out = []
        for t_, gh, gw in grids:
            hi, wi = torch.linspace(0, n - 1, gh), torch.linspace(0, n - 1, gw)
            hf, wf = hi.int(), wi.int()
            hc, wc = (hf + 1).clip(max=n - 1), (wf + 1).clip(max=n - 1)
            dh, dw = (hi - hf)[:, None], (wi - wf)[None, :]
            e = lambda a, b: tab[(a[:, None] * n + b[None, :]).long().flatten().to(tab.device)].view(gh, gw, -1)  # noqa: E731
            dh, dw = dh.to(tab.device)[..., None], dw.to(tab.device)[..., None]
            pe = e(hf, wf) * (1 - dh) * (1 - dw) + e(hf, wc) * (1 - dh) * dw + e(hc, wf) * dh * (1 - dw) + e(hc, wc) * dh * dw
            pe = pe.view(gh // m, m, gw // m, m, -1).permute(0, 2, 1, 3, 4).reshape(gh * gw, -1)
            out.append(pe.repeat(t_, 1))
        return torch.cat(out)

    def _merge(self, x: torch.Tensor, mw: dict, post: bool) -> torch.Tensor:
        R, wide = x.shape[0], self.dim * self.merge ** 2
        if post:
            y = rops.layernorm(x.view(R // self.merge ** 2, wide).contiguous(), mw["nw"], mw["nb"], 1e-6)
        else:
            y = rops.layernorm(x, mw["nw"], mw["nb"], 1e-6).view(R // self.merge ** 2, wide).contiguous()
        return ops.linear(rops.activation(ops.linear(y, mw["w1"], bias=mw["b1"]), "gelu"), mw["w2"], bias=mw["b2"])

    @torch.no_grad()
    def forward(self, rows: torch.Tensor, grids) -> torch.Tensor:
        from ..models.vision import _act
        x = ops.linear(F.pad(rows.to(self.device, self.dtype), (0, self.k_pad)).contiguous(), self.patch_w, bias=self.patch_b)
        x = (x.float() + self._pos_embed(grids).to(self.device)).to(self.dtype)
        R, H, D = x.shape[0], self.heads, self.dim // self.heads
        ang = self._rot_angles(grids).to(self.device)
        cos = torch.cat([ang.cos(), ang.cos()], dim=1)[:, None, :]
        sin = torch.cat([ang.sin(), ang.sin()], dim=1)[:, None, :]
        sizes = [gh * gw for t_, gh, gw in grids for _ in range(t_)]          # attention stays inside a frame

        def rot(v):
            half = D // 2
            return v * cos + torch.cat([-v[..., half:], v[..., :half]], dim=-1) * sin
        deep = []
        for li, b in enumerate(self.blocks):
            y = rops.layernorm(x, b["n1w"], b["n1b"], 1e-6)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(R, 3, H, D)
            q, k, v = rot(qkv[:, 0].float()), rot(qkv[:, 1].float()), qkv[:, 2].float()
            outs, o0 = [], 0
            for n in sizes:
                qi, ki, vi = (z[o0:o0 + n].transpose(0, 1)[None] for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qi, ki, vi)[0].transpose(0, 1).reshape(n, H * D))
                o0 += n
            a = torch.cat(outs).to(self.dtype).contiguous()
            x = ops.linear(a, b["wo"], bias=b["bo"], residual=x)
            y = rops.layernorm(x, b["n2w"], b["n2b"], 1e-6)
            x = ops.linear(_act(ops.linear(y, b["w1"], bias=b["b1"]), self.act), b["w2"], bias=b["b2"], residual=x)
            if li in self.deep_idx:
                deep.append(self._merge(x, self.deep_mergers[self.deep_idx.index(li)], post=True))
        return torch.cat([self._merge(x, self.merger, post=False)] + deep, dim=1)


class Glm4vVisionTower(Qwen2VisionTower):
    """GLM-4.1V tower (transformers `Glm4vVisionModel`; the reference's src/vision/encoders/glm4v.rs): biased
    patch embedding, RMSNorm, a learned position table sampled bicubically at each patch centre, blocks
    of RMSNorm + attention under the Qwen2-VL 2-D rotary positions + bias-free gated MLP, RMSNorm, a
    strided convolution that folds every merge x merge group into one row, and a merger (linear,
    LayerNorm, GELU, gated MLP). Rows come in merge-window order like the Qwen2-VL tower's."""

    def __init__(self, vc: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.depth, self.dim, self.heads = int(vc["depth"]), int(vc["hidden_size"]), int(vc["num_heads"])
        self.patch, self.merge = int(vc.get("patch_size", 14)), int(vc.get("spatial_merge_size", 2))
        self.eps = float(vc.get("rms_norm_eps", 1e-5))
        self.act = {"silu": "silu", "gelu": "gelu", "gelu_pytorch_tanh": "gelu_tanh"}.get(vc.get("hidden_act", "silu"), "silu")

        def t(n, required=True):
            if n not in tensors and not required:
                return None
            return tensors[n].to(dtype).to(self.device).contiguous()

        pw = t("patch_embed.proj.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.patch_b = t("patch_embed.proj.bias")
        # GLM-OCR drops the norm after the patch embedding and the position table, norms q and k per head,
        # and carries biases on the output projection and the MLP
        self.post_conv = t("post_conv_layernorm.weight", False)
        self.pos_table = t("embeddings.position_embedding.weight", False)
        self.side = int(round(self.pos_table.shape[0] ** 0.5)) if self.pos_table is not None else 0
        self.blocks = []
        for i in range(self.depth):
            b = f"blocks.{i}."
            bg, bu = t(b + "mlp.gate_proj.bias", False), t(b + "mlp.up_proj.bias", False)
            self.blocks.append(dict(
                n1=t(b + "norm1.weight"), n2=t(b + "norm2.weight"), wqkv=t(b + "attn.qkv.weight"), bqkv=t(b + "attn.qkv.bias", False),
                wo=t(b + "attn.proj.weight"), bo=t(b + "attn.proj.bias", False),
                qn=t(b + "attn.q_norm.weight", False), kn=t(b + "attn.k_norm.weight", False),
                wgu=torch.cat([t(b + "mlp.gate_proj.weight"), t(b + "mlp.up_proj.weight")]).contiguous(),
                bgu=None if bg is None else torch.cat([bg, bu]).contiguous(),
                wd=t(b + "mlp.down_proj.weight"), bd=t(b + "mlp.down_proj.bias", False)))
        self.post_ln = t("post_layernorm.weight")
        dw = t("downsample.weight")                                   # [out, C, m, m]
        self.down_w, self.down_b = dw.reshape(dw.shape[0], -1).contiguous(), t("downsample.bias")
        self.mg = dict(proj=t("merger.proj.weight"), nw=t("merger.post_projection_norm.weight"), nb=t("merger.post_projection_norm.bias"),
                       wgu=torch.cat([t("merger.gate_proj.weight"), t("merger.up_proj.weight")]).contiguous(),
                       wd=t("merger.down_proj.weight"))
        D = self.dim // self.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32) / (D // 2)))

    def _pos_embed(self, grids) -> torch.Tensor:
        tab = self.pos_table.float().view(self.side, self.side, -1).permute(2, 0, 1)[None]
        m, out = self.merge, []
        for t_, gh, gw in grids:
            hp = torch.arange(gh)[:, None].expand(gh, gw).reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).flatten()
            wp = torch.arange(gw)[None, :].expand(gh, gw).reshape(gh // m, m, gw // m, m).permute(0, 2, 1, 3).flatten()
            grid = torch.stack([(wp.float() + 0.5) / gw * 2 - 1, (hp.float() + 0.5) / gh * 2 - 1], dim=-1)[None, :, None, :]
            pe = F.grid_sample(tab, grid.to(tab.device), mode="bicubic", align_corners=False, padding_mode="border")
            out.append(pe[0, :, :, 0].t().repeat(t_, 1))
        return torch.cat(out)

    def _gated(self, y, wgu, wd, residual=None, bgu=None, bd=None):
        from ..models.vision import _act
        gu = ops.linear(y, wgu, bias=bgu)
        inter = gu.shape[1] // 2
        u = (_act(gu[:, :inter].contiguous(), self.act).float() * gu[:, inter:].float()).to(self.dtype).contiguous()
        return ops.linear(u, wd, bias=bd, residual=residual)

    @torch.no_grad()
    def forward(self, rows: torch.Tensor, grids) -> torch.Tensor:
        x = ops.linear(F.pad(rows.to(self.device, self.dtype), (0, self.k_pad)).contiguous(), self.patch_w, bias=self.patch_b)
        if self.post_conv is not None:
            x = ops.rmsnorm(x, self.post_conv, self.eps)
        if self.pos_table is not None:
            x = (x.float() + self._pos_embed(grids).to(self.device)).to(self.dtype)
        R, H, D = x.shape[0], self.heads, self.dim // self.heads
        ang = self._rot_angles(grids).to(self.device)
        cos = torch.cat([ang.cos(), ang.cos()], dim=1)[:, None, :]
        sin = torch.cat([ang.sin(), ang.sin()], dim=1)[:, None, :]
        sizes = [gh * gw for t_, gh, gw in grids for _ in range(t_)]

        def rot(v):
            half = D // 2
            return v * cos + torch.cat([-v[..., half:], v[..., :half]], dim=-1) * sin
        for b in self.blocks:
            y = ops.rmsnorm(x, b["n1"], self.eps)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(R, 3, H, D)
            q, k, v = qkv[:, 0].float(), qkv[:, 1].float(), qkv[:, 2].float()
            if b["qn"] is not None:
                hn = lambda z, w: z * torch.rsqrt(z.pow(2).mean(-1, keepdim=True) + self.eps) * w.float()  # noqa: E731
                q, k = hn(q, b["qn"]), hn(k, b["kn"])
            q, k = rot(q), rot(k)
            outs, o0 = [], 0
            for n in sizes:
                qi, ki, vi = (z[o0:o0 + n].transpose(0, 1)[None] for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qi, ki, vi)[0].transpose(0, 1).reshape(n, H * D))
                o0 += n
            x = ops.linear(torch.cat(outs).to(self.dtype).contiguous(), b["wo"], bias=b["bo"], residual=x)
            x = self._gated(ops.rmsnorm(x, b["n2"], self.eps), b["wgu"], b["wd"], residual=x, bgu=b["bgu"], bd=b["bd"])
        x = ops.rmsnorm(x, self.post_ln, self.eps)
        unit = self.merge ** 2
        y = x.view(R // unit, unit, self.dim).transpose(1, 2).reshape(R // unit, self.dim * unit).contiguous()
        y = ops.linear(y, self.down_w, bias=self.down_b)
        y = ops.linear(y, self.mg["proj"])
        y = rops.activation(rops.layernorm(y, self.mg["nw"], self.mg["nb"], 1e-5), "gelu")
        return self._gated(y, self.mg["wgu"], self.mg["wd"])


class RasterImageProcessor(Qwen2ImageProcessor):
    """The Qwen2-VL resize and normalisation with patches listed row by row (no merge-window order) and
    no temporal patch: rows are ``[C * patch * patch]`` (PaddleOCR-VL)."""

    def __call__(self, images: list):
        from PIL import Image
        p, m = self.patch, self.merge
        rows, grids = [], []
        for img in images:
            w, h = img.size
            nh, nw = smart_resize(h, w, p * m, self.min_pixels, self.max_pixels)
            a = np.asarray(img.resize((nw, nh), Image.Resampling.BICUBIC), dtype=np.float32) / 255.0
            a = ((a - self.mean) / self.std).transpose(2, 0, 1)
            gh, gw, C = nh // p, nw // p, a.shape[0]
            x = a.reshape(C, gh, p, gw, p).transpose(1, 3, 0, 2, 4)
            rows.append(torch.from_numpy(np.ascontiguousarray(x.reshape(gh * gw, C * p * p))))
            grids.append((1, gh, gw))
        return torch.cat(rows), grids


class PaddleOcrVisionTower(Qwen2VisionTower):
    """PaddleOCR-VL tower (transformers `PaddleOCRVisionModel` + `PaddleOCRProjector`; the reference's
    src/vision/encoders/paddleocr_vl.rs): SigLIP-layout blocks over patches in raster order, a learned
    position table resized bilinearly to the image's grid, 2-D rotary positions (row / column
    halves), a final LayerNorm; the projector norms each patch, folds merge x merge neighbours and
    applies linear, GELU, linear."""

    def __init__(self, vc: dict, tensors: dict, proj: dict, dtype=torch.bfloat16, device="cpu"):
        self.dtype, self.device = dtype, torch.device(device)
        self.depth, self.dim, self.heads = int(vc["num_hidden_layers"]), int(vc["hidden_size"]), int(vc["num_attention_heads"])
        self.patch, self.merge = int(vc.get("patch_size", 14)), int(vc.get("spatial_merge_size", 2))
        self.eps = float(vc.get("layer_norm_eps", 1e-6))
        self.act = {"gelu_pytorch_tanh": "gelu_tanh", "gelu": "gelu", "quick_gelu": "quick_gelu"}.get(
            vc.get("hidden_act", "gelu_pytorch_tanh"), "gelu_tanh")

        def t(n, src=tensors):
            return src[n].to(dtype).to(self.device).contiguous()

        pw = t("embeddings.patch_embedding.weight")
        pw = pw.reshape(pw.shape[0], -1)
        self.k_pad = (-pw.shape[1]) % 8
        self.patch_w = F.pad(pw, (0, self.k_pad)).contiguous()
        self.patch_b = t("embeddings.patch_embedding.bias")
        self.pos_table = t("embeddings.position_embedding.weight")
        self.side = int(round(self.pos_table.shape[0] ** 0.5))
        self.blocks = []
        for i in range(self.depth):
            b, a = f"encoder.layers.{i}.", f"encoder.layers.{i}.self_attn."
            self.blocks.append(dict(
                n1=(t(b + "layer_norm1.weight"), t(b + "layer_norm1.bias")), n2=(t(b + "layer_norm2.weight"), t(b + "layer_norm2.bias")),
                wqkv=torch.cat([t(a + "q_proj.weight"), t(a + "k_proj.weight"), t(a + "v_proj.weight")]).contiguous(),
                bqkv=torch.cat([t(a + "q_proj.bias"), t(a + "k_proj.bias"), t(a + "v_proj.bias")]).contiguous(),
                wo=t(a + "out_proj.weight"), bo=t(a + "out_proj.bias"),
                w1=t(b + "mlp.fc1.weight"), b1=t(b + "mlp.fc1.bias"), w2=t(b + "mlp.fc2.weight"), b2=t(b + "mlp.fc2.bias")))
        self.post_ln = (t("post_layernorm.weight"), t("post_layernorm.bias"))
        self.pj = dict(nw=t("pre_norm.weight", proj), nb=t("pre_norm.bias", proj), w1=t("linear_1.weight", proj), b1=t("linear_1.bias", proj),
                       w2=t("linear_2.weight", proj), b2=t("linear_2.bias", proj))
        D = self.dim // self.heads
        self.inv_freq = 1.0 / (10000.0 ** (torch.arange(0, D // 2, 2, dtype=torch.float32) / (D // 2)))

    @torch.no_grad()
    def forward(self, rows: torch.Tensor, grids) -> torch.Tensor:
        from ..models.vision import _act
        x = ops.linear(F.pad(rows.to(self.device, self.dtype), (0, self.k_pad)).contiguous(), self.patch_w, bias=self.patch_b)
        tab = self.pos_table.float().view(1, self.side, self.side, -1).permute(0, 3, 1, 2)
        pos, ang = [], []
        for t_, gh, gw in grids:
            pe = F.interpolate(tab, size=(gh, gw), mode="bilinear", align_corners=False)
            pos.append(pe.permute(0, 2, 3, 1).reshape(gh * gw, -1).repeat(t_, 1))
            hp = torch.arange(gh)[:, None].expand(gh, gw).flatten().float()
            wp = torch.arange(gw)[None, :].expand(gh, gw).flatten().float()
            ang.append(torch.cat([hp[:, None] * self.inv_freq[None], wp[:, None] * self.inv_freq[None]], dim=1).repeat(t_, 1))
        x = (x.float() + torch.cat(pos).to(self.device)).to(self.dtype)
        ang = torch.cat(ang).to(self.device)
        cos = torch.cat([ang.cos(), ang.cos()], dim=1)[:, None, :]
        sin = torch.cat([ang.sin(), ang.sin()], dim=1)[:, None, :]
        R, H, D = x.shape[0], self.heads, self.dim // self.heads
        sizes = [gh * gw for t_, gh, gw in grids for _ in range(t_)]

        def rot(v):
            half = D // 2
            return v * cos + torch.cat([-v[..., half:], v[..., :half]], dim=-1) * sin
        for b in self.blocks:
            y = rops.layernorm(x, *b["n1"], self.eps)
            qkv = ops.linear(y, b["wqkv"], bias=b["bqkv"]).view(R, 3, H, D)
            q, k, v = rot(qkv[:, 0].float()), rot(qkv[:, 1].float()), qkv[:, 2].float()
            outs, o0 = [], 0
            for n in sizes:
                qi, ki, vi = (z[o0:o0 + n].transpose(0, 1)[None] for z in (q, k, v))
                outs.append(F.scaled_dot_product_attention(qi, ki, vi)[0].transpose(0, 1).reshape(n, H * D))
                o0 += n
            x = ops.linear(torch.cat(outs).to(self.dtype).contiguous(), b["wo"], bias=b["bo"], residual=x)
            y = rops.layernorm(x, *b["n2"], self.eps)
            x = ops.linear(_act(ops.linear(y, b["w1"], bias=b["b1"]), self.act), b["w2"], bias=b["b2"], residual=x)
        x = rops.layernorm(x, *self.post_ln, self.eps)
        x = rops.layernorm(x, self.pj["nw"], self.pj["nb"], 1e-5)
        m, out, o0 = self.merge, [], 0
        for t_, gh, gw in grids:
            n = t_ * gh * gw
            y = x[o0:o0 + n].view(t_, gh // m, m, gw // m, m, self.dim).transpose(2, 3).reshape(n // (m * m), m * m * self.dim)
            out.append(y)
            o0 += n
        y = torch.cat(out).contiguous()
        return ops.linear(rops.activation(ops.linear(y, self.pj["w1"], bias=self.pj["b1"]), "gelu"), self.pj["w2"], bias=self.pj["b2"])


class Qwen2VisionLanguage(VisionLanguage):
    def __init__(self, tower: Qwen2VisionTower, processor: Qwen2ImageProcessor, image_token_id: int, model_type: str):
        super().__init__(tower, None, processor, image_token_id, model_type)

    @torch.no_grad()
    def encode_grids(self, images: list):
        import time
        t0 = time.perf_counter()
        rows, grids = self.processor(images)
        out = self.tower.forward(rows, grids)
        m2 = self.tower.merge ** 2
        parts, o = [], 0
        for t_, gh, gw in grids:
            n = t_ * gh * gw // m2
            parts.append(out[o:o + n])
            o += n
        self.stats["images"] += len(images)
        self.stats["image_tokens"] += int(out.shape[0])
        self.stats["encode_seconds"] += time.perf_counter() - t0
        return parts, grids

    def encode(self, images: list) -> list[torch.Tensor]:
        return self.encode_grids(images)[0] if images else []

    def prepare(self, prompt_ids: list[int], images: list):
        import hashlib
        n_ph = sum(1 for t in prompt_ids if t == self.image_token_id)
        if n_ph != len(images):
            raise ValueError(f"the prompt has {n_ph} image placeholders for {len(images)} images")
        parts, grids = self.encode_grids(images) if images else ([], [])
        m = self.tower.merge
        ids, keys, spans, pos = [], [], [], [[], [], []]
        nxt, it = 0, iter(zip(parts, grids))                 # nxt: rotary position of the next text token
        for t in prompt_ids:
            if t != self.image_token_id:
                ids.append(t)
                keys.append(t)
                for c in range(3):
                    pos[c].append(nxt)
                nxt += 1
                continue
            rows, (t_, gh, gw) = next(it)
            lh, lw = gh // m, gw // m
            n = int(rows.shape[0])
            salt = int.from_bytes(hashlib.sha1(rows.detach().float().cpu().numpy().tobytes()).digest()[:4], "little")
            spans.append((len(ids), rows))
            ids += [self.image_token_id] * n
            keys += [-(2 + ((salt + j) & 0x3FFFFFFF)) for j in range(n)]
            for ti in range(t_):
                for r in range(lh):
                    for c in range(lw):
                        pos[0].append(nxt + ti)
                        pos[1].append(nxt + r)
                        pos[2].append(nxt + c)
            nxt += max(t_, lh, lw)
        mm = dict(mm_embeds=spans, key_tokens=keys)
        if images:
            mm.update(rope_pos=np.asarray(pos, dtype=np.int32), rope_delta=nxt - len(ids))
        return ids, mm


def build_qwen2_vision(path, raw: dict, src, dtype, device) -> Qwen2VisionLanguage:
    import json
    from pathlib import Path
    mt = raw.get("model_type")
    if mt == "paddleocr_vl":
        vc = raw["vision_config"]
        tower = PaddleOcrVisionTower(vc, _sub(src, "model.visual.vision_model.", "visual.vision_model."),
                                     _sub(src, "mlp_AR.", "model.projector.", "projector."), dtype, device)
        f = Path(path) / "preprocessor_config.json"
        pc = json.loads(f.read_text()) if f.exists() else dict(image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5])
        return Qwen2VisionLanguage(tower, RasterImageProcessor(pc, tower.patch, tower.merge, 1), raw.get("image_token_id", 100295), mt)
    cls = (Qwen3VisionTower if mt in ("qwen3_vl", "qwen3_vl_moe") else Qwen25VisionTower if mt == "qwen2_5_vl"
           else Glm4vVisionTower if mt in ("glm4v", "glm4v_moe", "glm_ocr") else Qwen2VisionTower)
    tower = cls(raw["vision_config"], _sub(src, "model.visual.", "visual."), dtype, device)
    f = Path(path) / "preprocessor_config.json"
    pc = json.loads(f.read_text()) if f.exists() else None
    if pc is None and mt in ("qwen3_vl", "qwen3_vl_moe"):           # this family normalises to [-1, 1]
        pc = dict(image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5])
    proc = Qwen2ImageProcessor(pc, tower.patch, tower.merge,
                               int(raw["vision_config"].get("temporal_patch_size", 2)))
    return Qwen2VisionLanguage(tower, proc, raw.get("image_token_id", 151655), raw["model_type"])
