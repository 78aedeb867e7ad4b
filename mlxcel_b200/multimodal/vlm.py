"""Vision-language wrapper: images → rows of the language model's embedding stream.

``VisionLanguage.prepare(prompt_ids, images)`` expands every image placeholder token of the prompt
to as many tokens as the connector emits for that image, runs tower + connector, and returns the
expanded prompt, the embedding rows with their positions, and a *key* token sequence in which the
placeholder ids are replaced by values derived from the image content — the prefix cache hashes
those, so two requests share cached KV blocks only when text AND images are the same
(the reference's placeholder expansion and media hashing: src/multimodal/prompt*.rs,
src/multimodal/runtime*.rs).

Supported wrappers: ``llava`` (CLIP or SigLIP tower, two-layer MLP connector), ``idefics3`` /
``smolvlm`` (SigLIP-layout tower, pixel-shuffle connector, one tile per image), ``qwen2_vl`` and
``qwen2_5_vl``, ``qwen3_vl`` and ``glm4v`` (see `qwen2_vision.py`), ``internvl`` (InternViT tower, pixel-shuffle +
MLP connector, one tile per image) and ``mistral3`` (Pixtral tower at the image's own aspect ratio,
patch-merging connector; the prompt carries one row of image tokens per patch row, closed by a
break token, the last by an end token). The language model is loaded by the ordinary decoder loader
from the same checkpoint (its tensors live under ``language_model``).
"""
from __future__ import annotations

import hashlib
import json
import math
from pathlib import Path

import torch

from ..models.vision import (Cohere2VisionConnector, InternVLConnector, InternViTTower, LlavaConnector, Mistral3Connector, PixelShuffleConnector,
                             PixtralTower, ViTTower, VisionConfig)
from .images import ImageProcessor

SUPPORTED = ("llava", "qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "idefics3", "smolvlm", "internvl", "mistral3", "glm4v", "glm4v_moe", "cohere2_vision", "paddleocr_vl", "glm_ocr")


def is_vlm_checkpoint(path: str | Path) -> bool:
    f = Path(path) / "config.json"
    if not f.exists():
        return False
    raw = json.loads(f.read_text())
    return raw.get("model_type") in SUPPORTED and isinstance(raw.get("vision_config"), dict)


def _sub(src, *prefixes) -> dict:
    """Tensors of the first prefix that exists, with the prefix removed."""
    keys = list(src.keys())
    for p in prefixes:
        hit = [k for k in keys if k.startswith(p)]
        if hit:
            return {k[len(p):]: src.get(k) for k in hit}
    raise KeyError(f"no tensors under any of {prefixes}")


class VisionLanguage:
    def __init__(self, tower, connector, processor, image_token_id: int, model_type: str = "llava"):
        self.tower, self.connector, self.processor = tower, connector, processor
        self.image_token_id = int(image_token_id)
        self.model_type = model_type
        # what stands for one image in prompt text when the chat template does not place it itself
        self.placeholder_text = {"llava": "<image>", "qwen2_vl": "<|vision_start|><|image_pad|><|vision_end|>",
                                 "qwen2_5_vl": "<|vision_start|><|image_pad|><|vision_end|>",
                                 "qwen3_vl": "<|vision_start|><|image_pad|><|vision_end|>",
                                 "qwen3_vl_moe": "<|vision_start|><|image_pad|><|vision_end|>",
                                 "idefics3": "<fake_token_around_image><global-img><image><fake_token_around_image>",
                                 "smolvlm": "<fake_token_around_image><global-img><image><fake_token_around_image>",
                                 "internvl": "<img><IMG_CONTEXT></img>", "glm4v": "<|begin_of_image|><|image|><|end_of_image|>", "glm4v_moe": "<|begin_of_image|><|image|><|end_of_image|>", "glm_ocr": "<|begin_of_image|><|image|><|end_of_image|>",
                                 "cohere2_vision": "<|START_OF_IMG|><|IMG_PATCH|><|END_OF_IMG|>",
                                 "paddleocr_vl": "<|IMAGE_START|><|IMAGE_PLACEHOLDER|><|IMAGE_END|>", "mistral3": "[IMG]"}.get(
                                     model_type, "<image>")
        self.stats = dict(images=0, image_tokens=0, encode_seconds=0.0)

    @staticmethod
    def from_checkpoint(path: str | Path, dtype=torch.bfloat16, device="cpu") -> "VisionLanguage":
        from ..loading.checkpoint import TensorSource
        path = Path(path)
        raw = json.loads((path / "config.json").read_text())
        mt = raw.get("model_type")
        src = TensorSource(path)
        if mt == "llava":
            vc = VisionConfig.from_dict(raw["vision_config"], raw)
            tower = ViTTower(vc, _sub(src, "model.vision_tower.vision_model.", "vision_tower.vision_model."), dtype, device)
            conn = LlavaConnector(_sub(src, "model.multi_modal_projector.", "multi_modal_projector."),
                                  raw.get("projector_hidden_act", "gelu"), dtype, device)
            proc = ImageProcessor.from_path(path, vc.image_size)
            return VisionLanguage(tower, conn, proc, raw.get("image_token_index", raw.get("image_token_id", 32000)), mt)
        if mt in ("idefics3", "smolvlm"):
            # SigLIP-layout tower, pixel-shuffle connector. One tile per image (the whole image resized
            # to the tower's square input); the multi-tile split of large images is not done.
            vc = VisionConfig.from_dict(raw["vision_config"], {})
            vc.feature_layer, vc.drop_cls = -1, False
            tower = ViTTower(vc, _sub(src, "model.vision_model.", "vision_model."), dtype, device)
            conn = PixelShuffleConnector(_sub(src, "model.connector.", "connector."), int(raw.get("scale_factor", 2)), dtype, device)
            proc = ImageProcessor(dict(size={"height": vc.image_size, "width": vc.image_size}, do_center_crop=False,
                                       resample=1, image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5]), vc.image_size)
            return VisionLanguage(tower, conn, proc, raw.get("image_token_id", 128257), mt)
        if mt == "internvl":
            v = raw["vision_config"]
            fl = raw.get("vision_feature_layer", -1)
            tower = InternViTTower(v, _sub(src, "model.vision_tower.", "vision_tower."), int(fl if not isinstance(fl, list) else fl[-1]),
                                   raw.get("vision_feature_select_strategy", "default") == "default", dtype, device)
            conn = InternVLConnector(_sub(src, "model.multi_modal_projector.", "multi_modal_projector."),
                                     float(raw.get("downsample_ratio", 0.5)), raw.get("projector_hidden_act", "gelu"), dtype, device)
            f = path / "preprocessor_config.json"
            pc = json.loads(f.read_text()) if f.exists() else {}
            # one tile per image: the whole image resized to the tower's square input (the tiling of
            # large images into several crops plus a thumbnail is not done)
            proc = ImageProcessor(dict(size={"height": tower.image_size, "width": tower.image_size}, do_center_crop=False,
                                       resample=pc.get("resample", 3), image_mean=pc.get("image_mean", [0.485, 0.456, 0.406]),
                                       image_std=pc.get("image_std", [0.229, 0.224, 0.225])), tower.image_size)
            return VisionLanguage(tower, conn, proc, raw.get("image_token_id", 151667), mt)
        if mt == "cohere2_vision":
            # SigLIP tower (last state), one tile per image: the split of large images into several crops
            # plus a thumbnail is not done
            vc = VisionConfig.from_dict(raw["vision_config"], {})
            vc.kind, vc.feature_layer, vc.drop_cls = "siglip", -1, False
            tower = ViTTower(vc, _sub(src, "model.vision_tower.vision_model.", "vision_tower.vision_model."), dtype, device)
            conn = Cohere2VisionConnector(_sub(src, "model.multi_modal_projector.", "multi_modal_projector."),
                                          int(raw.get("downsample_factor", 2)), dtype, device)
            proc = ImageProcessor(dict(size={"height": vc.image_size, "width": vc.image_size}, do_center_crop=False,
                                       resample=3, image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5]), vc.image_size)
            return VisionLanguage(tower, conn, proc, raw.get("image_token_id", 255036), mt)
        if mt == "mistral3":
            return PixtralVisionLanguage.build(path, raw, src, dtype, device)
        if mt in ("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "glm4v", "glm4v_moe", "paddleocr_vl", "glm_ocr"):
            from .qwen2_vision import build_qwen2_vision
            return build_qwen2_vision(path, raw, src, dtype, device)
        raise ValueError(f"unsupported vision-language model_type {mt!r}; supported: {SUPPORTED}")

    # ------------------------------------------------------------------ encoding
    def tokens_for(self, image) -> int:
        return self.connector.tokens_out(self.tower.tokens_per_image)

    @torch.no_grad()
    def encode(self, images: list) -> list[torch.Tensor]:
        """One [tokens, text_hidden] tensor per image (on the tower's device)."""
        if not images:
            return []
        import time
        t0 = time.perf_counter()
        px = self.processor(images)
        rows = self.connector.forward(self.tower.forward(px))
        self.stats["images"] += len(images)
        self.stats["image_tokens"] += int(rows.shape[0] * rows.shape[1])
        self.stats["encode_seconds"] += time.perf_counter() - t0
        return [rows[i] for i in range(rows.shape[0])]

    def prepare(self, prompt_ids: list[int], images: list):
        """Returns ``(ids, mm)``: the prompt with every placeholder expanded and the keyword arguments
        `Engine.add_request` takes for it — ``mm_embeds = [(start, rows)]``, ``key_tokens`` for prefix
        hashing, and for the Qwen2-VL family ``rope_pos`` / ``rope_delta`` (3-D rotary positions)."""
        n_ph = sum(1 for t in prompt_ids if t == self.image_token_id)
        if n_ph != len(images):
            raise ValueError(f"the prompt has {n_ph} image placeholders for {len(images)} images")
        embeds = self.encode(images)
        ids, keys, spans = [], [], []
        it = iter(embeds)
        for t in prompt_ids:
            if t != self.image_token_id:
                ids.append(t)
                keys.append(t)
                continue
            rows = next(it)
            n = int(rows.shape[0])
            salt = int.from_bytes(hashlib.sha1(rows.detach().float().cpu().numpy().tobytes()).digest()[:4], "little")
            spans.append((len(ids), rows))
            ids += [self.image_token_id] * n
            keys += [-(2 + ((salt + j) & 0x3FFFFFFF)) for j in range(n)]
        return ids, dict(mm_embeds=spans, key_tokens=keys)


class PixtralVisionLanguage(VisionLanguage):
    """Mistral3 / Pixtral: every image keeps its aspect ratio (longest edge capped, sides rounded up to
    whole merged patches), and its placeholder expands to one run of image tokens per row of merged
    patches, each run followed by the break token and the last by the end token — those two are
    ordinary vocabulary entries, only the image tokens take the connector's rows
    (the reference's src/loading/vlm_pixtral.rs, src/vision/encoders/pixtral.rs)."""

    @staticmethod
    def build(path, raw, src, dtype, device) -> "PixtralVisionLanguage":
        v = raw["vision_config"]
        fl = raw.get("vision_feature_layer", -1)
        tower = PixtralTower(v, _sub(src, "model.vision_tower.", "vision_tower."), int(fl if not isinstance(fl, list) else fl[-1]),
                             dtype, device)
        conn = Mistral3Connector(_sub(src, "model.multi_modal_projector.", "multi_modal_projector."),
                                 int(raw.get("spatial_merge_size", 2)), float((raw.get("text_config") or {}).get("rms_norm_eps", 1e-5)),
                                 raw.get("projector_hidden_act", "gelu"), dtype, device)
        f = path / "preprocessor_config.json"
        pc = json.loads(f.read_text()) if f.exists() else {}
        vl = PixtralVisionLanguage(tower, conn, None, raw.get("image_token_index", raw.get("image_token_id", 10)), "mistral3")
        size = pc.get("size") or {}
        vl.longest_edge = int(size.get("longest_edge", tower.image_size))
        vl.mean = pc.get("image_mean", [0.48145466, 0.4578275, 0.40821073])
        vl.std = pc.get("image_std", [0.26862954, 0.26130258, 0.27577711])
        vl.break_id = int(raw.get("image_break_token_id", pc.get("image_break_token_id", 12)))
        vl.end_id = int(raw.get("image_end_token_id", pc.get("image_end_token_id", 13)))
        return vl

    def pixels(self, img) -> torch.Tensor:
        """Resize so the longest edge fits, sides rounded up to whole merged patches (bicubic), normalise."""
        import numpy as np
        from PIL import Image
        unit = self.tower.patch * self.connector.s
        w, h = img.size
        ratio = max(h / self.longest_edge, w / self.longest_edge)
        if ratio > 1:
            h, w = int(math.floor(h / ratio)), int(math.floor(w / ratio))
        nh, nw = max(1, -(-h // unit)) * unit, max(1, -(-w // unit)) * unit
        a = np.asarray(img.convert("RGB").resize((nw, nh), Image.Resampling.BICUBIC), dtype=np.float32) / 255.0
        a = (a - np.asarray(self.mean, dtype=np.float32)) / np.asarray(self.std, dtype=np.float32)
        return torch.from_numpy(np.ascontiguousarray(a.transpose(2, 0, 1))).float()

    @torch.no_grad()
    def encode(self, images: list) -> list:
        """One ``(rows [th * tw, text_hidden], th, tw)`` per image."""
        import time
        t0 = time.perf_counter()
        out = []
        for img in images:
            px = img if isinstance(img, torch.Tensor) else self.pixels(img)
            gh, gw = px.shape[1] // self.tower.patch, px.shape[2] // self.tower.patch
            rows = self.connector.forward_one(self.tower.forward_one(px), gh, gw)
            out.append((rows, gh // self.connector.s, gw // self.connector.s))
            self.stats["image_tokens"] += int(rows.shape[0])
        self.stats["images"] += len(images)
        self.stats["encode_seconds"] += time.perf_counter() - t0
        return out

    def tokens_for(self, image) -> int:
        px = image if isinstance(image, torch.Tensor) else self.pixels(image)
        unit = self.tower.patch * self.connector.s
        return (px.shape[1] // unit) * (px.shape[2] // unit + 1)

    def prepare(self, prompt_ids: list[int], images: list):
        n_ph = sum(1 for t in prompt_ids if t == self.image_token_id)
        if n_ph != len(images):
            raise ValueError(f"the prompt has {n_ph} image placeholders for {len(images)} images")
        it = iter(self.encode(images))
        ids, keys, spans = [], [], []
        for t in prompt_ids:
            if t != self.image_token_id:
                ids.append(t)
                keys.append(t)
                continue
            rows, th, tw = next(it)
            salt = int.from_bytes(hashlib.sha1(rows.detach().float().cpu().numpy().tobytes()).digest()[:4], "little")
            for r in range(th):
                spans.append((len(ids), rows[r * tw:(r + 1) * tw]))
                ids += [self.image_token_id] * tw
                keys += [-(2 + ((salt + r * tw + j) & 0x3FFFFFFF)) for j in range(tw)]
                closing = self.end_id if r == th - 1 else self.break_id
                ids.append(closing)
                keys.append(closing)
        return ids, dict(mm_embeds=spans, key_tokens=keys)
