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
``qwen2_5_vl`` and ``qwen3_vl`` (see `qwen2_vision.py`). The language model is loaded by the ordinary decoder loader
from the same checkpoint (its tensors live under ``language_model``).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from ..models.vision import LlavaConnector, PixelShuffleConnector, ViTTower, VisionConfig
from .images import ImageProcessor

SUPPORTED = ("llava", "qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe", "idefics3", "smolvlm")


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
                                 "smolvlm": "<fake_token_around_image><global-img><image><fake_token_around_image>"}.get(
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
        if mt in ("qwen2_vl", "qwen2_5_vl", "qwen3_vl", "qwen3_vl_moe"):
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
