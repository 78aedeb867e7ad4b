"""Image decoding and preprocessing.

`load_image` accepts what an OpenAI-style ``image_url`` part may carry: a ``data:`` URL, bare base64,
a local path (only below ``media_root`` when one is configured), raw bytes or a PIL image. Remote
``http(s)`` URLs are refused unless the caller allows them: a server that fetches arbitrary URLs on
behalf of its clients is a request-forgery hazard (the reference gates this the same way behind
its media options, src/multimodal/).

`ImageProcessor` reproduces the Hugging Face image processors the supported checkpoints ship with
(``preprocessor_config.json``): resize (shortest edge or fixed size, PIL resampling so results
equal the reference processors bit for bit), centre crop, rescale and normalise.
"""
from __future__ import annotations

import base64
import io
import json
import os
from pathlib import Path

import numpy as np
import torch


def load_image(src, media_root: str | None = None, allow_remote: bool = False):
    from PIL import Image

    if hasattr(src, "convert"):          # PIL image
        return src.convert("RGB")
    if isinstance(src, (bytes, bytearray)):
        return Image.open(io.BytesIO(bytes(src))).convert("RGB")
    if not isinstance(src, str):
        raise ValueError("image must be a data URL, base64 text, a path, bytes or a PIL image")
    if src.startswith("data:"):
        head, _, payload = src.partition(",")
        if ";base64" not in head:
            raise ValueError("data URLs must be base64-encoded")
        return Image.open(io.BytesIO(base64.b64decode(payload))).convert("RGB")
    if src.startswith(("http://", "https://")):
        if not allow_remote:
            raise ValueError("remote image URLs are disabled on this server; send a data: URL")
        import urllib.request
        with urllib.request.urlopen(src, timeout=30) as r:
            return Image.open(io.BytesIO(r.read(64 << 20))).convert("RGB")
    path = src.removeprefix("file://")
    if os.path.exists(path):
        real = os.path.realpath(path)
        if media_root is not None:
            root = os.path.realpath(media_root)
            if os.path.commonpath([real, root]) != root:
                raise ValueError("image path is outside the configured media directory")
        return Image.open(real).convert("RGB")
    try:
        return Image.open(io.BytesIO(base64.b64decode(src, validate=True))).convert("RGB")
    except Exception:
        raise ValueError("image is neither an existing path nor valid base64") from None


_RESAMPLE = {0: "NEAREST", 1: "LANCZOS", 2: "BILINEAR", 3: "BICUBIC", 4: "BOX", 5: "HAMMING"}


class ImageProcessor:
    def __init__(self, cfg: dict | None = None, image_size: int = 224):
        cfg = dict(cfg or {})
        size = cfg.get("size") or {"shortest_edge": image_size}
        if isinstance(size, int):
            size = {"shortest_edge": size}
        self.size = size
        crop = cfg.get("crop_size")
        if isinstance(crop, int):
            crop = {"height": crop, "width": crop}
        self.do_resize = cfg.get("do_resize", True)
        self.do_center_crop = bool(cfg.get("do_center_crop", crop is not None and "shortest_edge" in size))
        self.crop = crop or {"height": image_size, "width": image_size}
        self.resample = int(cfg.get("resample", 3))
        self.do_rescale = cfg.get("do_rescale", True)
        self.rescale = float(cfg.get("rescale_factor", 1 / 255))
        self.do_normalize = cfg.get("do_normalize", True)
        self.mean = [float(x) for x in cfg.get("image_mean", [0.48145466, 0.4578275, 0.40821073])]
        self.std = [float(x) for x in cfg.get("image_std", [0.26862954, 0.26130258, 0.27577711])]

    @staticmethod
    def from_path(path: str | Path, image_size: int = 224) -> "ImageProcessor":
        f = Path(path) / "preprocessor_config.json"
        return ImageProcessor(json.loads(f.read_text()) if f.exists() else None, image_size)

    def _resize(self, img):
        from PIL import Image
        rs = getattr(Image.Resampling, _RESAMPLE.get(self.resample, "BICUBIC"))
        w, h = img.size
        if "shortest_edge" in self.size:
            s = int(self.size["shortest_edge"])
            short, long = (w, h) if w <= h else (h, w)
            new_short, new_long = s, int(s * long / short)
            nw, nh = (new_short, new_long) if w <= h else (new_long, new_short)
        else:
            nh, nw = int(self.size["height"]), int(self.size["width"])
        return img.resize((nw, nh), rs)

    def __call__(self, images: list) -> torch.Tensor:
        """PIL images → float32 [N, 3, H, W]."""
        out = []
        for img in images:
            if self.do_resize:
                img = self._resize(img)
            a = np.asarray(img, dtype=np.float32)            # [H, W, 3]
            if self.do_center_crop:
                ch, cw = int(self.crop["height"]), int(self.crop["width"])
                h, w = a.shape[:2]
                top, left = (h - ch) // 2, (w - cw) // 2
                if top < 0 or left < 0:                       # pad small images symmetrically like the reference
                    ph, pw = max(ch - h, 0), max(cw - w, 0)
                    a = np.pad(a, ((ph // 2, ph - ph // 2), (pw // 2, pw - pw // 2), (0, 0)))
                    h, w = a.shape[:2]
                    top, left = (h - ch) // 2, (w - cw) // 2
                a = a[top:top + ch, left:left + cw]
            if self.do_rescale:
                a = a * self.rescale
            if self.do_normalize:
                a = (a - np.asarray(self.mean, dtype=np.float32)) / np.asarray(self.std, dtype=np.float32)
            out.append(torch.from_numpy(np.ascontiguousarray(a.transpose(2, 0, 1))).float())
        return torch.stack(out)
