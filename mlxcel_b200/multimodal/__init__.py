"""Multimodal glue: media decoding and preprocessing, placeholder expansion, and the wrapper that
pairs a vision tower + connector with the language model's embedding stream
(reference: src/multimodal/ prompt / placeholder / runtime helpers, src/vision/processors/)."""
from .images import ImageProcessor, load_image
from .vlm import VisionLanguage, is_vlm_checkpoint

__all__ = ["ImageProcessor", "load_image", "VisionLanguage", "is_vlm_checkpoint"]
