"""Vision-language path on a B200: towers, connectors and the engine's media rows on the CUDA kernels
(bf16) against the same checkpoint on the fp32 CPU path."""
import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")

from mlxcel_b200.config import ModelConfig  # noqa: E402
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams  # noqa: E402
from mlxcel_b200.loading.checkpoint import load_model_weights  # noqa: E402
from mlxcel_b200.models.decoder import DecoderModel  # noqa: E402
from mlxcel_b200.multimodal import VisionLanguage  # noqa: E402


def _run(d, kind, device, dtype):
    import test_vlm_cpu as t
    from mlxcel_b200.multimodal import ImageProcessor
    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    vl = VisionLanguage.from_checkpoint(d, dtype=dtype, device=device)
    if kind == "llava":
        vl.processor = ImageProcessor(dict(size={"shortest_edge": 28}, crop_size={"height": 28, "width": 28}), 28)
        ph = [t.IMG_TOKEN]
    elif kind == "qwen3_vl":
        vl.processor = Qwen2ImageProcessor(dict(min_pixels=64 * 64, max_pixels=32 * 32 * 16, patch_size=16,
                                                image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5]))
        ph = [292, t.IMG_TOKEN, 293]
    else:
        vl.processor = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16))
        ph = [292, t.IMG_TOKEN, 293]
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + ph + text(7) + ph + text(4)
    ids, mm = vl.prepare(prompt, [t._image(5, 90, 61), t._image(6, 50, 130)])
    cfg = ModelConfig.from_path(d)
    w = load_model_weights(d, cfg, device=device) if device != "cpu" else __import__(
        "mlxcel_b200.loading.checkpoint", fromlist=["load_full_weights"]).load_full_weights(d, cfg, dtype=dtype)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32,
                                                         max_model_len=256, cuda_graphs=device != "cpu",
                                                         prefill_chunk_alone=24, prefill_chunk_contended=24))
    sid = eng.add_request(ids, SamplingParams(max_tokens=12, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    rows = torch.cat([r.float().cpu() for _, r in mm["mm_embeds"]])
    return eng.seqs[sid].output, rows


@pytest.mark.parametrize("kind", ["llava", "qwen2_vl", "qwen3_vl"])
def test_vlm_gpu_matches_cpu(kind):
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).parent))
    import test_vlm_cpu as t
    # head size 64 (what the paged attention kernels serve)
    m, d = (t._tiny_llava(128, 2, 1) if kind == "llava" else t._tiny_qwen3_vl(128, 2, 1, 64, (12, 10, 10)) if kind == "qwen3_vl"
            else t._tiny_qwen2_vl(128, 2, 1, (8, 12, 12)))
    want, rows_cpu = _run(d, kind, "cpu", torch.float32)
    got, rows_gpu = _run(d, kind, "cuda", torch.bfloat16)
    # connector output: bf16 operands, fp32 accumulation
    err = (rows_gpu - rows_cpu).abs().max().item()
    assert err < 0.06 * max(rows_cpu.abs().max().item(), 1.0), err
    agree = sum(a == b for a, b in zip(got, want)) / len(want)
    assert got[0] == want[0] and agree >= 0.5, (got, want)
