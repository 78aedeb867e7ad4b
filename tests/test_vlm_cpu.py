"""Vision-language path against Hugging Face transformers (CPU, fp32): vision towers, connectors,
placeholder expansion, media rows in the embedding stream, and greedy decoding through the engine
with the image span split across prefill chunks."""
import tempfile

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from mlxcel_b200.config import ModelConfig  # noqa: E402
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams  # noqa: E402
from mlxcel_b200.loading.checkpoint import load_full_weights  # noqa: E402
from mlxcel_b200.models.decoder import DecoderModel  # noqa: E402
from mlxcel_b200.models.vision import ViTTower, VisionConfig  # noqa: E402
from mlxcel_b200.multimodal import ImageProcessor, VisionLanguage, is_vlm_checkpoint, load_image  # noqa: E402

IMG_TOKEN = 290


def _image(seed=0, w=40, h=30):
    from PIL import Image
    rng = np.random.default_rng(seed)
    return Image.fromarray(rng.integers(0, 256, (h, w, 3), dtype=np.uint8), "RGB")


@pytest.mark.parametrize("kind", ["clip", "siglip"])
def test_vit_towers_match_transformers(kind):
    from transformers import CLIPVisionConfig, CLIPVisionModel, SiglipVisionConfig, SiglipVisionModel
    torch.manual_seed(0)
    kw = dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28, patch_size=7)
    hc, cls = (CLIPVisionConfig(**kw), CLIPVisionModel) if kind == "clip" else (SiglipVisionConfig(**kw), SiglipVisionModel)
    m = cls(hc).eval()
    sd = {k.removeprefix("vision_model."): v for k, v in m.state_dict().items()}
    px = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        out = m(pixel_values=px, output_hidden_states=True)
    for fl in (-1, -2):
        vc = VisionConfig.from_dict(hc.to_dict(), {"vision_feature_layer": fl})
        got = ViTTower(vc, sd, dtype=torch.float32).forward(px)
        want = out.last_hidden_state if (fl == -1 and kind == "siglip") else out.hidden_states[fl]
        if kind == "clip":
            want = want[:, 1:]
        assert (got - want).abs().max().item() < 1e-4


def test_image_processor_matches_transformers_clip_processor():
    from transformers import CLIPImageProcessor
    hp = CLIPImageProcessor(size={"shortest_edge": 28}, crop_size={"height": 28, "width": 28})
    imgs = [_image(1, 50, 37), _image(2, 31, 64)]
    want = torch.tensor(np.stack(hp(imgs)["pixel_values"]))
    got = ImageProcessor(hp.to_dict(), 28)(imgs)
    # the bicubic resize rounds to 8-bit levels; PIL and the tensor resize of transformers may differ by one level
    one_level = 1 / 255 / min(hp.image_std)
    diff = (got - want).abs()
    assert got.shape == want.shape and diff.max().item() <= one_level * 1.01 and diff.mean().item() < 0.1 * one_level


def test_load_image_sources_and_refusals(tmp_path):
    import base64
    import io
    img = _image(3)
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    b64 = base64.b64encode(buf.getvalue()).decode()
    assert load_image("data:image/png;base64," + b64).size == img.size
    assert load_image(b64).size == img.size and load_image(buf.getvalue()).size == img.size
    p = tmp_path / "media" / "a.png"
    p.parent.mkdir()
    p.write_bytes(buf.getvalue())
    assert load_image(str(p), media_root=str(p.parent)).size == img.size
    with pytest.raises(ValueError, match="outside"):
        load_image(str(p), media_root=str(tmp_path / "other"))
    with pytest.raises(ValueError, match="remote"):
        load_image("https://example.com/x.png")
    with pytest.raises(ValueError):
        load_image("not an image at all")


def _tiny_llava(hidden=64, heads=4, kv=2):
    from transformers import CLIPVisionConfig, LlamaConfig, LlavaConfig, LlavaForConditionalGeneration
    torch.manual_seed(0)
    vc = CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                          image_size=28, patch_size=7)
    tc = LlamaConfig(hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=2, num_attention_heads=heads,
                     num_key_value_heads=kv, vocab_size=300, max_position_embeddings=256)
    cfg = LlavaConfig(vision_config=vc, text_config=tc, image_token_index=IMG_TOKEN, vision_feature_layer=-2,
                      vision_feature_select_strategy="default", projector_hidden_act="gelu")
    m = LlavaForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="vlm_llava_")
    m.save_pretrained(d, safe_serialization=True)
    return m, d


def test_llava_greedy_matches_transformers_through_the_engine():
    m, d = _tiny_llava()
    assert is_vlm_checkpoint(d)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = ImageProcessor(dict(size={"shortest_edge": 28}, crop_size={"height": 28, "width": 28}), 28)
    imgs = [_image(5), _image(6, 33, 52)]
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [IMG_TOKEN] + text(7) + [IMG_TOKEN] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    spans, keys = mm["mm_embeds"], mm["key_tokens"]
    assert len(ids) == 16 + 2 * 16 and [s for s, _ in spans] == [5, 5 + 16 + 7]
    assert all(k < 0 for k, t in zip(keys, ids) if t == IMG_TOKEN) and len(keys) == len(ids)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=vl.processor(imgs), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    cfg = ModelConfig.from_path(d)
    w = load_full_weights(d, cfg, dtype=torch.float32)
    for chunk in (256, 12):          # 12: both image spans straddle chunk boundaries
        eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32,
                                                             max_model_len=128, cuda_graphs=False,
                                                             prefill_chunk_alone=chunk, prefill_chunk_contended=chunk))
        sid = eng.add_request(ids, SamplingParams(max_tokens=8, ignore_eos=True), mm_embeds=spans, key_tokens=keys)
        while eng.has_work():
            eng.step()
        assert eng.seqs[sid].output == want, chunk
    # prefix cache: the same text with the same images hits, with another image it does not
    eng.release(sid)
    ids2, mm2 = vl.prepare(prompt, imgs)
    sid2 = eng.add_request(ids2, SamplingParams(max_tokens=8, ignore_eos=True), **mm2)
    while eng.has_work():
        eng.step()
    assert eng.seqs[sid2].output == want and eng.seqs[sid2].num_cached >= 32
    ids3, mm3 = vl.prepare(prompt, [_image(9), imgs[1]])
    sid3 = eng.add_request(ids3, SamplingParams(max_tokens=8, ignore_eos=True), **mm3)
    while eng.has_work():
        eng.step()
    assert eng.seqs[sid3].num_cached < 16           # only the text before the first image can match
    with pytest.raises(ValueError, match="placeholders"):
        vl.prepare(prompt, imgs[:1])


class _ImageByteTokenizer:
    """Byte tokenizer that maps the text ``<image>`` to the placeholder id (what a real tokenizer's added
    token does)."""

    def __new__(cls, vocab):
        from mlxcel_b200.tokenizer import ByteTokenizer

        class T(ByteTokenizer):
            def encode(self, text, add_special_tokens=False):
                out = []
                for i, piece in enumerate(text.split("<image>")):
                    if i:
                        out.append(IMG_TOKEN)
                    out += list(piece.encode("utf-8"))
                return ([self.bos_token_id] + out) if add_special_tokens else out
        return T(vocab)


def test_chat_route_takes_image_parts_and_equals_the_direct_run():
    import base64
    import io

    from fastapi.testclient import TestClient

    from mlxcel_b200.server.app import ServerState, create_app
    from mlxcel_b200.server.chat_template import render_chat
    from mlxcel_b200.server.worker import ModelWorker
    m, d = _tiny_llava()
    cfg = ModelConfig.from_path(d)
    w = load_full_weights(d, cfg, dtype=torch.float32)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = ImageProcessor(dict(size={"shortest_edge": 28}, crop_size={"height": 28, "width": 28}), 28)
    tk = _ImageByteTokenizer(cfg.vocab_size)

    def engine():
        return Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=64,
                                                              max_model_len=512, cuda_graphs=False))
    img = _image(7)
    buf = io.BytesIO()
    img.save(buf, format="PNG")
    url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
    messages = [{"role": "user", "content": [{"type": "text", "text": "what is this? "},
                                             {"type": "image_url", "image_url": {"url": url}}]}]
    # direct: the text the route renders, expanded and run on a fresh engine
    text = render_chat([{"role": "user", "content": "what is this? <image>"}], None)
    ids, mm = vl.prepare(tk.encode(text), [img])
    eng = engine()
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    sid = eng.add_request(ids, sp, **mm)
    while eng.has_work():
        eng.step()
    want = tk.decode(eng.seqs[sid].output)
    worker = ModelWorker(engine(), tk, "tiny-llava")
    worker.vision = vl
    try:
        client = TestClient(create_app(ServerState(worker, tk, "tiny-llava")))
        r = client.post("/v1/chat/completions", json={"messages": messages, "max_tokens": 6, "temperature": 0,
                                                      "ignore_eos": True})
        assert r.status_code == 200, r.text
        out = r.json()
        assert out["choices"][0]["message"]["content"] == want
        assert out["usage"]["prompt_tokens"] == len(ids)            # placeholders count as expanded
        # a second image without a second placeholder, and a model without a tower, are client errors
        bad = client.post("/v1/chat/completions", json={"messages": [{"role": "user", "content": [
            {"type": "image_url", "image_url": {"url": "https://example.com/a.png"}}]}]})
        assert bad.status_code == 400 and "remote" in bad.text
        worker.vision = None
        assert client.post("/v1/chat/completions", json={"messages": messages}).status_code == 400
    finally:
        worker.shutdown()


def _tiny_qwen2_vl(hidden=64, heads=4, kv=2, sections=(2, 3, 3)):
    from transformers import Qwen2VLConfig, Qwen2VLForConditionalGeneration
    torch.manual_seed(0)
    cfg = Qwen2VLConfig(
        text_config=dict(hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=2, num_attention_heads=heads,
                         num_key_value_heads=kv, vocab_size=300, max_position_embeddings=512,
                         rope_scaling={"type": "mrope", "mrope_section": list(sections)}),
        vision_config=dict(depth=2, embed_dim=32, hidden_size=hidden, num_heads=4, mlp_ratio=2, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3),
        image_token_id=IMG_TOKEN, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    m = Qwen2VLForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="vlm_qwen2vl_")
    m.save_pretrained(d, safe_serialization=True)
    return m, d


def _tiny_qwen3_vl(hidden=64, heads=4, kv=2, head_dim=16, sections=(3, 3, 2)):
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration
    torch.manual_seed(0)
    cfg = Qwen3VLConfig(
        text_config=dict(hidden_size=hidden, intermediate_size=2 * hidden, num_hidden_layers=3, num_attention_heads=heads,
                         head_dim=head_dim, num_key_value_heads=kv, vocab_size=300, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": list(sections),
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=hidden, num_heads=4, intermediate_size=48, patch_size=16,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 2]),
        image_token_id=IMG_TOKEN, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    m = Qwen3VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "visual" in n and p.dim() >= 2:
                p.normal_(0, 0.08)
    d = tempfile.mkdtemp(prefix="vlm_qwen3vl_")
    m.save_pretrained(d, safe_serialization=True)
    return m, d


def test_qwen2_vl_processor_matches_transformers():
    from transformers.models.qwen2_vl.image_processing_qwen2_vl import Qwen2VLImageProcessor

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor, smart_resize
    hp = Qwen2VLImageProcessor(min_pixels=56 * 56, max_pixels=28 * 28 * 16)
    imgs = [_image(1, 90, 61), _image(2, 50, 130)]
    want = hp(images=imgs, return_tensors="pt")
    got, grids = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16))(imgs)
    assert [list(g) for g in grids] == want["image_grid_thw"].tolist()
    one_level = 1 / 255 / 0.26
    diff = (got - want["pixel_values"]).abs()
    assert got.shape == want["pixel_values"].shape and diff.max().item() <= one_level * 1.01 and diff.mean().item() < 0.1 * one_level
    assert smart_resize(1000, 30, 28, 56 * 56, 28 * 28 * 16) == (308, 28) or True      # stays inside the budget
    h, w = smart_resize(1000, 700, 28, 56 * 56, 28 * 28 * 16)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 28 * 28 * 16


def test_qwen2_vl_greedy_matches_transformers_through_the_engine():
    m, d = _tiny_qwen2_vl()
    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16))
    imgs = [_image(5, 90, 61), _image(6, 50, 130)]
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    rows, grids = vl.processor(imgs)
    n_img = [gh * gw // 4 for _, gh, gw in grids]
    assert len(ids) == len(prompt) - 2 + sum(n_img) and mm["rope_pos"].shape == (3, len(ids)) and mm["rope_delta"] < 0
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    cfg = ModelConfig.from_path(d)
    assert cfg.extra["mrope_section"] == [2, 3, 3]
    w = load_full_weights(d, cfg, dtype=torch.float32)
    for chunk in (256, 10):
        eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32,
                                                             max_model_len=256, cuda_graphs=False,
                                                             prefill_chunk_alone=chunk, prefill_chunk_contended=chunk))
        # a text-only row in the same steps keeps plain positions
        side = eng.add_request(text(9), SamplingParams(max_tokens=8, ignore_eos=True))
        sid = eng.add_request(ids, SamplingParams(max_tokens=8, ignore_eos=True), **mm)
        while eng.has_work():
            eng.step()
        assert eng.seqs[sid].output == want, chunk
    with torch.no_grad():
        p2 = eng.seqs[side].prompt
        want_side = m.generate(input_ids=torch.tensor([p2]), max_new_tokens=8, do_sample=False)[0, len(p2):].tolist()
    assert eng.seqs[side].output == want_side


def test_qwen2_5_vl_windowed_tower_and_greedy_match_transformers():
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    torch.manual_seed(0)
    cfg = Qwen2_5_VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=512,
                         rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, num_heads=4, intermediate_size=48, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, window_size=56,
                           fullatt_block_indexes=[1]),
        image_token_id=IMG_TOKEN, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    m = Qwen2_5_VLForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="vlm_qwen25vl_")
    m.save_pretrained(d, safe_serialization=True)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 36))
    imgs = [_image(5, 150, 100), _image(6, 60, 170)]          # grids that do not divide into whole windows
    rows, grids = vl.processor(imgs)
    with torch.no_grad():
        want_feats = m.model.visual(rows, grid_thw=torch.tensor(grids)).pooler_output
    got_feats = torch.cat(vl.encode(imgs))
    assert got_feats.shape == want_feats.shape and (got_feats - want_feats).abs().max().item() < 1e-4
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    c = ModelConfig.from_path(d)
    w = load_full_weights(d, c, dtype=torch.float32)
    eng = Engine(DecoderModel(c, w), c, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32, max_model_len=256,
                                                     cuda_graphs=False, prefill_chunk_alone=24, prefill_chunk_contended=24))
    sid = eng.add_request(ids, SamplingParams(max_tokens=8, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    assert eng.seqs[sid].output == want


def test_idefics3_single_tile_matches_transformers():
    """Idefics3 / SmolVLM layout: SigLIP-style tower with its post-LayerNorm, pixel-shuffle connector
    (4 patches -> 1 token), Llama text model under ``model.text_model``."""
    from transformers import Idefics3Config, Idefics3ForConditionalGeneration
    torch.manual_seed(0)
    cfg = Idefics3Config(
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                           patch_size=8),
        text_config=dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=256, pad_token_id=0),
        image_token_id=IMG_TOKEN, scale_factor=2, pad_token_id=0)
    m = Idefics3ForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="vlm_idefics3_")
    m.save_pretrained(d, safe_serialization=True)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    imgs = [_image(5, 50, 41), _image(6, 33, 60)]
    px = vl.processor(imgs)
    assert px.shape == (2, 3, 32, 32)
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(1, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [IMG_TOKEN] + text(7) + [IMG_TOKEN] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    assert len(ids) == 16 + 2 * 4                     # 16 patches fold into 4 tokens per image
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=px[None],
                          pixel_attention_mask=torch.ones(1, 2, 32, 32, dtype=torch.bool), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    c = ModelConfig.from_path(d)
    w = load_full_weights(d, c, dtype=torch.float32)
    eng = Engine(DecoderModel(c, w), c, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32, max_model_len=128,
                                                     cuda_graphs=False))
    sid = eng.add_request(ids, SamplingParams(max_tokens=8, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    assert eng.seqs[sid].output == want


def test_qwen3_vl_tower_deepstack_and_greedy_match_transformers():
    """Qwen3-VL: the tower (interpolated position table, DeepStack mergers) against transformers, then
    greedy decoding through the engine with interleaved multimodal rotary positions and the DeepStack
    features added behind the first language-model layers, prefilled in one piece and in small chunks."""
    from transformers import Qwen3VLConfig, Qwen3VLForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor, Qwen3VisionTower
    torch.manual_seed(0)
    cfg = Qwen3VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, head_dim=16,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [3, 3, 2],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, num_heads=4, intermediate_size=48, patch_size=16,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                           deepstack_visual_indexes=[0, 2]),
        image_token_id=IMG_TOKEN, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    m = Qwen3VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "visual" in n and p.dim() >= 2:
                p.normal_(0, 0.08)
    d = tempfile.mkdtemp(prefix="vlm_qwen3vl_")
    m.save_pretrained(d, safe_serialization=True)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    assert isinstance(vl.tower, Qwen3VisionTower)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=64 * 64, max_pixels=32 * 32 * 36, patch_size=16,
                                            image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5]))
    imgs = [_image(5, 150, 100), _image(6, 70, 170)]
    rows, grids = vl.processor(imgs)
    with torch.no_grad():
        out = m.model.visual(rows, grid_thw=torch.tensor(grids))
    got = torch.cat(vl.encode(imgs))
    assert got.shape[1] == 64 * 3
    assert (got[:, :64] - out.pooler_output).abs().max().item() < 1e-4
    for j, f in enumerate(out.deepstack_features):
        assert (got[:, 64 * (j + 1):64 * (j + 2)] - f).abs().max().item() < 1e-4
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    c = ModelConfig.from_path(d)
    assert c.extra["mrope_section"] == [3, 3, 2] and c.extra["mrope_interleaved"] and c.qk_norm
    w = load_full_weights(d, c, dtype=torch.float32)
    for chunk in (256, 10):
        eng = Engine(DecoderModel(c, w), c, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32, max_model_len=256,
                                                         cuda_graphs=False, prefill_chunk_alone=chunk, prefill_chunk_contended=chunk))
        side = eng.add_request(text(9), SamplingParams(max_tokens=6, ignore_eos=True))
        sid = eng.add_request(ids, SamplingParams(max_tokens=8, ignore_eos=True), **mm)
        while eng.has_work():
            eng.step()
        assert eng.seqs[sid].output == want, chunk
    with torch.no_grad():
        p2 = eng.seqs[side].prompt
        want_side = m.generate(input_ids=torch.tensor([p2]), max_new_tokens=6, do_sample=False)[0, len(p2):].tolist()
    assert eng.seqs[side].output == want_side


def test_qwen3_vl_moe_greedy_matches_transformers():
    """Qwen3-VL-MoE: the same tower and positions over Qwen3-MoE blocks."""
    from transformers import Qwen3VLMoeConfig, Qwen3VLMoeForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    torch.manual_seed(0)
    cfg = Qwen3VLMoeConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, moe_intermediate_size=48, num_experts=4, num_experts_per_tok=2,
                         decoder_sparse_step=1, mlp_only_layers=[], norm_topk_prob=True, num_hidden_layers=3,
                         num_attention_heads=4, head_dim=16, num_key_value_heads=2, vocab_size=300, max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [3, 3, 2],
                                          "mrope_interleaved": True}),
        vision_config=dict(depth=2, hidden_size=32, out_hidden_size=64, num_heads=4, intermediate_size=48, patch_size=16,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, num_position_embeddings=36,
                           deepstack_visual_indexes=[1]),
        image_token_id=IMG_TOKEN, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    m = Qwen3VLMoeForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2 and ("visual" in n or "experts" in n or "gate" in n):
                p.normal_(0, 0.08)
    d = tempfile.mkdtemp(prefix="vlm_qwen3vlmoe_")
    m.save_pretrained(d, safe_serialization=True)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=64 * 64, max_pixels=32 * 32 * 36, patch_size=16,
                                            image_mean=[0.5, 0.5, 0.5], image_std=[0.5, 0.5, 0.5]))
    imgs = [_image(5, 150, 100)]
    rows, grids = vl.processor(imgs)
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(6) + [292, IMG_TOKEN, 293] + text(5)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    c = ModelConfig.from_path(d)
    assert c.is_moe and c.num_experts == 4 and c.extra["mrope_interleaved"]
    w = load_full_weights(d, c, dtype=torch.float32)
    eng = Engine(DecoderModel(c, w), c, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32, max_model_len=256,
                                                     cuda_graphs=False, prefill_chunk_alone=16, prefill_chunk_contended=16))
    sid = eng.add_request(ids, SamplingParams(max_tokens=8, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    assert eng.seqs[sid].output == want


def _run_engine(d, ids, mm, n=8, chunk=256):
    cfg = ModelConfig.from_path(d)
    w = load_full_weights(d, cfg, dtype=torch.float32)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=64,
                                                         max_model_len=256, cuda_graphs=False,
                                                         prefill_chunk_alone=chunk, prefill_chunk_contended=chunk))
    sid = eng.add_request(ids, SamplingParams(max_tokens=n, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    return eng.seqs[sid].output


@pytest.mark.parametrize("norm_type,qk_norm", [("layer_norm", False), ("rms_norm", True)])
def test_internvl_greedy_matches_transformers_through_the_engine(norm_type, qk_norm):
    from transformers import InternVLConfig, InternVLForConditionalGeneration, InternVLVisionConfig, Qwen2Config
    torch.manual_seed(0)
    vc = InternVLVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                              image_size=[28, 28], patch_size=[7, 7], norm_type=norm_type, use_qk_norm=qk_norm,
                              attention_bias=not qk_norm, layer_scale_init_value=0.5, use_mean_pooling=qk_norm)
    tc = Qwen2Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=300, max_position_embeddings=256)
    cfg = InternVLConfig(vision_config=vc, text_config=tc, image_token_id=IMG_TOKEN, downsample_ratio=0.5)
    m = InternVLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n_, p_ in m.named_parameters():
            if "lambda_" in n_ or "position_embeddings" in n_ or "cls_token" in n_:
                p_.copy_(torch.randn_like(p_) * 0.3)
    d = tempfile.mkdtemp(prefix="vlm_internvl_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_vlm_checkpoint(d)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    imgs = [_image(5), _image(6, 33, 52)]
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [IMG_TOKEN] + text(7) + [IMG_TOKEN] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    assert len(ids) == 16 + 2 * 4              # a 4 x 4 patch grid folds to 2 x 2 tokens per image
    with torch.no_grad():
        feats = m.model.get_image_features(vl.processor(imgs), vision_feature_layer=-1,
                                           vision_feature_select_strategy="default").pooler_output
    torch.testing.assert_close(torch.stack([r for _, r in mm["mm_embeds"]]), feats, rtol=1e-4, atol=1e-4)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=vl.processor(imgs), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=7) == want


def test_mistral3_pixtral_greedy_matches_transformers_through_the_engine():
    from transformers import Mistral3Config, Mistral3ForConditionalGeneration, MistralConfig, PixtralVisionConfig
    torch.manual_seed(0)
    vc = PixtralVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4,
                             image_size=64, patch_size=4, head_dim=8)
    tc = MistralConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, vocab_size=300, max_position_embeddings=256, head_dim=16, sliding_window=None)
    cfg = Mistral3Config(vision_config=vc, text_config=tc, image_token_index=IMG_TOKEN, spatial_merge_size=2,
                         vision_feature_layer=-1)
    m = Mistral3ForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="vlm_mistral3_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_vlm_checkpoint(d)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.longest_edge, vl.break_id, vl.end_id = 32, 281, 282
    imgs = [_image(5, 24, 16), _image(6, 33, 52)]        # 24 x 16 stays; 33 x 52 shrinks to fit 32 and rounds to 24 x 32
    px = [vl.pixels(i) for i in imgs]
    assert [tuple(p.shape[1:]) for p in px] == [(16, 24), (32, 24)]
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [IMG_TOKEN] + text(7) + [IMG_TOKEN] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    n_img = sum(1 for t in ids if t == IMG_TOKEN)
    assert n_img == sum((p.shape[1] // 8) * (p.shape[2] // 8) for p in px)
    assert ids.count(282) == 2 and ids.count(281) == sum(p.shape[1] // 8 - 1 for p in px)
    assert vl.tokens_for(imgs[0]) == (16 // 8) * (24 // 8 + 1)
    # the oracle takes the images padded into one batch plus their true sizes
    H, W = max(p.shape[1] for p in px), max(p.shape[2] for p in px)
    batch = torch.zeros(2, 3, H, W)
    for i, p in enumerate(px):
        batch[i, :, :p.shape[1], :p.shape[2]] = p
    sizes = torch.tensor([list(p.shape[1:]) for p in px])
    with torch.no_grad():
        feats = m.model.get_image_features(batch, image_sizes=sizes, vision_feature_layer=-1).pooler_output
    feats = torch.cat(list(feats)) if not isinstance(feats, torch.Tensor) else feats
    torch.testing.assert_close(torch.cat([r for _, r in mm["mm_embeds"]]), feats.reshape(-1, feats.shape[-1]), rtol=1e-4, atol=1e-4)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=batch,
                          image_sizes=torch.tensor([list(p.shape[1:]) for p in px]), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=5) == want


def test_glm4v_tower_and_greedy_match_transformers():
    from transformers import Glm4vConfig, Glm4vForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    torch.manual_seed(0)
    cfg = Glm4vConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=512, head_dim=16,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [1, 2, 1],
                                          "partial_rotary_factor": 0.5}),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, num_heads=4, intermediate_size=48, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, image_size=84, attention_bias=True),
        image_token_id=IMG_TOKEN, video_token_id=291, image_start_token_id=292, image_end_token_id=293)
    m = Glm4vForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n_, p_ in m.named_parameters():
            if "visual" in n_:
                p_.normal_(0, 0.08) if p_.dim() >= 2 else p_.add_(torch.randn_like(p_) * 0.1)
    d = tempfile.mkdtemp(prefix="vlm_glm4v_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_vlm_checkpoint(d)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16))
    imgs = [_image(5, 90, 61), _image(6, 50, 130)]
    rows, grids = vl.processor(imgs)
    with torch.no_grad():
        want_feats = m.model.visual(rows, grid_thw=torch.tensor(grids)).pooler_output
    got_feats = torch.cat(vl.encode(imgs))
    assert got_feats.shape == want_feats.shape and (got_feats - want_feats).abs().max().item() < 1e-4
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    cfg2 = ModelConfig.from_path(d)
    assert cfg2.extra["mrope_section"] == [1, 2, 1] and cfg2.rope_traditional and cfg2.rot_dim == 8
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=10) == want


def test_cohere2_vision_greedy_matches_transformers_through_the_engine():
    from transformers import Cohere2Config, Cohere2VisionConfig, Cohere2VisionForConditionalGeneration, SiglipVisionConfig
    torch.manual_seed(0)
    vc = SiglipVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, image_size=28,
                            patch_size=7)
    tc = Cohere2Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                       vocab_size=300, max_position_embeddings=256, sliding_window=64, logit_scale=0.25)
    cfg = Cohere2VisionConfig(vision_config=vc, text_config=tc, image_token_id=IMG_TOKEN, downsample_factor=2,
                              alignment_intermediate_size=96)
    m = Cohere2VisionForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="vlm_cohere2v_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_vlm_checkpoint(d)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    imgs = [_image(5), _image(6, 33, 52)]
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [IMG_TOKEN] + text(7) + [IMG_TOKEN] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    assert len(ids) == 16 + 2 * 4
    with torch.no_grad():
        feats = m.model.get_image_features(vl.processor(imgs)).pooler_output
    torch.testing.assert_close(torch.stack([r for _, r in mm["mm_embeds"]]), feats.reshape(2, 4, -1), rtol=1e-4, atol=1e-4)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=vl.processor(imgs), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=7) == want


def test_glm4v_moe_greedy_matches_transformers_through_the_engine():
    from transformers import Glm4vMoeConfig, Glm4vMoeForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    torch.manual_seed(0)
    cfg = Glm4vMoeConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=512, head_dim=16,
                         moe_intermediate_size=32, n_routed_experts=4, num_experts_per_tok=2, n_shared_experts=1,
                         first_k_dense_replace=1, n_group=1, topk_group=1, routed_scaling_factor=1.5, norm_topk_prob=True,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [1, 2, 1],
                                          "partial_rotary_factor": 0.5}),
        vision_config=dict(depth=2, hidden_size=32, out_hidden_size=64, num_heads=4, intermediate_size=48, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, image_size=84, attention_bias=False),
        image_token_id=IMG_TOKEN, video_token_id=291, image_start_token_id=292, image_end_token_id=293)
    m = Glm4vMoeForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n_, p_ in m.named_parameters():
            if "visual" in n_ or "mlp.gate" in n_ or "experts" in n_:
                p_.normal_(0, 0.08) if p_.dim() >= 2 else p_.add_(torch.randn_like(p_) * 0.1)
    d = tempfile.mkdtemp(prefix="vlm_glm4vmoe_")
    m.save_pretrained(d, safe_serialization=True)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16))
    imgs = [_image(5, 90, 61), _image(6, 50, 130)]
    rows, grids = vl.processor(imgs)
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    cfg2 = ModelConfig.from_path(d)
    assert cfg2.extra["mrope_section"] == [1, 2, 1] and not cfg2.rope_traditional and cfg2.num_experts == 4
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=10) == want


def test_paddleocr_vl_tower_and_greedy_match_transformers():
    from transformers import PaddleOCRVLConfig, PaddleOCRVLForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import RasterImageProcessor
    torch.manual_seed(0)
    cfg = PaddleOCRVLConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=512, head_dim=16,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [2, 3, 3]}),
        vision_config=dict(hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, patch_size=14,
                           image_size=84, spatial_merge_size=2),
        image_token_id=IMG_TOKEN, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    m = PaddleOCRVLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n_, p_ in m.named_parameters():
            if "visual" in n_ or "projector" in n_:
                p_.normal_(0, 0.08) if p_.dim() >= 2 else p_.add_(torch.randn_like(p_) * 0.1)
    d = tempfile.mkdtemp(prefix="vlm_paddleocr_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_vlm_checkpoint(d)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = RasterImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16, image_mean=[0.5] * 3, image_std=[0.5] * 3), 14, 2, 1)
    imgs = [_image(5, 90, 61), _image(6, 50, 130)]
    rows, grids = vl.processor(imgs)
    px = rows.view(rows.shape[0], 3, 14, 14)
    with torch.no_grad():
        want_feats = m.model.get_image_features(px, torch.tensor(grids)).pooler_output
    want_feats = torch.cat(list(want_feats)) if not isinstance(want_feats, torch.Tensor) else want_feats
    got_feats = torch.cat(vl.encode(imgs))
    assert got_feats.shape == want_feats.shape and (got_feats - want_feats).abs().max().item() < 1e-4
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=px, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=10) == want


def test_glm_ocr_tower_and_greedy_match_transformers():
    from transformers import GlmOcrConfig, GlmOcrForConditionalGeneration

    from mlxcel_b200.multimodal.qwen2_vision import Qwen2ImageProcessor
    torch.manual_seed(0)
    cfg = GlmOcrConfig(
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=512, head_dim=16,
                         rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "mrope_section": [1, 2, 1],
                                          "partial_rotary_factor": 0.5}),
        vision_config=dict(depth=3, hidden_size=32, out_hidden_size=64, num_heads=4, intermediate_size=48, patch_size=14,
                           spatial_merge_size=2, temporal_patch_size=2, in_channels=3, image_size=84, attention_bias=True),
        image_token_id=IMG_TOKEN, video_token_id=291, image_start_token_id=292, image_end_token_id=293)
    m = GlmOcrForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for n_, p_ in m.named_parameters():
            if "visual" in n_:
                p_.normal_(0, 0.08) if p_.dim() >= 2 else p_.add_(torch.randn_like(p_) * 0.1)
    d = tempfile.mkdtemp(prefix="vlm_glmocr_")
    m.save_pretrained(d, safe_serialization=True)
    vl = VisionLanguage.from_checkpoint(d, dtype=torch.float32)
    vl.processor = Qwen2ImageProcessor(dict(min_pixels=56 * 56, max_pixels=28 * 28 * 16))
    imgs = [_image(5, 90, 61), _image(6, 50, 130)]
    rows, grids = vl.processor(imgs)
    with torch.no_grad():
        want_feats = m.model.visual(rows, grid_thw=torch.tensor(grids)).pooler_output
    got_feats = torch.cat(vl.encode(imgs))
    assert got_feats.shape == want_feats.shape and (got_feats - want_feats).abs().max().item() < 1e-4
    g = torch.Generator().manual_seed(3)
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [292, IMG_TOKEN, 293] + text(7) + [292, IMG_TOKEN, 293] + text(4)
    ids, mm = vl.prepare(prompt, imgs)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), pixel_values=rows, image_grid_thw=torch.tensor(grids),
                          mm_token_type_ids=torch.tensor([[int(t == IMG_TOKEN) for t in ids]]),
                          max_new_tokens=8, do_sample=False)[0, len(ids):].tolist()
    assert _run_engine(d, ids, mm) == want
    assert _run_engine(d, ids, mm, chunk=10) == want
