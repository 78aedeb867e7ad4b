"""Speech-language checkpoints (Whisper encoder + projector + text decoder) against transformers."""
import tempfile

import pytest
import torch

from mlxcel_b200.config import ModelConfig
from mlxcel_b200.engine.engine import Engine, EngineConfig
from mlxcel_b200.engine.params import SamplingParams
from mlxcel_b200.loading.checkpoint import load_full_weights
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.multimodal.audio_lm import AudioLanguage, is_audio_lm_checkpoint

AUD = 290


def _run(d, ids, mm, chunk=256, n=8):
    cfg = ModelConfig.from_path(d)
    w = load_full_weights(d, cfg, dtype=torch.float32)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=64,
                                                         max_model_len=256, cuda_graphs=False,
                                                         prefill_chunk_alone=chunk, prefill_chunk_contended=chunk))
    sid = eng.add_request(ids, SamplingParams(max_tokens=n, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    return eng.seqs[sid].output


def test_voxtral_greedy_matches_transformers_through_the_engine():
    from transformers import VoxtralConfig, VoxtralForConditionalGeneration
    torch.manual_seed(0)
    cfg = VoxtralConfig(
        audio_config=dict(hidden_size=32, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_mel_bins=16,
                          max_source_positions=20, vocab_size=300),
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         vocab_size=300, max_position_embeddings=256, head_dim=16),
        audio_token_id=AUD)
    m = VoxtralForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="alm_voxtral_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_audio_lm_checkpoint(d)
    al = AudioLanguage.from_checkpoint(d, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    clips = [torch.randn(2, 16, 40, generator=g), torch.randn(1, 16, 40, generator=g)]      # two chunks, one chunk
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [AUD] + text(7) + [AUD] + text(4)
    ids, mm = al.prepare(prompt, clips)
    assert [r.shape[0] for _, r in mm["mm_embeds"]] == [10, 5] and len(ids) == 16 + 15
    assert al.tokens_for(clips[0]) == 10
    with torch.no_grad():
        feats = m.get_audio_features(torch.cat(clips)).pooler_output
    torch.testing.assert_close(torch.cat([r for _, r in mm["mm_embeds"]]), feats, rtol=1e-4, atol=1e-4)
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), input_features=torch.cat(clips), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    assert _run(d, ids, mm) == want
    assert _run(d, ids, mm, chunk=6) == want
    with pytest.raises(ValueError, match="placeholders"):
        al.prepare(prompt, clips[:1])


def test_qwen2_audio_greedy_matches_transformers_through_the_engine():
    from transformers import Qwen2AudioConfig, Qwen2AudioForConditionalGeneration
    torch.manual_seed(0)
    cfg = Qwen2AudioConfig(
        audio_config=dict(d_model=32, encoder_ffn_dim=64, encoder_layers=2, encoder_attention_heads=4, num_mel_bins=16,
                          max_source_positions=20),
        text_config=dict(model_type="qwen2", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=300, max_position_embeddings=256),
        audio_token_index=AUD)
    m = Qwen2AudioForConditionalGeneration(cfg).eval()
    d = tempfile.mkdtemp(prefix="alm_qwen2audio_")
    m.save_pretrained(d, safe_serialization=True)
    assert is_audio_lm_checkpoint(d)
    al = AudioLanguage.from_checkpoint(d, dtype=torch.float32)
    g = torch.Generator().manual_seed(3)
    clips = [torch.randn(1, 16, 40, generator=g), torch.randn(1, 16, 40, generator=g)]
    valid = [40, 27]                                        # the second clip ends inside its chunk
    clips[1][..., valid[1]:] = 0
    for c, v in zip(clips, valid):
        c.valid_frames = v
    text = lambda n: torch.randint(0, 280, (n,), generator=g).tolist()  # noqa: E731
    prompt = text(5) + [AUD] + text(7) + [AUD] + text(4)
    ids, mm = al.prepare(prompt, clips)
    assert [r.shape[0] for _, r in mm["mm_embeds"]] == [10, 7]
    fmask = torch.zeros(2, 40, dtype=torch.long)
    for i, v in enumerate(valid):
        fmask[i, :v] = 1
    with torch.no_grad():
        want = m.generate(input_ids=torch.tensor([ids]), input_features=torch.cat(clips), feature_attention_mask=fmask,
                          attention_mask=torch.ones(1, len(ids), dtype=torch.long), max_new_tokens=8,
                          do_sample=False)[0, len(ids):].tolist()
    assert _run(d, ids, mm) == want
    assert _run(d, ids, mm, chunk=6) == want


def test_input_audio_parts_reach_the_model_through_the_chat_route():
    import base64

    import numpy as np
    from fastapi.testclient import TestClient
    from transformers import VoxtralConfig, VoxtralForConditionalGeneration

    from mlxcel_b200.audio.wav import write_wav
    from mlxcel_b200.server.app import ServerState, create_app
    from mlxcel_b200.server.chat_template import render_chat
    from mlxcel_b200.server.worker import ModelWorker
    from mlxcel_b200.tokenizer import ByteTokenizer
    torch.manual_seed(0)
    cfg = VoxtralConfig(
        audio_config=dict(hidden_size=32, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_mel_bins=16,
                          max_source_positions=20, vocab_size=300),
        text_config=dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         vocab_size=300, max_position_embeddings=512, head_dim=16),
        audio_token_id=AUD)
    d = tempfile.mkdtemp(prefix="alm_voxtral_srv_")
    VoxtralForConditionalGeneration(cfg).eval().save_pretrained(d, safe_serialization=True)
    al = AudioLanguage.from_checkpoint(d, dtype=torch.float32)
    mc = ModelConfig.from_path(d)
    w = load_full_weights(d, mc, dtype=torch.float32)

    class Tok(ByteTokenizer):
        def encode(self, text, add_special_tokens=True):
            out = []
            for i, piece in enumerate(text.split("[AUDIO]")):
                if i:
                    out.append(AUD)
                out += super().encode(piece, add_special_tokens=False)
            return out
    tk = Tok(mc.vocab_size)

    def engine():
        return Engine(DecoderModel(mc, w), mc, EngineConfig(max_batch=2, max_num_batched_tokens=128, num_blocks=64,
                                                            max_model_len=512, cuda_graphs=False))
    # 0.55 s of a tone: two 0.4 s chunks of this tiny encoder (40 frames of 10 ms each)
    samples = (0.3 * np.sin(np.arange(int(0.55 * 16000)) * 2 * np.pi * 440 / 16000)).astype(np.float32)
    wav = base64.b64encode(write_wav(samples, 16000)).decode()
    text = render_chat([{"role": "user", "content": "what is said? [AUDIO]"}], None)
    ids, mm = al.prepare(tk.encode(text), [samples])
    assert sum(1 for t in ids if t == AUD) == 10
    eng = engine()
    sid = eng.add_request(ids, SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True), **mm)
    while eng.has_work():
        eng.step()
    want = tk.decode(eng.seqs[sid].output)
    worker = ModelWorker(engine(), tk, "tiny-voxtral")
    worker.vision = al
    try:
        client = TestClient(create_app(ServerState(worker, tk, "tiny-voxtral")))
        messages = [{"role": "user", "content": [{"type": "text", "text": "what is said? "},
                                                 {"type": "input_audio", "input_audio": {"data": wav, "format": "wav"}}]}]
        r = client.post("/v1/chat/completions", json={"messages": messages, "max_tokens": 6, "temperature": 0, "ignore_eos": True})
        assert r.status_code == 200, r.text
        assert r.json()["choices"][0]["message"]["content"] == want and r.json()["usage"]["prompt_tokens"] == len(ids)
        img = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}]
        assert client.post("/v1/chat/completions", json={"messages": img}).status_code == 400
        bad = [{"role": "user", "content": [{"type": "input_audio", "input_audio": {"data": "!!!", "format": "wav"}}]}]
        assert client.post("/v1/chat/completions", json={"messages": bad}).status_code == 400
    finally:
        worker.shutdown()
