"""Speech-to-text: WAV decoding, log-mel features, the Whisper encoder / decoder against transformers,
the chunked transcription driver and the OpenAI audio routes (CPU, fp32, tiny random model)."""
import io
import json
import tempfile

import numpy as np
import pytest
import torch

transformers = pytest.importorskip("transformers")

from mlxcel_b200.audio import LogMel, decode_audio, read_wav, resample, write_wav  # noqa: E402
from mlxcel_b200.audio.transcribe import Transcriber, is_whisper_checkpoint  # noqa: E402
from mlxcel_b200.models.whisper import WhisperModel  # noqa: E402

SOT, EOS, EN, FR, TRANSCRIBE, TRANSLATE, NOTS = 390, 391, 380, 381, 382, 383, 384


def _tone(seconds=1.0, sr=16000, f=440.0, seed=0):
    t = np.arange(int(seconds * sr)) / sr
    rng = np.random.default_rng(seed)
    return (0.3 * np.sin(2 * np.pi * f * t) + 0.02 * rng.standard_normal(t.size)).astype(np.float32)


def test_wav_round_trip_formats_and_resampling():
    x = _tone(0.25)
    y, sr = read_wav(write_wav(x, 16000))
    assert sr == 16000 and np.abs(y - x).max() < 1e-4
    # stereo float32 at 44.1 kHz through the extensible header path
    import struct
    st = np.stack([x, x], axis=1).astype("<f4").tobytes()
    hdr = b"RIFF" + struct.pack("<I", 36 + len(st)) + b"WAVE" + b"fmt " + struct.pack("<IHHIIHH", 16, 3, 2, 44100, 44100 * 8, 8, 32)
    y2, sr2 = read_wav(hdr + b"data" + struct.pack("<I", len(st)) + st)
    assert sr2 == 44100 and np.abs(y2 - x).max() < 1e-6
    assert abs(len(resample(y2, 44100, 16000)) - round(len(x) * 16000 / 44100)) <= 1
    assert decode_audio(write_wav(x, 8000)).shape[0] == 2 * len(x)
    with pytest.raises(ValueError, match="flac"):
        read_wav(b"fLaC" + b"\0" * 64)


def test_log_mel_matches_transformers_feature_extractor():
    from transformers import WhisperFeatureExtractor
    x = _tone(3.0)
    for n_mels in (80, 128):
        want = WhisperFeatureExtractor(feature_size=n_mels)(x, sampling_rate=16000, return_tensors="pt")["input_features"][0]
        got = LogMel(n_mels)(x)
        assert got.shape == want.shape == (n_mels, 3000) and (got - want).abs().max().item() < 1e-4


def _tiny_whisper():
    from transformers import WhisperConfig, WhisperForConditionalGeneration
    torch.manual_seed(0)
    hc = WhisperConfig(vocab_size=400, num_mel_bins=80, encoder_layers=2, encoder_attention_heads=4, decoder_layers=2,
                       decoder_attention_heads=4, encoder_ffn_dim=64, decoder_ffn_dim=64, d_model=32,
                       max_source_positions=1500, max_target_positions=40, decoder_start_token_id=SOT, eos_token_id=EOS,
                       pad_token_id=392, bos_token_id=393, suppress_tokens=None, begin_suppress_tokens=None)
    m = WhisperForConditionalGeneration(hc).eval()
    d = tempfile.mkdtemp(prefix="whisper_")
    m.save_pretrained(d, safe_serialization=True)
    gen = dict(decoder_start_token_id=SOT, eos_token_id=EOS, lang_to_id={"<|en|>": EN, "<|fr|>": FR},
               task_to_id={"transcribe": TRANSCRIBE, "translate": TRANSLATE}, no_timestamps_token_id=NOTS,
               suppress_tokens=[1, 2, SOT, EN, FR, TRANSCRIBE, TRANSLATE, NOTS], begin_suppress_tokens=[EOS, 7])
    with open(d + "/generation_config.json", "w") as f:
        json.dump(gen, f)
    return m, d


def _hf_greedy(m, mel, prompt, n, suppress, begin_suppress):
    ids = list(prompt)
    out = []
    with torch.no_grad():
        for step in range(n):
            lg = m(input_features=mel, decoder_input_ids=torch.tensor([ids])).logits[0, -1].clone()
            lg[suppress] = float("-inf")
            if step == 0:
                lg[begin_suppress] = float("-inf")
            t = int(lg.argmax())
            if t == EOS:
                break
            out.append(t)
            ids.append(t)
    return out


class _Tok:
    def decode(self, ids, skip_special_tokens=True):
        return "".join(f" w{i}" for i in ids)


def test_whisper_matches_transformers_and_transcribes_in_chunks():
    m, d = _tiny_whisper()
    assert is_whisper_checkpoint(d)
    ours = WhisperModel.from_pretrained(d, dtype=torch.float32)
    fe = LogMel(80)
    audio = np.concatenate([_tone(30.0, f=300.0, seed=1), _tone(12.0, f=900.0, seed=2)])       # 42 s -> two windows
    mel = torch.stack([fe(audio[:480000]), fe(audio[480000:])])
    with torch.no_grad():
        want_enc = m.model.encoder(mel).last_hidden_state
    assert (ours.encode(mel) - want_enc).abs().max().item() < 1e-4
    tr = Transcriber(ours, _Tok())
    sup, bsup = tr.suppress, tr.begin_suppress
    r = tr.transcribe(audio, language="en", max_new_tokens=10)
    prompt = [SOT, EN, TRANSCRIBE, NOTS]
    want = [_hf_greedy(m, mel[i:i + 1], prompt, 10, sup, bsup) for i in range(2)]
    assert [s["tokens"] for s in r["segments"]] == want
    assert r["text"] == "".join(f" w{i}" for t in want for i in t).strip() and abs(r["duration"] - 42.0) < 1e-6
    assert r["segments"][1]["start"] == 30.0 and abs(r["segments"][1]["end"] - 42.0) < 1e-6
    # language detection = argmax over the language tokens after start-of-transcript
    with torch.no_grad():
        lg = m(input_features=mel[:1], decoder_input_ids=torch.tensor([[SOT]])).logits[0, -1]
    assert tr.detect_language(mel) == ("en" if lg[EN] >= lg[FR] else "fr")
    t2 = tr.transcribe(audio[:16000], task="translate", max_new_tokens=4)
    assert t2["task"] == "translate" and t2["language"] in ("en", "fr")
    with pytest.raises(ValueError, match="unknown language"):
        tr.transcribe(audio[:16000], language="xx")


def test_audio_routes():
    from fastapi.testclient import TestClient

    from mlxcel_b200.server.audio import create_audio_app
    m, d = _tiny_whisper()
    tr = Transcriber(WhisperModel.from_pretrained(d, dtype=torch.float32), _Tok())
    client = TestClient(create_audio_app(tr, "tiny-whisper", {"k"}))
    wav = write_wav(_tone(2.0), 16000)
    h = {"Authorization": "Bearer k"}
    assert client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav)}).status_code == 401
    r = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav)}, data={"language": "en"}, headers=h)
    assert r.status_code == 200 and r.json()["text"].startswith("w")
    direct = tr.transcribe(decode_audio(wav), language="en")
    assert r.json()["text"] == direct["text"]
    v = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav)},
                    data={"language": "en", "response_format": "verbose_json"}, headers=h).json()
    assert v["language"] == "en" and abs(v["duration"] - 2.0) < 1e-6 and v["segments"][0]["tokens"] == direct["segments"][0]["tokens"]
    srt = client.post("/v1/audio/transcriptions", files={"file": ("a.wav", wav)},
                      data={"language": "en", "response_format": "srt"}, headers=h).text
    assert srt.startswith("1\n00:00:00,000 --> 00:00:02,000\n")
    assert client.post("/v1/audio/translations", files={"file": ("a.wav", wav)}, headers=h).status_code == 200
    assert client.post("/v1/audio/transcriptions", files={"file": ("a.mp3", b"ID3" + b"\0" * 100)}, headers=h).status_code == 400
    assert client.post("/v1/audio/speech", headers=h).status_code == 501
    assert client.get("/health").status_code == 200 and "mlxcel_audio_requests" in client.get("/metrics", headers=h).text
