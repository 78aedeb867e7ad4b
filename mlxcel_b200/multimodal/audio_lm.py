"""Speech-language wrapper: audio clips → rows of the language model's embedding stream.

Voxtral (transformers `VoxtralForConditionalGeneration`) keeps a Whisper encoder (128 mel bins, 30 s
chunks) in front of a projector that folds four consecutive encoder frames into one row (linear,
GELU, linear) and a Llama-layout decoder; every audio placeholder token of the prompt expands to
one token per projected row (375 per 30 s chunk). Qwen2-Audio (`Qwen2AudioForConditionalGeneration`)
averages pairs of encoder frames, applies the encoder's final LayerNorm after that pooling and
projects with one linear; a clip is one chunk whose padded tail is masked inside the encoder and
dropped from the rows. The reference's counterparts are its omni-model audio towers
(src/audio/encoder.rs, src/audio/qwen3_omni_moe/, src/multimodal/).

`AudioLanguage` has the interface of `VisionLanguage` (``image_token_id`` is the audio placeholder's
id, ``prepare`` returns the expanded prompt with ``mm_embeds`` and content-derived ``key_tokens``), so
the engine, the prefix cache and the server's media path treat both the same way.
"""
from __future__ import annotations

import hashlib
import json
import time
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

from .. import ops
from ..models.vision import _ACT_NAMES, _act
from ..ops import recurrent as rops
from .vlm import _sub

SUPPORTED_AUDIO = ("voxtral", "qwen2_audio")


def is_audio_lm_checkpoint(path: str | Path) -> bool:
    f = Path(path) / "config.json"
    if not f.exists():
        return False
    raw = json.loads(f.read_text())
    return raw.get("model_type") in SUPPORTED_AUDIO and isinstance(raw.get("audio_config"), dict)


class AudioLanguage:
    modality = "audio"

    def __init__(self, encoder, proj: dict, audio_token_id: int, model_type: str, act: str = "gelu"):
        self.encoder, self.proj, self.model_type = encoder, proj, model_type
        self.image_token_id = int(audio_token_id)
        self.act = _ACT_NAMES.get(act, "gelu")
        self.placeholder_text = {"voxtral": "[AUDIO]", "qwen2_audio": "<|audio_bos|><|AUDIO|><|audio_eos|>"}[model_type]
        c = encoder.cfg
        self.chunk_frames = 2 * c.max_source_positions                   # mel frames of one chunk (3000 = 30 s)
        self.stats = dict(clips=0, audio_tokens=0, encode_seconds=0.0)
        self._mel = None

    @staticmethod
    def from_checkpoint(path: str | Path, dtype=torch.bfloat16, device="cpu") -> "AudioLanguage":
        from ..loading.checkpoint import TensorSource
        from ..models.whisper import WhisperConfig, WhisperModel
        path = Path(path)
        raw = json.loads((path / "config.json").read_text())
        mt, a = raw.get("model_type"), dict(raw["audio_config"])
        if mt not in SUPPORTED_AUDIO:
            raise ValueError(f"unsupported speech-language model_type {mt!r}; supported: {SUPPORTED_AUDIO}")
        ffn = int(a.get("intermediate_size", a.get("encoder_ffn_dim", 4 * int(a.get("hidden_size", a.get("d_model", 1280))))))
        d_model = int(a.get("hidden_size", a.get("d_model", 1280)))
        heads = int(a.get("num_attention_heads", a.get("encoder_attention_heads", 20)))
        layers = int(a.get("num_hidden_layers", a.get("encoder_layers", 32)))
        wc = WhisperConfig(d_model=d_model, n_mels=int(a.get("num_mel_bins", 128)), enc_layers=layers, enc_heads=heads,
                           dec_layers=0, dec_heads=heads, enc_ffn=ffn, dec_ffn=ffn, vocab_size=int(a.get("vocab_size", 51866)),
                           max_source_positions=int(a.get("max_source_positions", 1500)),
                           act={"gelu": "gelu", "gelu_new": "gelu_tanh"}.get(a.get("activation_function", "gelu"), "gelu"))
        src = TensorSource(path)
        enc_t = _sub(src, "audio_tower.", "model.audio_tower.")
        enc = WhisperModel(wc, enc_t, dtype, device, encoder_only=True, prefix="")
        pt = _sub(src, "multi_modal_projector.", "model.multi_modal_projector.")
        proj = {k: v.to(dtype).to(device).contiguous() for k, v in pt.items()}
        tok = raw.get("audio_token_id", raw.get("audio_token_index", 24 if mt == "voxtral" else 151646))
        al = AudioLanguage(enc, proj, tok, mt, raw.get("projector_hidden_act", "gelu"))
        al.ffn = ffn
        return al

    # ------------------------------------------------------------------ features
    def mel(self, samples: np.ndarray) -> torch.Tensor:
        """16 kHz mono samples → [chunks, n_mels, chunk_frames] log-mel features (the last chunk zero-padded)."""
        from ..audio.features import LogMel
        if self._mel is None:
            self._mel = LogMel(n_mels=self.encoder.cfg.n_mels)
        hop, per = 160, self.chunk_frames * 160
        x = np.asarray(samples, dtype=np.float32)
        n = max(1, -(-len(x) // per))
        out = []
        for i in range(n):
            seg = x[i * per:(i + 1) * per]
            m = self._mel(np.pad(seg, (0, per - len(seg))), pad=False)
            out.append(m[..., :self.chunk_frames] if m.shape[-1] >= self.chunk_frames else F.pad(m, (0, self.chunk_frames - m.shape[-1])))
        feats = torch.stack([o.reshape(self.encoder.cfg.n_mels, -1) for o in out])
        feats.valid_frames = -(-len(x) // hop)
        return feats

    @torch.no_grad()
    def encode_one(self, feats: torch.Tensor, valid_frames: int | None = None) -> torch.Tensor:
        """[chunks, n_mels, frames] → [rows, text_hidden]."""
        enc, p = self.encoder, self.proj
        if self.model_type == "voxtral":
            h = enc.encode(feats)                                            # [chunks, frames / 2, d]
            h = h.reshape(-1, self.ffn).contiguous()                        # four frames per row
            u = _act(ops.linear(h, p["linear_1.weight"], bias=p.get("linear_1.bias")), self.act)
            return ops.linear(u, p["linear_2.weight"], bias=p.get("linear_2.bias"))
        # qwen2_audio: one chunk per clip; frames behind the clip's end are masked out of the attention
        if feats.shape[0] != 1:
            raise ValueError("qwen2_audio takes clips of at most one chunk (30 s)")
        total = feats.shape[-1]
        valid = min(int(valid_frames if valid_frames is not None else total), total)
        t_enc = (valid - 1) // 2 + 1                                         # encoder frames that carry audio
        h = enc.encode(feats, key_len=t_enc, final_norm=False)               # [1, total / 2, d]
        T = h.shape[1] // 2 * 2
        h = h[:, :T].float().view(1, T // 2, 2, -1).mean(2).to(enc.dtype)    # average pairs of frames
        h = rops.layernorm(h[0].contiguous(), *enc.enc_ln, 1e-5)
        rows = ops.linear(h, p["linear.weight"], bias=p.get("linear.bias"))
        return rows[:(t_enc - 2) // 2 + 1]

    def tokens_for(self, audio) -> int:
        feats = audio if isinstance(audio, torch.Tensor) else self.mel(audio)
        if self.model_type == "voxtral":
            return feats.shape[0] * (self.chunk_frames // 2) // 4
        valid = min(int(getattr(feats, "valid_frames", feats.shape[-1])), feats.shape[-1])
        return (((valid - 1) // 2 + 1) - 2) // 2 + 1

    def prepare(self, prompt_ids: list[int], audios: list):
        n_ph = sum(1 for t in prompt_ids if t == self.image_token_id)
        if n_ph != len(audios):
            raise ValueError(f"the prompt has {n_ph} audio placeholders for {len(audios)} clips")
        t0 = time.perf_counter()
        rows_of = []
        for a in audios:
            feats = a if isinstance(a, torch.Tensor) else self.mel(a)
            rows_of.append(self.encode_one(feats, getattr(feats, "valid_frames", None)))
        ids, keys, spans = [], [], []
        it = iter(rows_of)
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
            self.stats["audio_tokens"] += n
        self.stats["clips"] += len(audios)
        self.stats["encode_seconds"] += time.perf_counter() - t0
        return ids, dict(mm_embeds=spans, key_tokens=keys)
