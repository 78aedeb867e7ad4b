"""Speech-to-text driver around `WhisperModel`: chunking, language / task prompt, token suppression,
text assembly (reference: the Whisper request path behind /v1/audio/transcriptions,
src/server/routes/audio*.rs, src/audio/preprocessing_policy.rs).

Audio of any length is cut into 30-second windows; the windows of one request are decoded together
as one batch (one encoder pass, one decoder loop), each after the forced prompt
``<|startoftranscript|> <|lang|> <|transcribe or translate|> <|notimestamps|>``. Without a language
the first window is asked for its language token first. Windows are independent (no text carried
from one window into the next window's prompt).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch

from .features import LogMel


class Transcriber:
    def __init__(self, model, tokenizer, generation: dict | None = None, max_batch: int = 16):
        self.model, self.tokenizer = model, tokenizer
        g = dict(generation or getattr(model, "generation", None) or {})
        self.lang_to_id: dict = dict(g.get("lang_to_id") or {})
        self.task_to_id: dict = dict(g.get("task_to_id") or {})
        self.no_timestamps = g.get("no_timestamps_token_id")
        self.suppress = list(g.get("suppress_tokens") or [])
        self.begin_suppress = list(g.get("begin_suppress_tokens") or [])
        self.sot = int(g.get("decoder_start_token_id", model.cfg.decoder_start_token_id))
        self.eos = int(g.get("eos_token_id", model.cfg.eos_token_id) if not isinstance(g.get("eos_token_id"), list)
                       else g["eos_token_id"][0])
        self.mel = LogMel(model.cfg.n_mels)
        self.max_batch = max_batch
        self.stats = dict(requests=0, seconds_of_audio=0.0, chunks=0, tokens=0)

    @staticmethod
    def from_pretrained(path: str | Path, dtype=torch.bfloat16, device="cpu") -> "Transcriber":
        from ..models.whisper import WhisperModel
        from ..tokenizer import load_tokenizer
        return Transcriber(WhisperModel.from_pretrained(path, dtype, device), load_tokenizer(path))

    def _lang_token(self, language: str | None) -> int | None:
        if not self.lang_to_id or language is None:
            return None
        key = language if language.startswith("<|") else f"<|{language.lower()}|>"
        if key not in self.lang_to_id:
            raise ValueError(f"unknown language {language!r}")
        return int(self.lang_to_id[key])

    @torch.no_grad()
    def detect_language(self, mel: torch.Tensor) -> str | None:
        """The most likely language token right after start-of-transcript, for the first window."""
        if not self.lang_to_id:
            return None
        m = self.model
        enc = m.encode(mel[:1])
        cache = [(torch.zeros(1, 4, m.cfg.d_model, dtype=m.dtype, device=m.device),
                  torch.zeros(1, 4, m.cfg.d_model, dtype=m.dtype, device=m.device)) for _ in m.dec]
        logits = m._decode_rows(torch.tensor([[self.sot]], device=m.device), 0, cache, m._cross_kv(enc))[0, -1]
        ids = torch.tensor(list(self.lang_to_id.values()), device=logits.device)
        best = int(ids[logits[ids].argmax()])
        return next(k for k, v in self.lang_to_id.items() if int(v) == best).strip("<|>")

    def transcribe(self, samples: np.ndarray, language: str | None = None, task: str = "transcribe",
                   max_new_tokens: int = 224) -> dict:
        """16 kHz mono float samples → ``{"text", "language", "duration", "segments"}``."""
        if task not in ("transcribe", "translate"):
            raise ValueError("task must be transcribe or translate")
        n, win = len(samples), self.mel.n_samples
        chunks = [samples[i:i + win] for i in range(0, max(n, 1), win)]
        mel = torch.stack([self.mel(c) for c in chunks])
        if language is None:
            language = self.detect_language(mel)
        prompt = [self.sot]
        lt = self._lang_token(language)
        if lt is not None:
            prompt.append(lt)
        if self.task_to_id:
            prompt.append(int(self.task_to_id[task]))
        if self.no_timestamps is not None:
            prompt.append(int(self.no_timestamps))
        ids: list[list[int]] = []
        for i in range(0, len(chunks), self.max_batch):
            ids += self.model.generate(mel[i:i + self.max_batch], prompt, max_new_tokens, self.suppress,
                                       self.begin_suppress, self.eos)
        segs = []
        for i, t in enumerate(ids):
            text = self.tokenizer.decode(t, skip_special_tokens=True)
            segs.append(dict(id=i, start=i * win / self.mel.sr, end=min(n, (i + 1) * win) / self.mel.sr, text=text, tokens=t))
        self.stats["requests"] += 1
        self.stats["seconds_of_audio"] += n / self.mel.sr
        self.stats["chunks"] += len(chunks)
        self.stats["tokens"] += sum(len(t) for t in ids)
        return dict(text="".join(s["text"] for s in segs).strip(), language=language, duration=n / self.mel.sr,
                    segments=segs, task=task)


def is_whisper_checkpoint(path: str | Path) -> bool:
    f = Path(path) / "config.json"
    return f.exists() and json.loads(f.read_text()).get("model_type") == "whisper"
