"""Tokenizers and incremental detokenisation.

Loads HF ``tokenizer.json`` (the `tokenizers` library), falls back to SentencePiece
(``tokenizer.model``) and to a byte-level tokenizer when a directory has neither (synthetic
models). Mirrors the reference's tokenizer layer (src/tokenizer/*): chat template lookup in
``tokenizer_config.json`` / ``chat_template.jinja``, EOS merge from ``generation_config.json``,
thinking-token ids, FIM tokens, and a streaming-safe detokeniser that never emits half a UTF-8
sequence.
"""
from __future__ import annotations

import json
from pathlib import Path


class ByteTokenizer:
    """256 byte tokens + BOS/EOS; enough to drive the engine and server without a vocabulary file."""

    def __init__(self, vocab_size: int = 260):
        self.vocab_size = max(vocab_size, 258)
        self.bos_token_id, self.eos_token_id = 256, 257
        self.chat_template = None
        self.special = {"<bos>": 256, "<eos>": 257}

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = list(text.encode("utf-8"))
        return ([self.bos_token_id] + ids) if add_special_tokens else ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", errors="replace")

    def token_bytes(self, i: int) -> bytes:
        return bytes([i]) if 0 <= i < 256 else b""

    def eos_ids(self) -> list[int]:
        return [self.eos_token_id]


class HFTokenizer:
    def __init__(self, path: Path):
        from tokenizers import Tokenizer

        self.tk = Tokenizer.from_file(str(path / "tokenizer.json"))
        self.vocab_size = self.tk.get_vocab_size(with_added_tokens=True)
        cfg = {}
        if (path / "tokenizer_config.json").exists():
            cfg = json.loads((path / "tokenizer_config.json").read_text())
        self.config = cfg
        self.chat_template = cfg.get("chat_template")
        if isinstance(self.chat_template, list):   # named templates
            named = {t.get("name"): t.get("template") for t in self.chat_template}
            self.chat_template = named.get("default") or next(iter(named.values()), None)
        if (path / "chat_template.jinja").exists():
            self.chat_template = (path / "chat_template.jinja").read_text()

        def tok_id(v):
            if isinstance(v, dict):
                v = v.get("content")
            return self.tk.token_to_id(v) if isinstance(v, str) else None

        self.bos_token, self.eos_token = cfg.get("bos_token"), cfg.get("eos_token")
        if isinstance(self.bos_token, dict):
            self.bos_token = self.bos_token.get("content")
        if isinstance(self.eos_token, dict):
            self.eos_token = self.eos_token.get("content")
        self.bos_token_id, self.eos_token_id = tok_id(self.bos_token), tok_id(self.eos_token)
        self._eos = set([self.eos_token_id] if self.eos_token_id is not None else [])
        gen = path / "generation_config.json"
        if gen.exists():
            e = json.loads(gen.read_text()).get("eos_token_id")
            if e is not None:
                self._eos.update(e if isinstance(e, list) else [e])
        self.think_open, self.think_close = tok_id("<think>"), tok_id("</think>")
        # fill-in-the-middle sentinels: Qwen / CodeGemma, StarCoder, CodeLlama and DeepSeek-Coder spellings
        spellings = dict(prefix=("<|fim_prefix|>", "<fim_prefix>", "\u2581<PRE>", "<PRE>", "<\uff5cfim\u2581begin\uff5c>"),
                         suffix=("<|fim_suffix|>", "<fim_suffix>", "\u2581<SUF>", "<SUF>", "<\uff5cfim\u2581hole\uff5c>"),
                         middle=("<|fim_middle|>", "<fim_middle>", "\u2581<MID>", "<MID>", "<\uff5cfim\u2581end\uff5c>"))
        self.fim = {k: next((i for i in map(tok_id, v) if i is not None), None) for k, v in spellings.items()}

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        return self.tk.encode(text, add_special_tokens=add_special_tokens).ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        return self.tk.decode(list(ids), skip_special_tokens=skip_special_tokens)

    def eos_ids(self) -> list[int]:
        return sorted(self._eos)

    def fingerprint(self) -> str:
        import hashlib
        return hashlib.sha256(self.tk.to_str().encode()).hexdigest()[:16]


class SPTokenizer:
    def __init__(self, path: Path):
        import sentencepiece as spm

        self.sp = spm.SentencePieceProcessor(model_file=str(path / "tokenizer.model"))
        self.vocab_size = self.sp.vocab_size()
        self.bos_token_id, self.eos_token_id = self.sp.bos_id(), self.sp.eos_id()
        self.chat_template = None

    def encode(self, text, add_special_tokens=False):
        ids = self.sp.encode(text)
        return ([self.bos_token_id] + ids) if add_special_tokens and self.bos_token_id >= 0 else ids

    def decode(self, ids, skip_special_tokens=True):
        return self.sp.decode(list(ids))

    def eos_ids(self):
        return [self.eos_token_id] if self.eos_token_id >= 0 else []


def load_tokenizer(path: str | Path):
    p = Path(path)
    if (p / "tokenizer.json").exists():
        return HFTokenizer(p)
    if (p / "tokenizer.model").exists():
        return SPTokenizer(p)
    vocab = 260
    if (p / "config.json").exists():
        vocab = int(json.loads((p / "config.json").read_text()).get("vocab_size", 260))
    return ByteTokenizer(vocab)


class IncrementalDetokenizer:
    """Streams text for a growing token list. Holds back output while the tail decodes to an
    incomplete UTF-8 sequence (replacement character at the end), and decodes with a short
    prefix window so tokenizers that merge across tokens (byte-level BPE, SentencePiece spaces)
    produce the same text as a one-shot decode."""

    def __init__(self, tokenizer, prompt_ids: list[int] | None = None, window: int = 6):
        self.tk = tokenizer
        self.ids: list[int] = list(prompt_ids[-window:]) if prompt_ids else []
        self.prefix_len = len(self.ids)
        self.read = self.prefix_len     # tokens already turned into emitted text
        self.window = window

    def push(self, token_id: int) -> str:
        self.ids.append(token_id)
        start = max(0, self.read - self.window)
        prev = self.tk.decode(self.ids[start:self.read]) if self.read > start else ""
        full = self.tk.decode(self.ids[start:])
        if full.endswith("�"):
            return ""                   # wait for the rest of the character
        self.read = len(self.ids)
        return full[len(prev):] if full.startswith(prev) else full

    def flush(self) -> str:
        if self.read >= len(self.ids):
            return ""
        start = max(0, self.read - self.window)
        prev = self.tk.decode(self.ids[start:self.read]) if self.read > start else ""
        full = self.tk.decode(self.ids[start:])
        self.read = len(self.ids)
        return full[len(prev):] if full.startswith(prev) else full
