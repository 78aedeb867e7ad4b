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


class TiktokenTokenizer:
    """Byte-level BPE from a tiktoken vocabulary file (``tiktoken.model`` / ``*.tiktoken``: one
    ``base64(token bytes) rank`` pair per line), as shipped by the Kimi and some Qwen / Llama-3 original
    checkpoints (reference: the tiktoken branch of the tokenizer loader, src/server/state.rs:723-760).
    Control tokens come from ``tokenizer_config.json`` (``added_tokens_decoder``) and sit above the
    ranks. Text is split by the vocabulary's pre-tokenization pattern, each piece's bytes are merged
    greedily by rank (lowest rank first), and control-token literals in the text map to their ids."""

    # the pattern of the cl100k / Llama-3 family; a checkpoint may carry its own as ``pat_str`` in
    # tokenizer_config.json
    DEFAULT_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|"
                       r"\s*[\r\n]+|\s+(?!\S)|\s+")

    def __init__(self, path: Path):
        import base64

        import regex

        f = next((c for c in [path / "tiktoken.model", *sorted(path.glob("*.tiktoken"))] if c.exists()), None)
        if f is None:
            raise FileNotFoundError(f"{path}: no tiktoken vocabulary")
        self.ranks: dict[bytes, int] = {}
        for line in f.read_text().splitlines():
            if line.strip():
                tok, rank = line.split()
                self.ranks[base64.b64decode(tok)] = int(rank)
        self.by_id: dict[int, bytes] = {r: b for b, r in self.ranks.items()}
        cfg = json.loads((path / "tokenizer_config.json").read_text()) if (path / "tokenizer_config.json").exists() else {}
        self.config = cfg
        self.chat_template = cfg.get("chat_template")
        if (path / "chat_template.jinja").exists():
            self.chat_template = (path / "chat_template.jinja").read_text()
        self.special: dict[str, int] = {}
        for i, ent in (cfg.get("added_tokens_decoder") or {}).items():
            self.special[ent["content"] if isinstance(ent, dict) else str(ent)] = int(i)
        self.special_by_id = {i: t for t, i in self.special.items()}
        self.vocab_size = max([*self.by_id, *self.special_by_id, -1]) + 1
        self.pattern = regex.compile(cfg.get("pat_str") or self.DEFAULT_PATTERN)
        self._special_re = (regex.compile("|".join(regex.escape(t) for t in sorted(self.special, key=len, reverse=True)))
                            if self.special else None)

        def name(v):
            return v.get("content") if isinstance(v, dict) else v
        self.bos_token, self.eos_token = name(cfg.get("bos_token")), name(cfg.get("eos_token"))
        self.bos_token_id, self.eos_token_id = self.special.get(self.bos_token), self.special.get(self.eos_token)
        self._eos = set([self.eos_token_id] if self.eos_token_id is not None else [])
        gen = path / "generation_config.json"
        if gen.exists():
            e = json.loads(gen.read_text()).get("eos_token_id")
            if e is not None:
                self._eos.update(e if isinstance(e, list) else [e])
        self.think_open, self.think_close = self.special.get("<think>"), self.special.get("</think>")
        self.fim = dict(prefix=None, suffix=None, middle=None)
        self._cache: dict[bytes, list[int]] = {}

    def control_id(self, literal: str) -> int | None:
        return self.special.get(literal)

    def _bpe(self, piece: bytes) -> list[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        if piece in self.ranks:
            out = [self.ranks[piece]]
        else:
            parts = [piece[i:i + 1] for i in range(len(piece))]
            while len(parts) > 1:
                best, at = None, -1
                for i in range(len(parts) - 1):
                    r = self.ranks.get(parts[i] + parts[i + 1])
                    if r is not None and (best is None or r < best):
                        best, at = r, i
                if best is None:
                    break
                parts[at:at + 2] = [parts[at] + parts[at + 1]]
            out = [self.ranks[p] for p in parts]
        if len(self._cache) < 1 << 16:
            self._cache[piece] = out
        return out

    def _encode_plain(self, text: str) -> list[int]:
        ids: list[int] = []
        for m in self.pattern.finditer(text):
            ids += self._bpe(m.group().encode("utf-8"))
        return ids

    def encode(self, text: str, add_special_tokens: bool = False) -> list[int]:
        ids = [self.bos_token_id] if add_special_tokens and self.bos_token_id is not None else []
        if self._special_re is None:
            return ids + self._encode_plain(text)
        pos = 0
        for m in self._special_re.finditer(text):
            ids += self._encode_plain(text[pos:m.start()])
            ids.append(self.special[m.group()])
            pos = m.end()
        return ids + self._encode_plain(text[pos:])

    def token_bytes(self, i: int) -> bytes:
        b = self.by_id.get(int(i))
        return b if b is not None else self.special_by_id.get(int(i), "").encode("utf-8")

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        out = bytearray()
        for i in ids:
            b = self.by_id.get(int(i))
            if b is not None:
                out += b
            elif not skip_special_tokens:
                out += self.special_by_id.get(int(i), "").encode("utf-8")
        return out.decode("utf-8", errors="replace")

    def eos_ids(self) -> list[int]:
        return sorted(self._eos)

    def fingerprint(self) -> str:
        import hashlib
        h = hashlib.sha256()
        for b, r in sorted(self.ranks.items(), key=lambda kv: kv[1]):
            h.update(b + b"\0" + str(r).encode())
        return h.hexdigest()[:16]


def load_tokenizer(path: str | Path):
    p = Path(path)
    if (p / "tokenizer.json").exists():
        return HFTokenizer(p)
    if (p / "tiktoken.model").exists() or any(p.glob("*.tiktoken")):
        return TiktokenTokenizer(p)
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
