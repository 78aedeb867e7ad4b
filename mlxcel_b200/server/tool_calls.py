"""Tool-call extraction from generated text, one-shot and streaming.

Formats (the reference's src/server/tool_calls/formats.rs): Hermes / Qwen
``<tool_call>{json}</tool_call>``, Llama-3 JSON (``{"name": .., "parameters": ..}`` optionally after
``<|python_tag|>``), Mistral ``[TOOL_CALLS] [ {...}, ... ]``, Functionary-style
``<function=name>{json}</function>``. The streaming filter withholds text that may be the start of
a tool-call marker and emits parsed calls as soon as their closing marker arrives
(src/server/tool_calls/stream_filter.rs).
"""
from __future__ import annotations

import json
import re
import uuid
from dataclasses import dataclass, field


@dataclass
class ToolCall:
    name: str
    arguments: str  # JSON text
    id: str = field(default_factory=lambda: "call_" + uuid.uuid4().hex[:24])

    def to_openai(self, index: int | None = None) -> dict:
        d = {"id": self.id, "type": "function", "function": {"name": self.name, "arguments": self.arguments}}
        if index is not None:
            d["index"] = index
        return d


_HERMES = re.compile(r"<tool_call>\s*(.*?)\s*</tool_call>", re.S)
_FUNC = re.compile(r"<function=([\w.\-]+)>\s*(.*?)\s*</function>", re.S)
_MISTRAL = re.compile(r"\[TOOL_CALLS\]\s*(\[.*\])", re.S)


def _mk(obj) -> ToolCall | None:
    if not isinstance(obj, dict):
        return None
    name = obj.get("name") or (obj.get("function") or {}).get("name")
    args = obj.get("arguments", obj.get("parameters", (obj.get("function") or {}).get("arguments", {})))
    if not name:
        return None
    return ToolCall(name, args if isinstance(args, str) else json.dumps(args, ensure_ascii=False))


def _json_objects(text: str):
    """Yield (start, end, obj) for top-level JSON objects embedded in text."""
    dec = json.JSONDecoder()
    i = 0
    while True:
        i = text.find("{", i)
        if i < 0:
            return
        try:
            obj, end = dec.raw_decode(text, i)
            yield i, end, obj
            i = end
        except json.JSONDecodeError:
            i += 1


def parse_tool_calls(text: str, allowed: set[str] | None = None) -> tuple[str, list[ToolCall]]:
    """Returns (remaining content, tool calls)."""
    calls: list[ToolCall] = []
    content = text

    def ok(c):
        return c is not None and (allowed is None or c.name in allowed)

    ms = list(_HERMES.finditer(text))
    if ms:
        for m in ms:
            try:
                c = _mk(json.loads(m.group(1)))
            except json.JSONDecodeError:
                c = None
            if ok(c):
                calls.append(c)
        return _HERMES.sub("", text).strip(), calls
    ms = list(_FUNC.finditer(text))
    if ms:
        for m in ms:
            c = ToolCall(m.group(1), m.group(2) or "{}")
            if ok(c):
                calls.append(c)
        return _FUNC.sub("", text).strip(), calls
    m = _MISTRAL.search(text)
    if m:
        try:
            for o in json.loads(m.group(1)):
                c = _mk(o)
                if ok(c):
                    calls.append(c)
            return text[: m.start()].strip(), calls
        except json.JSONDecodeError:
            pass
    body = text.split("<|python_tag|>", 1)[-1] if "<|python_tag|>" in text else text
    stripped = body.strip()
    if stripped.startswith("{") or stripped.startswith("["):
        spans = []
        for s, e, obj in _json_objects(body):
            c = _mk(obj)
            if ok(c) and ("parameters" in obj or "arguments" in obj):
                calls.append(c)
                spans.append((s, e))
        if calls:
            content = text.split("<|python_tag|>", 1)[0] if "<|python_tag|>" in text else ""
            return content.strip(), calls
    return content, calls


class ToolCallStreamFilter:
    """Incremental version: feed text deltas, get (visible text, finished tool calls)."""

    MARKERS = ("<tool_call>", "<function=", "[TOOL_CALLS]", "<|python_tag|>")
    CLOSERS = {"<tool_call>": "</tool_call>", "<function=": "</function>"}

    def __init__(self, allowed: set[str] | None = None):
        self.buf = ""
        self.in_call: str | None = None
        self.allowed = allowed
        self.calls: list[ToolCall] = []

    def feed(self, delta: str) -> tuple[str, list[ToolCall]]:
        self.buf += delta
        out, new = "", []
        while True:
            if self.in_call is None:
                idx, mk = -1, None
                for m in self.MARKERS:
                    i = self.buf.find(m)
                    if i >= 0 and (idx < 0 or i < idx):
                        idx, mk = i, m
                if mk is None:
                    keep = 0
                    for m in self.MARKERS:
                        for n in range(min(len(m) - 1, len(self.buf)), 0, -1):
                            if self.buf.endswith(m[:n]):
                                keep = max(keep, n)
                                break
                    out += self.buf[: len(self.buf) - keep]
                    self.buf = self.buf[len(self.buf) - keep:]
                    return out, new
                out += self.buf[:idx]
                self.buf = self.buf[idx:]
                self.in_call = mk
            closer = self.CLOSERS.get(self.in_call)
            if closer is None:
                return out, new      # open-ended formats are parsed at flush()
            j = self.buf.find(closer)
            if j < 0:
                return out, new
            seg = self.buf[: j + len(closer)]
            self.buf = self.buf[j + len(closer):]
            _, cs = parse_tool_calls(seg, self.allowed)
            new += cs
            self.calls += cs
            self.in_call = None

    def flush(self) -> tuple[str, list[ToolCall]]:
        text, self.buf = self.buf, ""
        if not text:
            return "", []
        content, cs = parse_tool_calls(text, self.allowed)
        self.calls += cs
        return (content if not cs else content), cs


def split_reasoning(text: str, open_tag: str = "<think>", close_tag: str = "</think>") -> tuple[str, str]:
    """(reasoning, answer) split used by the reasoning_content field of chat responses."""
    if close_tag in text:
        head, tail = text.split(close_tag, 1)
        return head.replace(open_tag, "").strip(), tail.lstrip()
    if text.lstrip().startswith(open_tag):
        return text.replace(open_tag, "").strip(), ""
    return "", text
