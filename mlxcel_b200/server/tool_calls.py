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
_MISTRAL_ARGS = re.compile(r"\[TOOL_CALLS\]\s*([\w.\-]+)\s*\[ARGS\]\s*", re.S)


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
    ms = list(_MISTRAL_ARGS.finditer(text))
    if ms:       # [TOOL_CALLS]name[ARGS]{json}, repeated per call
        dec = json.JSONDecoder()
        for m in ms:
            try:
                obj, _ = dec.raw_decode(text, m.end())
            except json.JSONDecodeError:
                continue
            c = ToolCall(m.group(1), json.dumps(obj, ensure_ascii=False))
            if ok(c):
                calls.append(c)
        return text[: ms[0].start()].strip(), calls
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



class _CallScanner:
    """Scans ONE JSON call object while its text arrives (``{"name": .., "arguments": {..}}``, the
    ``parameters`` spelling, or the nested ``{"function": {..}}`` form). It reports the name as soon
    as its string closes and hands out the raw text of the arguments object as it grows, so a route
    can stream argument fragments instead of one burst at the closing marker
    (src/server/tool_calls/incremental.rs, incremental/json_call.rs)."""

    NAME_KEYS, ARG_KEYS = ("name",), ("arguments", "parameters")

    def __init__(self):
        self.text = ""
        self.pos = 0
        self.depth = 0
        self.level = 1             # depth at which the call's keys live (2 inside {"function": {..}})
        self.in_str = self.esc = False
        self.str_start = 0
        self.key = self.pending = None
        self.after_colon = False
        self.name = None
        self.args_start = self.args_end = None
        self.args_string = None    # arguments given as a JSON-encoded string
        self.done = False
        self.sent = 0

    def feed(self, chunk: str) -> str:
        """Consume text; returns what follows the object's closing brace (empty while inside)."""
        self.text += chunk
        t = self.text
        while self.pos < len(t) and not self.done:
            ch = t[self.pos]
            if self.in_str:
                if self.esc:
                    self.esc = False
                elif ch == "\\":
                    self.esc = True
                elif ch == '"':
                    self.in_str = False
                    if self.depth == self.level and self._outside_args():
                        try:
                            val = json.loads(t[self.str_start:self.pos + 1])
                        except json.JSONDecodeError:
                            val = None
                        if self.after_colon:
                            if self.key in self.NAME_KEYS and isinstance(val, str):
                                self.name = val
                            elif self.key in self.ARG_KEYS and isinstance(val, str) and self.args_string is None:
                                self.args_string = val
                            self.after_colon = False
                        else:
                            self.pending = val
            elif ch == '"':
                self.in_str, self.str_start = True, self.pos
            elif ch == ":" and self.depth == self.level and self._outside_args():
                self.key, self.after_colon = self.pending, True
            elif ch in "{[":
                if self.depth == self.level and self.after_colon and self._outside_args():
                    if ch == "{" and self.key in self.ARG_KEYS and self.args_start is None:
                        self.args_start = self.pos
                    elif ch == "{" and self.key == "function" and self.level == 1:
                        self.level = 2
                    self.after_colon = False
                self.depth += 1
            elif ch in "}]":
                self.depth -= 1
                if self.args_start is not None and self.args_end is None and self.depth == self.level:
                    self.args_end = self.pos + 1
                if self.depth < self.level and self.level == 2:
                    self.level = 1
                if self.depth <= 0:
                    self.done = True
            elif ch == "," and self.depth == self.level and self._outside_args():
                self.after_colon = False
            elif self.depth == self.level and self.after_colon and self._outside_args() and not ch.isspace():
                pass                    # a bare literal (number, true, null) as a value
            self.pos += 1
        if self.done:
            rest, self.text = t[self.pos:], t[:self.pos]
            return rest
        return ""

    def _outside_args(self) -> bool:
        return self.args_start is None or self.args_end is not None

    def take_args(self) -> str:
        """New argument text since the last call (raw slice of the object; a string-encoded value is
        handed out whole once it closed)."""
        if self.args_string is not None:
            out, self.sent = self.args_string[self.sent:], len(self.args_string)
            return out
        if self.args_start is None:
            return ""
        end = self.args_end if self.args_end is not None else self.pos
        out = self.text[self.args_start + self.sent:end]
        self.sent += len(out)
        return out

    @property
    def args_complete(self) -> bool:
        return self.args_end is not None or self.args_string is not None


class IncrementalToolCallStreamer:
    """Streaming tool-call extraction with argument fragments.

    ``feed(delta)`` returns ``(visible text, deltas)`` where each delta is an entry of an OpenAI
    ``delta.tool_calls`` list: the first one of a call carries ``id``, ``type`` and the name with empty
    arguments, the following ones only ``{"index", "function": {"arguments": fragment}}``. Streamed
    formats: Hermes / Qwen ``<tool_call>{json}</tool_call>``, Llama-3 ``<|python_tag|>{json}``, Mistral
    ``[TOOL_CALLS] [{..}, ..]`` and ``[TOOL_CALLS]name[ARGS]{json}``. Other formats, and calls the
    scanner could not announce (unknown tool, name after malformed text), are sent whole when their
    region closes: `parse_tool_calls` on the region's text stays authoritative for what counts as
    a call. Only a partial marker and the object being scanned are held back."""

    MARKERS = ToolCallStreamFilter.MARKERS
    CLOSERS = ToolCallStreamFilter.CLOSERS
    SCANNED = ("<tool_call>", "<|python_tag|>", "[TOOL_CALLS]")

    def __init__(self, allowed: set[str] | None = None):
        self.allowed = allowed
        self.buf = ""
        self.region: str | None = None
        self.region_text = ""
        self.n = 0                            # next call index
        self.calls: list[ToolCall] = []       # every call reported, in index order
        self.scan: _CallScanner | None = None
        self.cur: ToolCall | None = None      # call the scanner announced for the object it is in
        self.cur_index = 0
        self.announced: list[ToolCall] = []   # announced in the open region, not yet confirmed
        self.header = ""                      # Mistral: text between the marker and the first object
        self.fixed_name: str | None = None

    @staticmethod
    def _partial_suffix(text: str, markers) -> int:
        keep = 0
        for m in markers:
            for n in range(min(len(m) - 1, len(text)), 0, -1):
                if text.endswith(m[:n]):
                    keep = max(keep, n)
                    break
        return keep

    def _payload(self, text: str, deltas: list) -> None:
        self.region_text += text
        if self.region not in self.SCANNED:
            return
        while text:
            if self.scan is None:
                if self.region == "[TOOL_CALLS]" and self.fixed_name is None:
                    self.header += text
                    m = re.match(r"\s*([\w.\-]+)\s*\[ARGS\]", self.header)
                    if m:
                        self.fixed_name, text, self.header = m.group(1), self.header[m.end():], ""
                    elif "{" in self.header or "[" in self.header.strip()[:1]:
                        text, self.header = self.header, ""
                    else:
                        return          # still undecided between "name[ARGS]" and the list form
                i = text.find("{")
                if i < 0:
                    return
                text = text[i:]
                self.scan, self.cur = _CallScanner(), None
                if self.fixed_name is not None:     # name[ARGS]{json}: the object IS the arguments
                    self.scan.args_start, self.scan.level = 0, 0
            rest = self.scan.feed(text)
            name = self.fixed_name or self.scan.name
            if self.cur is None and name is not None and (self.allowed is None or name in self.allowed):
                self.cur = ToolCall(name, "")
                self.cur_index, self.n = self.n, self.n + 1
                self.calls.append(self.cur)
                self.announced.append(self.cur)
                deltas.append({"index": self.cur_index, "id": self.cur.id, "type": "function",
                               "function": {"name": name, "arguments": ""}})
            if self.cur is not None:
                frag = self.scan.take_args()
                if frag:
                    self.cur.arguments += frag
                    deltas.append({"index": self.cur_index, "function": {"arguments": frag}})
            if not self.scan.done:
                return
            self.scan, self.cur, self.fixed_name, text = None, None, None, rest

    def _close_region(self, deltas: list) -> str:
        """The region's text is complete: confirm what was streamed, send the rest whole. Returns the
        text to show when the region held no call at all."""
        content, parsed = parse_tool_calls(self.region_text, self.allowed)
        pending = list(self.announced)
        for c in parsed:
            hit = next((a for a in pending if a.name == c.name), None)
            if hit is not None:
                pending.remove(hit)
                continue
            self.calls.append(c)
            deltas.append(c.to_openai(self.n))
            self.n += 1
        shown = "" if (parsed or self.announced) else content
        self.region, self.region_text, self.announced = None, "", []
        self.scan, self.cur, self.header, self.fixed_name = None, None, "", None
        return shown

    def feed(self, delta: str, final: bool = False) -> tuple[str, list[dict]]:
        self.buf += delta
        out, deltas = "", []
        while True:
            if self.region is None:
                idx, mk = -1, None
                for m in self.MARKERS:
                    i = self.buf.find(m)
                    if i >= 0 and (idx < 0 or i < idx):
                        idx, mk = i, m
                if mk is None:
                    keep = 0 if final else self._partial_suffix(self.buf, self.MARKERS)
                    out += self.buf[: len(self.buf) - keep]
                    self.buf = self.buf[len(self.buf) - keep:]
                    break
                out += self.buf[:idx]
                self.buf = self.buf[idx + len(mk):]
                self.region, self.region_text = mk, mk
            closer = self.CLOSERS.get(self.region)
            if closer is None:                     # open-ended: runs to the end of the text
                text, self.buf = self.buf, ""
                self._payload(text, deltas)
                break
            j = self.buf.find(closer)
            if j < 0:
                keep = 0 if final else self._partial_suffix(self.buf, (closer,))
                text, self.buf = self.buf[: len(self.buf) - keep], self.buf[len(self.buf) - keep:]
                self._payload(text, deltas)
                break
            self._payload(self.buf[:j], deltas)
            self.region_text += closer
            self.buf = self.buf[j + len(closer):]
            out += self._close_region(deltas)
        if final and self.region is not None:
            out += self._close_region(deltas)
        return out, deltas

    def flush(self) -> tuple[str, list[dict]]:
        return self.feed("", final=True)


def split_reasoning(text: str, open_tag: str = "<think>", close_tag: str = "</think>") -> tuple[str, str]:
    """(reasoning, answer) split used by the reasoning_content field of chat responses."""
    if close_tag in text:
        head, tail = text.split(close_tag, 1)
        return head.replace(open_tag, "").strip(), tail.lstrip()
    if text.lstrip().startswith(open_tag):
        return text.replace(open_tag, "").strip(), ""
    return "", text
