"""Streaming-safe stop-string matching (src/server/batch/stop_matcher.rs in the reference):
text is released only once it can no longer be the beginning of a stop string, and everything
from the first stop string on is cut."""
from __future__ import annotations


class StopMatcher:
    def __init__(self, stops: list[str]):
        self.stops = [s for s in stops if s]
        self.held = ""
        self.stopped: str | None = None

    def feed(self, text: str) -> str:
        """Returns the text that is safe to emit now."""
        if self.stopped is not None:
            return ""
        if not self.stops:
            return text
        buf = self.held + text
        best = -1
        which = None
        for s in self.stops:
            i = buf.find(s)
            if i >= 0 and (best < 0 or i < best):
                best, which = i, s
        if best >= 0:
            self.stopped = which
            self.held = ""
            return buf[:best]
        keep = 0
        for s in self.stops:
            for n in range(min(len(s) - 1, len(buf)), 0, -1):
                if buf.endswith(s[:n]):
                    keep = max(keep, n)
                    break
        self.held = buf[len(buf) - keep:] if keep else ""
        return buf[: len(buf) - keep] if keep else buf

    def flush(self) -> str:
        out, self.held = ("" if self.stopped is not None else self.held), ""
        return out
