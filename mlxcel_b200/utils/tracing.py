"""Host-side tracing: Chrome-trace spans and optional NVTX ranges.

Counterpart of the reference's per-tick `tracing` spans (src/server/batch/scheduler/decode_tick.rs:287),
its TTFT phase profile (src/lib/mlxcel-core/src/generate.rs:1741-1813) and the pipeline Chrome-trace
writer behind ``--debug-pp-trace`` (src/distributed/pipeline/trace.rs:15-60).

``MLXCEL_B200_TRACE=<file>`` (or ``Tracer.enable(path)``) records ``span(name, **args)`` intervals
with wall-clock microseconds and writes ``{"traceEvents": [...]}`` at exit or on ``flush()`` — load
it in chrome://tracing or Perfetto. ``MLXCEL_B200_NVTX=1`` additionally pushes NVTX ranges so the
same spans show up in a CUDA timeline. With neither set, ``span`` is a no-op context manager.
"""
from __future__ import annotations

import atexit
import json
import os
import threading
import time
from contextlib import contextmanager


class Tracer:
    def __init__(self):
        self.path: str | None = None
        self.nvtx = False
        self.events: list[dict] = []
        self._lock = threading.Lock()
        self._t0 = time.perf_counter()
        self.pid = os.getpid()

    def enable(self, path: str | None = None, nvtx: bool | None = None) -> None:
        if path:
            if self.path is None:
                atexit.register(self.flush)
            self.path = path
        if nvtx is not None:
            self.nvtx = nvtx

    @property
    def active(self) -> bool:
        return self.path is not None or self.nvtx

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    @contextmanager
    def span(self, name: str, cat: str = "engine", **args):
        if not self.active:
            yield
            return
        if self.nvtx:
            import torch
            torch.cuda.nvtx.range_push(name)
        t = self._now_us()
        try:
            yield
        finally:
            if self.nvtx:
                import torch
                torch.cuda.nvtx.range_pop()
            if self.path is not None:
                ev = {"name": name, "cat": cat, "ph": "X", "ts": t, "dur": self._now_us() - t, "pid": self.pid,
                      "tid": threading.get_ident() % 100000, "args": args}
                with self._lock:
                    self.events.append(ev)

    def instant(self, name: str, cat: str = "engine", **args) -> None:
        if self.path is None:
            return
        with self._lock:
            self.events.append({"name": name, "cat": cat, "ph": "i", "s": "t", "ts": self._now_us(), "pid": self.pid,
                                "tid": threading.get_ident() % 100000, "args": args})

    def flush(self) -> None:
        if self.path is None:
            return
        with self._lock:
            doc = {"traceEvents": list(self.events), "displayTimeUnit": "ms"}
        rank = os.environ.get("RANK")
        path = self.path if rank is None else f"{self.path}.rank{rank}"
        with open(path, "w") as f:
            json.dump(doc, f)


TRACER = Tracer()
if os.environ.get("MLXCEL_B200_TRACE"):
    TRACER.enable(path=os.environ["MLXCEL_B200_TRACE"])
if os.environ.get("MLXCEL_B200_NVTX") == "1":
    TRACER.enable(nvtx=True)

span = TRACER.span
instant = TRACER.instant
