"""Import shim for the C++ host runtime (``lib/_mlxcel_host*.so``), building it on first use."""
from __future__ import annotations

import importlib.util
import sys

from . import _build


def _load():
    path = _build.host_ext_path()
    stale = not path.exists() or any(
        s.stat().st_mtime > path.stat().st_mtime for s in _build.HOST.glob("*.cpp"))
    if stale:
        _build.build_host()
    spec = importlib.util.spec_from_file_location("_mlxcel_host", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_mlxcel_host"] = mod
    return mod


_host = sys.modules.get("_mlxcel_host") or _load()

BlockManager = _host.BlockManager
TickAction = _host.TickAction
TickState = _host.TickState
TickDecision = _host.TickDecision
decide_tick = _host.decide_tick
prefill_piece = _host.prefill_piece
