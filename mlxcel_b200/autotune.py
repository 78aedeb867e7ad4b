"""Offline kernel autotuner: profile the launch knobs of the hot kernels on this machine, keep the
winners in a cache file, apply them at process start.

Reference contract (src/lib/mlxcel-core/src/autotune/{mod,bucket,store,tactic,profile}.rs,
src/commands/tune.rs): tactics are keyed by (op, shape bucket, extras) with shapes rounded up to
powers of two; a cached tactic carries the environment it was measured in (package version, library
versions, device) and is discarded on any mismatch; precedence is explicit environment variable >
valid cached tactic > tactic profiled now > the op's default; with the switch variable unset the
tuner is inert (no file is read); ``tune`` profiles offline and writes the cache, and nothing
consumes it until the switch is set.

Design here. The tunable knobs of this package are read once per process by the native library
(``MLXCEL_B200_GEMM_STAGES``, ``MLXCEL_B200_GEMM_RASTER``, ...), so a candidate is measured in a
child process started with that variable set (``python -m mlxcel_b200.autotune --measure ...``, CUDA
events around the op after warm-up, L2 flushed between iterations), and a cached tactic is applied by
exporting the variable before the library is loaded (:func:`apply_cached`, called from the library
loader). ``MLXCEL_B200_AUTOTUNE=cache`` applies cached tactics; ``=1`` additionally profiles an op
whose bucket has no entry the first time it is resolved. The model geometry (hidden size,
intermediate size, head geometry) is the shape key: one serving process runs one model.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable

SWITCH = "MLXCEL_B200_AUTOTUNE"
FORMAT = 1


def bucket(n: int) -> int:
    """Round up to a power of two (minimum 1): nearby shapes share one entry."""
    n = max(1, int(n))
    return 1 << (n - 1).bit_length()


@dataclass(frozen=True)
class Geometry:
    """The shape key of a model: what the tuned kernels' problem sizes derive from."""
    hidden: int = 4096
    intermediate: int = 14336
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128

    @staticmethod
    def from_config(cfg) -> "Geometry":
        return Geometry(cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                        cfg.head_dim)

    def key(self) -> str:
        return f"h{bucket(self.hidden)}-i{bucket(self.intermediate)}-q{self.heads}-kv{self.kv_heads}-d{self.head_dim}"


@dataclass
class TunableOp:
    name: str
    env: str                        # the knob: an environment variable the native library reads once
    candidates: list[str]
    default: str
    what: str
    measure: str                    # name of the measurement routine run in the child process
    rows: int = 64                  # token rows of the measured problem

    def matrix(self) -> list[dict]:
        return [dict(op=self.name, env=self.env, value=v, default=v == self.default) for v in self.candidates]


OPS: dict[str, TunableOp] = {o.name: o for o in (
    TunableOp("gemm-decode-stages", "MLXCEL_B200_GEMM_STAGES", ["0", "3", "4", "6", "8"], "0",
              "shared-memory ring depth of the tcgen05 GEMM on decode-sized batches", "linear", rows=64),
    TunableOp("gemm-decode-l2-prefetch", "MLXCEL_B200_GEMM_L2_PREFETCH_KB", ["0", "32", "64", "128"], "0",
              "weight-slice L2 prefetch ahead of the dependent-launch wait on decode-sized batches", "linear", rows=64),
    TunableOp("gemm-prefill-raster", "MLXCEL_B200_GEMM_RASTER", ["0", "4", "8", "16", "32"], "16",
              "lane tiles per panel of the prefill tile walk", "linear", rows=8192),
    TunableOp("qmv-max-rows", "MLXCEL_B200_QMV_MAX_M", ["1", "2", "4", "8"], "1",
              "largest batch served by the quantized GEMV kernel before the fused dequant GEMM takes over",
              "qlinear", rows=4),
)}


def environment_stamp(device: str | None = None) -> dict:
    """What a cached tactic is only valid under: a mismatch in any field discards the entry."""
    import torch

    from . import __version__
    if device is None:
        device = torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu"
    return dict(format=FORMAT, package=__version__, torch=torch.__version__, cuda=str(torch.version.cuda), device=device)


def cache_dir() -> Path:
    root = os.environ.get("MLXCEL_B200_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "mlxcel_b200")
    return Path(root) / "autotune"


class TacticStore:
    """One JSON file per machine: ``{"stamp": {...}, "tactics": {"<op>|<geometry key>": {"value", "us", "tried"}}}``."""

    def __init__(self, path: str | Path | None = None, stamp: dict | None = None):
        self.path = Path(path) if path else cache_dir() / "tactics.json"
        self.stamp = stamp or environment_stamp()
        self.tactics: dict[str, dict] = {}
        self.discarded = False
        if self.path.exists():
            try:
                doc = json.loads(self.path.read_text())
            except (OSError, ValueError):
                doc = {}
            if doc.get("stamp") == self.stamp:
                self.tactics = dict(doc.get("tactics") or {})
            else:
                self.discarded = bool(doc)          # measured elsewhere or by another build: not applied

    @staticmethod
    def _key(op: str, geo: Geometry) -> str:
        return f"{op}|{geo.key()}"

    def lookup(self, op: str, geo: Geometry) -> dict | None:
        return self.tactics.get(self._key(op, geo))

    def put(self, op: str, geo: Geometry, value: str, us: float, tried: dict[str, float]) -> None:
        self.tactics[self._key(op, geo)] = dict(value=value, us=us, tried=tried, time=time.time())

    def save(self) -> None:
        self.path.parent.mkdir(parents=True, exist_ok=True)
        tmp = self.path.with_suffix(".tmp")
        tmp.write_text(json.dumps(dict(stamp=self.stamp, tactics=self.tactics), indent=1, sort_keys=True))
        os.replace(tmp, self.path)


Runner = Callable[[TunableOp, str, Geometry], float]        # -> microseconds of one launch


def child_runner(op: TunableOp, value: str, geo: Geometry, timeout: float = 300.0) -> float:
    """Measure one candidate in a fresh process (the native library reads its knobs once)."""
    env = dict(os.environ)
    env[op.env] = value
    env.pop(SWITCH, None)
    cmd = [sys.executable, "-m", "mlxcel_b200.autotune", "--measure", op.measure, "--rows", str(op.rows),
           "--geometry", json.dumps(geo.__dict__)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    if out.returncode != 0:
        raise RuntimeError(f"{op.name}={value}: measurement failed: {out.stderr.strip()[-400:]}")
    return float(json.loads(out.stdout.strip().splitlines()[-1])["us"])


@dataclass
class TuneResult:
    op: str
    value: str
    us: float
    tried: dict[str, float] = field(default_factory=dict)
    skipped: str | None = None


def tune(ops: list[str] | None, geo: Geometry, store: TacticStore, runner: Runner = child_runner,
         log: Callable[[str], None] | None = None) -> list[TuneResult]:
    """Profile every candidate of the chosen ops and record the fastest. A candidate whose measurement
    fails is left out; an op with no successful candidate keeps its default and gets no entry. Ties
    within 1 % go to the default so that noise does not move a knob."""
    results = []
    for name in ops or list(OPS):
        op = OPS[name]
        tried: dict[str, float] = {}
        for v in op.candidates:
            try:
                tried[v] = float(runner(op, v, geo))
            except Exception as e:  # noqa: BLE001 - a failing candidate is simply not eligible
                if log:
                    log(f"{op.name}: {op.env}={v} failed ({e})")
                continue
            if log:
                log(f"{op.name}: {op.env}={v} -> {tried[v]:.1f} us")
        if not tried:
            results.append(TuneResult(op.name, op.default, float("nan"), skipped="no candidate could be measured"))
            continue
        best = min(tried, key=tried.get)
        if op.default in tried and tried[op.default] <= tried[best] * 1.01:
            best = op.default
        store.put(op.name, geo, best, tried[best], tried)
        results.append(TuneResult(op.name, best, tried[best], tried))
    store.save()
    return results


def resolve(op_name: str, geo: Geometry, store: TacticStore | None = None, runner: Runner = child_runner,
            environ: dict | None = None) -> tuple[str, str]:
    """The value of one knob and where it came from (``env`` | ``cache`` | ``profiled`` | ``default``)."""
    environ = os.environ if environ is None else environ
    op = OPS[op_name]
    if environ.get(op.env) not in (None, ""):
        return environ[op.env], "env"
    mode = environ.get(SWITCH, "")
    if mode not in ("1", "cache"):
        return op.default, "default"                 # inert: nothing is read
    store = store or TacticStore()
    hit = store.lookup(op_name, geo)
    if hit is not None and hit.get("value") in op.candidates:
        return hit["value"], "cache"
    if mode == "1":
        res = tune([op_name], geo, store, runner)[0]
        if res.skipped is None:
            return res.value, "profiled"
    return op.default, "default"


def apply_cached(geo: Geometry | None = None, store: TacticStore | None = None, environ: dict | None = None) -> dict:
    """Export the cached knobs into the environment (before the native library reads them). Variables
    the user set stay as they are. Returns ``{variable: (value, source)}`` for the knobs that changed.
    With a geometry the matching entries are used; without one, an entry is used only when every
    geometry in the cache agrees on the value."""
    environ = os.environ if environ is None else environ
    if environ.get(SWITCH, "") not in ("1", "cache"):
        return {}
    store = store or TacticStore()
    changed = {}
    for op in OPS.values():
        if environ.get(op.env) not in (None, ""):
            continue
        if geo is not None:
            hit = store.lookup(op.name, geo)
            values = {hit["value"]} if hit else set()
        else:
            values = {t["value"] for k, t in store.tactics.items() if k.split("|", 1)[0] == op.name}
        if len(values) == 1:
            v = next(iter(values))
            if v in op.candidates and v != op.default:
                environ[op.env] = v
                changed[op.env] = (v, "cache")
    return changed


# ------------------------------------------------------------------ measurement (child process, needs a GPU)
def _measure(kind: str, rows: int, geo: Geometry, iters: int = 30, warmup: int = 5) -> float:
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("measurement needs a CUDA device")
    from . import ops
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(0)
    x = (torch.randn(rows, geo.hidden, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    shapes = [((geo.heads + 2 * geo.kv_heads) * geo.head_dim, geo.hidden), (2 * geo.intermediate, geo.hidden)]
    if kind == "qlinear":
        from .ops import quant
        ws = [quant.quantize((torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev), "affine", 4, 64)
              for n, k in shapes]
    else:
        ws = [(torch.randn(n, k, generator=g) * 0.02).to(torch.bfloat16).to(dev) for n, k in shapes]
    flush = torch.empty(160 * 1024 * 1024, dtype=torch.uint8, device=dev)      # larger than the L2

    def step():
        for w in ws:
            ops.linear(x, w)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        step()
        b.record()
        torch.cuda.synchronize()
        total += a.elapsed_time(b)
    return total / iters * 1e3


def main(argv: list[str] | None = None) -> None:
    import argparse

    ap = argparse.ArgumentParser(prog="python -m mlxcel_b200.autotune")
    ap.add_argument("--measure", required=True, choices=["linear", "qlinear"])
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--geometry", default="{}")
    a = ap.parse_args(argv)
    us = _measure(a.measure, a.rows, Geometry(**json.loads(a.geometry)))
    print(json.dumps(dict(us=us)))


if __name__ == "__main__":
    main()
