"""Every MLXCEL_B200_* literal in the sources is documented; the tracer writes a loadable trace."""
import json
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_every_env_var_is_documented():
    doc = (ROOT / "docs" / "environment-variables.md").read_text()
    pat = re.compile(r"MLXCEL_B200_[A-Z0-9_]+")
    used = set()
    files = [ROOT / "bench.py", ROOT / "__graft_entry__.py"] + list((ROOT / "benchmarks").glob("*.py"))
    for ext in ("*.py", "*.cu", "*.cuh", "*.h", "*.cpp"):
        files += list((ROOT / "mlxcel_b200").rglob(ext))
    for f in files:
        used |= set(pat.findall(f.read_text(errors="ignore")))
    missing = sorted(v for v in used if f"`{v}`" not in doc)
    assert not missing, f"undocumented environment variables: {missing}"


def test_tracer_writes_chrome_trace(tmp_path):
    from mlxcel_b200.utils.tracing import Tracer
    t = Tracer()
    with t.span("noop"):      # inactive: no events
        pass
    assert t.events == []
    out = tmp_path / "trace.json"
    t.enable(path=str(out))
    with t.span("step", cat="engine", decode=3, prefill_tokens=17):
        with t.span("forward"):
            pass
    t.instant("finished", seq=1)
    t.flush()
    doc = json.loads(out.read_text())
    names = [e["name"] for e in doc["traceEvents"]]
    assert names == ["forward", "step", "finished"]
    step = doc["traceEvents"][1]
    assert step["ph"] == "X" and step["dur"] >= doc["traceEvents"][0]["dur"] and step["args"]["decode"] == 3
