"""Autotuner contract: bucketing, cache invalidation, precedence, inert default, the tune loop and CLI."""
import json

import pytest

from mlxcel_b200 import autotune as at
from mlxcel_b200 import cli

STAMP = dict(format=at.FORMAT, package="t", torch="t", cuda="t", device="fake B200")


def test_buckets_round_up_to_powers_of_two():
    assert [at.bucket(n) for n in (0, 1, 2, 3, 4, 5, 1000, 1024, 1025)] == [1, 1, 2, 4, 4, 8, 1024, 1024, 2048]
    a, b = at.Geometry(hidden=4000), at.Geometry(hidden=4096)
    assert a.key() == b.key() != at.Geometry(hidden=4097).key()


def _fake_runner(table):
    calls = []

    def run(op, value, geo):
        calls.append((op.name, value))
        t = table[op.name][value]
        if t is None:
            raise RuntimeError("candidate does not launch")
        return t
    run.calls = calls
    return run


def test_tune_picks_fastest_keeps_default_on_ties_and_skips_failures(tmp_path):
    store = at.TacticStore(tmp_path / "t.json", STAMP)
    run = _fake_runner({"gemm-prefill-raster": {"0": 130.0, "4": 110.0, "8": 100.0, "16": 100.5, "32": None},
                        "gemm-decode-stages": {"0": 50.0, "3": 40.0, "4": 45.0, "6": 41.0, "8": 60.0},
                        "qmv-max-rows": {"1": None, "2": None, "4": None, "8": None}})
    res = {r.op: r for r in at.tune(["gemm-prefill-raster", "gemm-decode-stages", "qmv-max-rows"], at.Geometry(), store, run)}
    assert res["gemm-prefill-raster"].value == "16"          # within 1 % of the best: the default stays
    assert "32" not in res["gemm-prefill-raster"].tried
    assert res["gemm-decode-stages"].value == "3" and res["gemm-decode-stages"].us == 40.0
    assert res["qmv-max-rows"].skipped and store.lookup("qmv-max-rows", at.Geometry()) is None
    again = at.TacticStore(tmp_path / "t.json", STAMP)
    assert again.lookup("gemm-decode-stages", at.Geometry())["value"] == "3"
    other = at.TacticStore(tmp_path / "t.json", dict(STAMP, device="another GPU"))
    assert other.tactics == {} and other.discarded          # measured elsewhere: not applied


def test_resolve_precedence_and_inert_default(tmp_path):
    geo = at.Geometry()
    store = at.TacticStore(tmp_path / "t.json", STAMP)
    store.put("gemm-decode-stages", geo, "6", 1.0, {})
    run = _fake_runner({"gemm-prefill-raster": {"0": 1.0, "4": 9.0, "8": 9.0, "16": 9.0, "32": 9.0}})
    assert at.resolve("gemm-decode-stages", geo, store, run, environ={}) == ("0", "default")           # switch unset
    assert at.resolve("gemm-decode-stages", geo, store, run, environ={at.SWITCH: "cache"}) == ("6", "cache")
    env = {at.SWITCH: "cache", "MLXCEL_B200_GEMM_STAGES": "4"}
    assert at.resolve("gemm-decode-stages", geo, store, run, environ=env) == ("4", "env")
    assert at.resolve("gemm-prefill-raster", geo, store, run, environ={at.SWITCH: "cache"}) == ("16", "default")
    assert run.calls == []                                   # cache mode never profiles
    assert at.resolve("gemm-prefill-raster", geo, store, run, environ={at.SWITCH: "1"}) == ("0", "profiled")
    assert at.resolve("gemm-prefill-raster", geo, store, run, environ={at.SWITCH: "cache"}) == ("0", "cache")


def test_apply_cached_exports_only_when_switched_on(tmp_path):
    geo = at.Geometry()
    store = at.TacticStore(tmp_path / "t.json", STAMP)
    store.put("gemm-decode-stages", geo, "6", 1.0, {})
    store.put("gemm-prefill-raster", geo, "16", 1.0, {})          # the default: nothing to export
    env: dict = {}
    assert at.apply_cached(geo, store, env) == {} and env == {}
    env = {at.SWITCH: "cache", "MLXCEL_B200_GEMM_L2_PREFETCH_KB": "64"}
    assert at.apply_cached(geo, store, env) == {"MLXCEL_B200_GEMM_STAGES": ("6", "cache")}
    assert env["MLXCEL_B200_GEMM_STAGES"] == "6" and env["MLXCEL_B200_GEMM_L2_PREFETCH_KB"] == "64"
    store.put("gemm-decode-stages", at.Geometry(hidden=8192), "3", 1.0, {})
    env = {at.SWITCH: "cache"}
    assert at.apply_cached(None, store, env) == {}              # geometries disagree and none was named


def test_tune_cli_dry_run_prints_matrix(capsys):
    cli.main(["tune", "--dry-run", "--json", "--op", "gemm-prefill-raster", "-m", "preset:tiny-llama"])
    doc = json.loads(capsys.readouterr().out)
    assert [r["value"] for r in doc["matrix"]] == ["0", "4", "8", "16", "32"] and doc["geometry"].startswith("h")
    with pytest.raises(SystemExit):
        cli.main(["tune", "--dry-run", "--op", "nope"])
