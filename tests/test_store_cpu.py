"""Local model store: listing, sorting, removal guards, HuggingFace-cache reuse, CLI verbs."""
import json
import os

import pytest

from mlxcel_b200 import cli, store


def _mk(root, rid, nbytes, mtime):
    p = root.joinpath(*rid.split("/"))
    p.mkdir(parents=True)
    (p / "config.json").write_text("{}")
    (p / "model.safetensors").write_bytes(b"x" * nbytes)
    for f in p.iterdir():
        os.utime(f, (mtime, mtime))
    return p


def test_list_sort_and_format(tmp_path):
    _mk(tmp_path, "org/alpha", 5000, 1_000_000)
    _mk(tmp_path, "org/beta", 100, 3_000_000)
    _mk(tmp_path, "solo", 2000, 2_000_000)
    (tmp_path / "org" / "notamodel").mkdir()
    assert [m.repo_id for m in store.list_models(str(tmp_path))] == ["org/alpha", "org/beta", "solo"]
    assert [m.repo_id for m in store.list_models(str(tmp_path), "size")] == ["org/alpha", "solo", "org/beta"]
    assert [m.repo_id for m in store.list_models(str(tmp_path), "modified")] == ["org/beta", "solo", "org/alpha"]
    table = store.format_table(store.list_models(str(tmp_path)), verbose=True)
    assert table.splitlines()[0].split() == ["NAME", "SIZE", "MODIFIED", "PATH"] and "5.0 KB" in table
    assert store.human_age(100.0, now=100.0 + 3 * 86400) == "3 days ago" and store.human_age(None) == "-"


def test_remove_guards_and_frees(tmp_path):
    p = _mk(tmp_path, "org/alpha", 5000, 1_000_000)
    with pytest.raises(ValueError):
        store.remove_model("../outside", str(tmp_path))
    with pytest.raises(ValueError):
        store.model_path("a/b/c", str(tmp_path))
    with pytest.raises(FileNotFoundError):
        store.remove_model("org/missing", str(tmp_path))
    assert store.remove_model("org/alpha", str(tmp_path)) >= 5000
    assert not p.exists() and not (tmp_path / "org").exists() and tmp_path.exists()


def test_download_links_huggingface_cache_copy(tmp_path, monkeypatch):
    hub = tmp_path / "hub"
    snap = hub / "models--org--gamma" / "snapshots" / "abc123"
    snap.mkdir(parents=True)
    (snap / "config.json").write_text("{}")
    monkeypatch.setenv("HF_HUB_CACHE", str(hub))
    monkeypatch.setenv("MLXCEL_B200_MODELS_DIR", str(tmp_path / "store"))
    dest = store.download_model("org/gamma")
    assert dest.is_symlink() and (dest / "config.json").exists()
    assert [m.repo_id for m in store.list_models()] == ["org/gamma"]
    assert store.remove_model("org/gamma") == 0 and snap.exists()          # only the link goes
    with pytest.raises(RuntimeError):
        store.download_model("org/nowhere")


def test_cli_verbs(tmp_path, capsys):
    _mk(tmp_path, "org/alpha", 10, 1_000_000)
    cli.main(["list", "--models-dir", str(tmp_path), "--json"])
    rows = json.loads(capsys.readouterr().out)
    assert rows[0]["repo_id"] == "org/alpha" and rows[0]["size_bytes"] >= 10
    cli.main(["ls", "--models-dir", str(tmp_path), "-q"])
    assert capsys.readouterr().out.strip() == "org/alpha"
    cli.main(["rm", "org/alpha", "--models-dir", str(tmp_path), "--yes"])
    assert "removed org/alpha" in capsys.readouterr().out
    with pytest.raises(SystemExit):
        cli.main(["rm", "org/alpha", "--models-dir", str(tmp_path), "--yes"])


def test_resolve_model_prefers_paths_then_store(tmp_path, monkeypatch):
    monkeypatch.setenv("MLXCEL_B200_MODELS_DIR", str(tmp_path))
    monkeypatch.setenv("HF_HUB_CACHE", str(tmp_path / "nohub"))
    p = _mk(tmp_path, "org/alpha", 10, 1_000_000)
    assert store.resolve_model("org/alpha") == str(p)
    assert store.resolve_model(str(p)) == str(p)
    assert store.resolve_model("preset:tiny-llama") == "preset:tiny-llama"
    assert store.resolve_model("org/unknown") == "org/unknown"
