"""Local model store: where downloaded checkpoints live, listing them, removing one, and reuse of an
existing HuggingFace cache copy.

Reference behaviour (src/main.rs:161 ``list``, :199 ``download``, :328 ``rm``; src/commands/models.rs):
snapshots sit under ``<store>/<owner>/<name>``; the store root is ``--models-dir``, else
``$MLXCEL_B200_MODELS_DIR``, else ``${MLXCEL_B200_CACHE_DIR:-$HOME/.cache/mlxcel_b200}/models``;
``list`` prints NAME / SIZE / MODIFIED (``--json``, ``-q``, ``-v``, ``--sort``), ``rm`` deletes one
snapshot after confirmation and never touches the HuggingFace cache, ``download`` first looks for the
repository in the HuggingFace cache and links that copy instead of fetching it again. There is no
network fetch here: a repository that is in neither place is reported as such.
"""
from __future__ import annotations

import os
import shutil
import time
from dataclasses import asdict, dataclass
from pathlib import Path


@dataclass
class StoredModel:
    repo_id: str
    path: str
    size_bytes: int
    modified: float | None


def store_root(models_dir: str | None = None) -> Path:
    if models_dir:
        return Path(models_dir).expanduser()
    env = os.environ.get("MLXCEL_B200_MODELS_DIR")
    if env:
        return Path(env).expanduser()
    cache = os.environ.get("MLXCEL_B200_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "mlxcel_b200")
    return Path(cache) / "models"


def _tree_stats(p: Path) -> tuple[int, float | None]:
    size, newest = 0, None
    for root, _, files in os.walk(p, followlinks=True):
        for f in files:
            try:
                st = os.stat(os.path.join(root, f))
            except OSError:
                continue
            size += st.st_size
            newest = st.st_mtime if newest is None else max(newest, st.st_mtime)
    return size, newest


def list_models(models_dir: str | None = None, sort: str = "name") -> list[StoredModel]:
    """Every ``<owner>/<name>`` (or top-level ``<name>``) directory of the store holding a ``config.json``."""
    root = store_root(models_dir)
    out: list[StoredModel] = []
    if not root.is_dir():
        return out
    for a in sorted(root.iterdir()):
        if not a.is_dir():
            continue
        cands = [(a.name, a)] if (a / "config.json").exists() else [
            (f"{a.name}/{b.name}", b) for b in sorted(a.iterdir()) if b.is_dir() and (b / "config.json").exists()]
        for rid, p in cands:
            size, mod = _tree_stats(p)
            out.append(StoredModel(rid, str(p.resolve()), size, mod))
    if sort == "size":
        out.sort(key=lambda m: -m.size_bytes)
    elif sort == "modified":
        out.sort(key=lambda m: (m.modified is None, -(m.modified or 0.0)))
    else:
        out.sort(key=lambda m: m.repo_id)
    return out


def human_size(n: int) -> str:
    x = float(n)
    for unit in ("B", "KB", "MB", "GB", "TB"):
        if x < 1000.0 or unit == "TB":
            return f"{x:.0f} {unit}" if unit == "B" else f"{x:.1f} {unit}"
        x /= 1000.0
    return f"{n} B"


def human_age(ts: float | None, now: float | None = None) -> str:
    if ts is None:
        return "-"
    d = max(0.0, (now if now is not None else time.time()) - ts)
    for span, name in ((86400 * 365, "year"), (86400 * 30, "month"), (86400 * 7, "week"), (86400, "day"),
                       (3600, "hour"), (60, "minute")):
        if d >= span:
            k = int(d // span)
            return f"{k} {name}{'s' if k != 1 else ''} ago"
    return "just now"


def format_table(models: list[StoredModel], verbose: bool = False) -> str:
    rows = [("NAME", "SIZE", "MODIFIED") + (("PATH",) if verbose else ())]
    for m in models:
        rows.append((m.repo_id, human_size(m.size_bytes), human_age(m.modified)) + ((m.path,) if verbose else ()))
    w = [max(len(r[i]) for r in rows) for i in range(len(rows[0]))]
    return "\n".join("  ".join(c.ljust(w[i]) for i, c in enumerate(r)).rstrip() for r in rows)


def as_json(models: list[StoredModel]) -> list[dict]:
    return [asdict(m) for m in models]


def _check_repo_id(repo_id: str) -> list[str]:
    parts = repo_id.strip("/").split("/")
    if not 1 <= len(parts) <= 2 or any(p in ("", ".", "..") or os.sep in p for p in parts):
        raise ValueError(f"not a repository id: {repo_id!r} (expected owner/name)")
    return parts


def model_path(repo_id: str, models_dir: str | None = None) -> Path:
    return store_root(models_dir).joinpath(*_check_repo_id(repo_id))


def hf_cache_snapshot(repo_id: str) -> Path | None:
    """Newest snapshot directory of ``repo_id`` in the HuggingFace hub cache, if any."""
    hub = os.environ.get("HF_HUB_CACHE") or os.path.join(
        os.environ.get("HF_HOME") or os.path.join(os.path.expanduser("~"), ".cache", "huggingface"), "hub")
    snaps = Path(hub) / ("models--" + "--".join(_check_repo_id(repo_id))) / "snapshots"
    if not snaps.is_dir():
        return None
    cands = [p for p in snaps.iterdir() if (p / "config.json").exists()]
    return max(cands, key=lambda p: p.stat().st_mtime) if cands else None


def remove_model(repo_id: str, models_dir: str | None = None) -> int:
    """Delete one snapshot of the store; returns the bytes freed. Refuses anything that does not resolve
    to a directory strictly inside the store root."""
    root = store_root(models_dir).resolve()
    target = model_path(repo_id, models_dir)
    if not target.exists():
        where = hf_cache_snapshot(repo_id)
        hint = f" (a copy exists in the HuggingFace cache at {where}; that cache is not managed here)" if where else ""
        raise FileNotFoundError(f"{repo_id} is not in the store {root}{hint}")
    if target.is_symlink():                      # a link into the HuggingFace cache: drop the link only
        target.unlink()
        freed = 0
    else:
        real = target.resolve()
        if root == real or root not in real.parents:
            raise ValueError(f"refusing to remove {real}: outside the store {root}")
        freed, _ = _tree_stats(real)
        shutil.rmtree(real)
    parent = target.parent
    if parent != store_root(models_dir) and parent.is_dir() and not any(parent.iterdir()):
        parent.rmdir()
    return freed


def download_model(repo_id: str, models_dir: str | None = None, local_dir: str | None = None) -> Path:
    """Make ``repo_id`` available in the store. An existing store copy is returned as is; a HuggingFace
    cache copy is linked in; otherwise the fetch would need the network, which this build does not use."""
    dest = Path(local_dir).expanduser() if local_dir else model_path(repo_id, models_dir)
    if (dest / "config.json").exists():
        return dest
    snap = hf_cache_snapshot(repo_id)
    if snap is None:
        raise RuntimeError(f"{repo_id}: not in the store and not in the HuggingFace cache; fetching from the hub is "
                           f"not available in this build (place the snapshot at {dest})")
    dest.parent.mkdir(parents=True, exist_ok=True)
    os.symlink(snap.resolve(), dest, target_is_directory=True)
    return dest


def resolve_model(ref: str, models_dir: str | None = None) -> str:
    """Turn what ``-m`` was given into a directory: an existing path stays; an ``owner/name`` id is looked
    up in the store, then in the HuggingFace cache; anything else is returned unchanged for the loader
    to report."""
    if ref.startswith("preset:") or os.path.exists(ref):
        return ref
    try:
        p = model_path(ref, models_dir)
    except ValueError:
        return ref
    if (p / "config.json").exists():
        return str(p)
    snap = hf_cache_snapshot(ref)
    return str(snap) if snap is not None else ref
