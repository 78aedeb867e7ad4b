"""In-tree native build.

Two artefacts are produced next to the sources (never in a user cache, so that a copied
tree carries them):

* ``mlxcel_b200/lib/libmlxcel_b200.so`` — the sm_100a CUDA kernel library (plain C ABI,
  declared in ``csrc/api.h``), compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``mlxcel_b200/lib/_mlxcel_host*.so`` — the C++ host runtime (block manager, page-table
  builder, scheduler core, prompt-cache trie) as a pybind11 module.

Objects are rebuilt only when their source (or a shared header) is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
LIB = PKG / "lib"
OBJ = LIB / "obj"

CUDA_LIB = LIB / "libmlxcel_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc")
    if cand:
        return cand
    p = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "bin" / "nvcc"
    return str(p) if p.exists() else None


def _newer(src: Path, dst: Path, extra: list[Path]) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(s.stat().st_mtime > t for s in [src, *extra])


def host_ext_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return LIB / f"_mlxcel_host{suffix}"


def build_cuda(verbose: bool = False, force: bool = False) -> Path:
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernel library")
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    logs: dict[str, str] = {}

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        if force or _newer(src, obj, headers):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            logs[src.name] = r.stderr
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stderr[-4000:]}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or not CUDA_LIB.exists() or any(o.stat().st_mtime > CUDA_LIB.stat().st_mtime for o in objs):
        cmd = [nvcc, "-shared", "-o", str(CUDA_LIB), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    if logs:
        (LIB / "ptxas_info.txt").write_text(
            "\n".join(f"==== {k}\n{v}" for k, v in sorted(logs.items())))
    if verbose:
        for k, v in sorted(logs.items()):
            print(f"==== {k}\n{v}")
    return CUDA_LIB


def build_host(force: bool = False) -> Path:
    import pybind11

    LIB.mkdir(parents=True, exist_ok=True)
    out = host_ext_path()
    sources = sorted(HOST.glob("*.cpp"))
    headers = sorted(HOST.glob("*.h"))
    if not sources:
        raise RuntimeError("no host sources")
    if not force and out.exists() and all(
            s.stat().st_mtime <= out.stat().st_mtime for s in [*sources, *headers]):
        return out
    cxx = shutil.which("g++") or "g++"
    inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{HOST}"]
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", *inc,
           *map(str, sources), "-o", str(out), "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host build failed:\n{r.stderr[-4000:]}")
    return out


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_host(force=force)
    build_cuda(verbose=verbose, force=force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built:", CUDA_LIB, host_ext_path())
