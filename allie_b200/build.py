"""Builds the native libraries of the package in-tree.

Every ``csrc/*.cu`` file is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``) into one shared library,
``allie_b200/lib/liballie_b200.so``, with a plain C ABI that the Python side
binds through ``ctypes``.  Host-only C++ (chess move generation, MCTS) goes
into ``allie_b200/lib/liballie_host.so`` with g++.  Objects are rebuilt only
when their source (or a header) is newer.

Run ``python -m allie_b200.build`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--use_fast_math",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-march=x86-64-v2", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header_mtime(exts) -> float:
    m = 0.0
    for ext in exts:
        for h in CSRC.glob(f"*{ext}"):
            m = max(m, h.stat().st_mtime)
    return m


def _compile(cmd: list[str], log: Path) -> None:
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    hdr = _newest_header_mtime([".cuh", ".h"])
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            jobs.append((cmd, OBJ / (src.stem + ".log")))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(lambda j: _compile(*j), jobs))
    out = LIB / "liballie_b200.so"
    if jobs or not out.exists():
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(out), *map(str, objs), "-cudart", "static"]
        _compile(cmd, OBJ / "link.log")
    if verbose:
        for src in sources:
            log = OBJ / (src.stem + ".log")
            if log.exists():
                print(log.read_text())
    return out


def build_host(force: bool = False) -> Path | None:
    OBJ.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cpp"))
    if not sources:
        return None
    out = LIB / "liballie_host.so"
    hdr = _newest_header_mtime([".hpp", ".h"])
    newest = max([s.stat().st_mtime for s in sources] + [hdr])
    if force or not out.exists() or out.stat().st_mtime < newest:
        cxx = os.environ.get("CXX", "g++")
        cmd = [cxx, *CXX_FLAGS, "-shared", "-I", str(CSRC), "-o", str(out), *map(str, sources)]
        _compile(cmd, OBJ / "host.log")
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_host(force)
    build_cuda(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", *(p.name for p in LIB.glob("*.so")))
