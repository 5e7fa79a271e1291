"""Builds libizwi_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libizwi_b200.so"

COMPILE_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]
OBJ_DIR = PKG_DIR / "csrc" / ".obj"


HOST_SELFTEST = PKG_DIR / "host" / "host_selftest"


def build_host_selftest() -> Path:
    """The C++ host layer's own test program (links the library; rpath points back at it)."""
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O2", "-std=c++17", "-o", str(HOST_SELFTEST), str(PKG_DIR / "host" / "host_selftest.cpp"),
           "-L", str(PKG_DIR), "-lizwi_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."]
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    return HOST_SELFTEST


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*")) + [PKG_DIR.parent / "include" / "izwi_b200.h"]
    return any(p.stat().st_mtime > built for p in deps if p.is_file())


def _run(cmd: list[str], env: dict) -> str:
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Every source file is compiled to an object of its own (in parallel; an object newer than its
    source and every header is reused), then the objects are linked into the shared library."""
    if not force and not needs_build():
        return LIB_PATH
    from concurrent.futures import ThreadPoolExecutor
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a gcc wrapper without its runtime specs; use the system one
    env.pop("CC", None)
    env.pop("CXX", None)
    OBJ_DIR.mkdir(exist_ok=True)
    headers = [p for p in CSRC.glob("*") if p.suffix in (".cuh", ".h", ".hpp")] + [PKG_DIR.parent / "include" / "izwi_b200.h"]
    newest_header = max(p.stat().st_mtime for p in headers)
    jobs, objects = [], []
    for src in sources():
        obj = OBJ_DIR / (src.name + ".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header):
            cmd = [nvcc, *COMPILE_FLAGS, *(["-Xptxas", "-v"] if verbose else []), "-c", "-o", str(obj), str(src)]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        logs = list(pool.map(lambda c: _run(c, env), jobs))
    if verbose:
        print("\n".join(logs))
    # linked under another name and moved into place, so a reader never sees a half-written library
    tmp = LIB_PATH.with_suffix(".so.tmp")
    _run([nvcc, "-shared", "-o", str(tmp), *map(str, objects), "-ldl"], env)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
