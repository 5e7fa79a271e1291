"""Builds libizwi_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU)."""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libizwi_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-shared",
]


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


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB_PATH
    nvcc = os.environ.get("NVCC") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH), *map(str, sources()), "-ldl"]
    env = dict(os.environ)
    # the image exports CC/CXX pointing at a gcc wrapper without its runtime specs; use the system one
    env.pop("CC", None)
    env.pop("CXX", None)
    proc = subprocess.run(cmd, capture_output=True, text=True, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
