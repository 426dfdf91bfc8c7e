"""Builds the native libraries of the package in-tree with nvcc for sm_100a.

``python -m tuckmill_b200.build`` compiles ``csrc/*.cu`` into
``tuckmill_b200/libtm_cuda.so`` (the C ABI declared in ``include/tm_cuda.h``).
nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
OBJ = PKG / "build"
LIB = PKG / "libtm_cuda.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CUDA_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-Wall", "-I", str(ROOT / "include"), "-I", str(CSRC),
]


def _stale(target: Path, deps: list[Path]) -> bool:
    return not target.exists() or any(d.stat().st_mtime > target.stat().st_mtime for d in deps)


def build(verbose: bool = False, force: bool = False) -> Path:
    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.hpp")) + list((ROOT / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.name + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [NVCC, *CUDA_FLAGS, "-Xptxas", "-v" if verbose else "-warn-spills", "-x", "cu",
                   "-c", str(src), "-o", str(obj)]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))

    with ThreadPoolExecutor(max_workers=min(8, len(jobs) or 1)) as ex:
        list(ex.map(run, jobs))
    if jobs or not LIB.exists():
        run([NVCC, "-shared", "-o", str(LIB), *map(str, objs), "-Xlinker", "--no-undefined",
             "-ldl", "-lpthread"])
    build_engine(verbose, force)
    return LIB


ENGINE_LIB = PKG / "libtm_engine.so"
CXX = os.environ.get("CXX", "g++")


def build_engine(verbose: bool = False, force: bool = False) -> Path:
    """The C++ host layer (csrc/engine) -> libtm_engine.so, linked against
    libtm_cuda.so next to it (rpath $ORIGIN)."""
    src_dir = CSRC / "engine"
    sources = sorted(src_dir.glob("*.cpp"))
    deps = sources + list(src_dir.glob("*.hpp")) + list((ROOT / "include").glob("*.h")) + [LIB]
    if not force and not _stale(ENGINE_LIB, deps):
        return ENGINE_LIB
    cmd = [CXX, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-Wextra", "-I", str(ROOT / "include"),
           "-I", str(src_dir), *map(str, sources), "-o", str(ENGINE_LIB),
           "-L", str(PKG), "-ltm_cuda", "-Wl,-rpath,$ORIGIN",
           "-Wl,--no-undefined", "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("engine build failed: " + " ".join(cmd))
    return ENGINE_LIB


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
