"""Builds libkiln_cuda.so (and the host-scheduler library) in-tree for sm_100a.

Run as ``python -m kiln_b200.build``. nvcc cross-compiles without a GPU. The shared objects land
next to this file so that they travel with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_CUDA = PKG / "libkiln_cuda.so"
LIB_HOST = PKG / "libkiln_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libkiln_cuda.so cannot be built")
    return nvcc


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(s.stat().st_mtime > t for s in sources)


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    cu = sorted(CSRC.glob("*.cu"))
    deps = cu + sorted(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "kiln_cuda.h"]
    if not force and not _stale(LIB_CUDA, deps):
        return LIB_CUDA
    objs = []
    build_dir = PKG / "build"
    build_dir.mkdir(exist_ok=True)
    procs = []
    for src in cu:
        obj = build_dir / (src.stem + ".o")
        objs.append(obj)
        if not force and not _stale(obj, [src] + deps[len(cu):]):
            continue
        cmd = [_nvcc(), *NVCC_FLAGS, *os.environ.get("KILN_B200_NVCC_FLAGS", "").split(), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
        if verbose and out:
            print(out)
    cmd = [_nvcc(), "-shared", "-o", str(LIB_CUDA), *map(str, objs), "-lnccl", "-lcudart"]
    subprocess.run(cmd, check=True)
    return LIB_CUDA


def build_host(force: bool = False) -> Path:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    deps = srcs + sorted((CSRC / "host").glob("*.hpp")) + [PKG.parent / "include" / "kiln_host.h"]
    if not srcs:
        return LIB_HOST
    if not force and not _stale(LIB_HOST, deps):
        return LIB_HOST
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall",
           "-o", str(LIB_HOST), *map(str, srcs)]
    subprocess.run(cmd, check=True)
    return LIB_HOST


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(LIB_CUDA)
    print(LIB_HOST)
