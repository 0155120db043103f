"""In-tree build of the native libraries.

Two shared objects are produced under ``mini_trainer_b200/_native``:

* ``libmtb200_host.so``   — C++ host code (the LPT/greedy packers), built with g++.
* ``libmtb200_cuda.so``   — every sm_100a CUDA kernel, built with nvcc
  (``-gencode arch=compute_100a,code=sm_100a``). nvcc cross-compiles without a GPU.

Both expose a plain C ABI and are loaded with ``ctypes``; nothing here needs the torch C++
headers, so a full rebuild takes seconds rather than minutes.

Run ``python -m mini_trainer_b200.build`` to (re)build; ``build_all()`` is incremental (it
compares source and header mtimes with the output's).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_native"

HOST_LIB = OUT / "libmtb200_host.so"
CUDA_LIB = OUT / "libmtb200_cuda.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.stderr.strip() and os.environ.get("MTB200_BUILD_VERBOSE"):
        sys.stderr.write(proc.stderr)


def build_host(force: bool = False) -> Path:
    OUT.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cpp"))
    if force or _stale(HOST_LIB, srcs):
        _run(["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-o", str(HOST_LIB)] + [str(s) for s in srcs])
    return HOST_LIB


def cuda_sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build_cuda(force: bool = False, verbose_ptxas: bool = False) -> Path | None:
    """Compiles every ``csrc/*.cu`` to an object and links one shared library."""
    nvcc = _nvcc()
    if nvcc is None:
        return CUDA_LIB if CUDA_LIB.exists() else None
    OUT.mkdir(exist_ok=True)
    objdir = OUT / "obj"
    objdir.mkdir(exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    objs, relink = [], force
    procs = []
    for src in cuda_sources():
        obj = objdir / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + ["-c", str(src), "-o", str(obj)]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)))
            relink = True
    for cmd, p in procs:
        out, err = p.communicate()
        if p.returncode != 0:
            raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + out + err)
        if verbose_ptxas:
            sys.stderr.write(err)
    if relink or not CUDA_LIB.exists():
        _run([nvcc, "-shared", "-o", str(CUDA_LIB)] + [str(o) for o in objs] + ["-gencode", "arch=compute_100a,code=sm_100a"])
    return CUDA_LIB


def build_all(force: bool = False, verbose_ptxas: bool = False) -> None:
    build_host(force)
    build_cuda(force, verbose_ptxas)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose_ptxas="-v" in sys.argv)
    print("built:", HOST_LIB.exists() and HOST_LIB, CUDA_LIB.exists() and CUDA_LIB)
