"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``libowl_b200_cuda.so`` -- every ``csrc/*.cu`` kernel file, compiled by nvcc for sm_100a
  only (``-gencode arch=compute_100a,code=sm_100a``) with a static CUDA runtime, exposing
  plain ``extern "C"`` launchers that take raw device pointers and a ``cudaStream_t``.
* ``libowl_b200_host.so`` -- the host-side C++ runtime (``csrc/host/*.cpp``): store core,
  GGUF reader / block codecs, pinned staging, ledger.

The launchers are called through ``ctypes`` (see ``owl_engine_b200._native``), so no torch
headers are involved and a rebuild takes seconds per file. The reference builds per-``.cu``
fatbins in ``crates/kernels/build.rs``; here there is exactly one target architecture.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE.parent / "csrc"
OBJ = HERE / "build"
CUDA_LIB = HERE / "libowl_b200_cuda.so"
HOST_LIB = HERE / "libowl_b200_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-cudart", "static",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall"]


def _nvcc() -> str:
    for cand in (os.environ.get("OWL_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; cannot build the sm_100a kernels")


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _run(cmd: list[str]) -> str:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("native build failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_cuda(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    stamp = OBJ / "cuda.stamp"
    dig = _digest(srcs + hdrs, " ".join(NVCC_FLAGS))
    if not force and CUDA_LIB.exists() and stamp.exists() and stamp.read_text() == dig:
        return CUDA_LIB
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    hdig = _digest(hdrs, " ".join(NVCC_FLAGS))

    def one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        ostamp = OBJ / (src.stem + ".stamp")
        d = hashlib.sha256((hdig + src.read_text()).encode()).hexdigest()
        if not force and obj.exists() and ostamp.exists() and ostamp.read_text() == d:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd[1:1] = ["-Xptxas", "-v"]
        out = _run(cmd)
        if verbose or ptxas_info:
            print(out, file=sys.stderr)
        ostamp.write_text(d)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(one, srcs))
    _run([nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
          "-Xcompiler", "-fPIC", "-o", str(CUDA_LIB), *map(str, objs), "-ldl", "-lrt", "-lpthread"])
    stamp.write_text(dig)
    return CUDA_LIB


def build_host(force: bool = False) -> Path | None:
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    if not srcs:
        return None
    hdrs = sorted((CSRC / "host").glob("*.h"))
    stamp = OBJ / "host.stamp"
    dig = _digest(srcs + hdrs, " ".join(CXX_FLAGS))
    if not force and HOST_LIB.exists() and stamp.exists() and stamp.read_text() == dig:
        return HOST_LIB
    OBJ.mkdir(exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    _run([cxx, *CXX_FLAGS, "-shared", "-I", str(CSRC / "host"), "-o", str(HOST_LIB), *map(str, srcs), "-lrt"])
    stamp.write_text(dig)
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> dict:
    out = {"cuda": str(build_cuda(force, verbose, ptxas_info)), "host": None}
    h = build_host(force)
    out["host"] = str(h) if h else None
    return out


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser(description="build the owl_engine_b200 native libraries in-tree")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--ptxas-info", action="store_true", help="print registers / spills / smem per kernel")
    a = ap.parse_args()
    print(json.dumps(build_all(a.force, True, a.ptxas_info)))
