"""Ahead-of-time build of the sm_100a shared library (no JIT at call time).

The reference compiles every kernel variant at first use with NVCC/NVRTC (csrc/jit/compiler.hpp:117-140);
here all variants are compiled once, in-tree, into ``asymgemm_b200/lib/libasymgemm_b200.so``.
Run ``python -m asymgemm_b200.build`` (or ``__graft_entry__.build()``).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libasymgemm_b200.so"
TORCH_OPS_PATH = LIB_DIR / "libasymgemm_b200_torch.so"
TORCH_OPS_SRC = CSRC / "torch_ops.cpp"
OBJ_DIR = CSRC / "build"

SOURCES = ["capi.cu", "inst_bf16.cu", "inst_fp8.cu", "inst_int8.cu", "inst_fp4.cu", "inst_fp8_ue8m0.cu", "sf_layout.cu", "no_alloc.cu", "selftest.cu", "moe_glue.cu", "hostlink.cu", "ep_peer.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found (set NVCC or CUDA_HOME)")
    return cand


def _sources() -> list[Path]:
    return [CSRC / s for s in SOURCES if (CSRC / s).exists()]


def _deps() -> list[Path]:
    return _sources() + sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "asymgemm_b200.h"]


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(d.stat().st_mtime > t for d in _deps() if d.exists())


def build_torch_ops(force: bool = False) -> Path:
    """Compile the thin PyTorch extension (csrc/torch_ops.cpp: tensors -> C descriptor -> C ABI) with the host compiler
    against this interpreter's torch headers, linked to the C library that sits in the same folder."""
    header = PKG_DIR.parent / "include" / "asymgemm_b200.h"
    if not force and TORCH_OPS_PATH.exists() and all(
            TORCH_OPS_PATH.stat().st_mtime >= p.stat().st_mtime for p in (TORCH_OPS_SRC, header, LIB_PATH)):
        return TORCH_OPS_PATH
    import logging
    import torch
    logging.getLogger("torch.utils.cpp_extension").setLevel(logging.ERROR)
    from torch.utils import cpp_extension as ce
    cuda_home = os.environ.get("CUDA_HOME") or "/usr/local/cuda"
    tmp = TORCH_OPS_PATH.with_suffix(".so.tmp")
    # Host compilers to try, the system one first. The extension throws c10::Error across its boundary and formats
    # messages with iostreams, so it must share the process's libstdc++: a toolchain whose default link pulls in a static
    # libstdc++ (a private copy with its own, never initialised, locale) builds a library that crashes on its first
    # error message. The result is checked, and the next candidate is tried when libstdc++.so is not among its dependencies.
    cands = []
    for c in (os.environ.get("ASYMGEMM_CXX"), shutil.which("g++"), "/usr/bin/g++", os.environ.get("CXX")):
        if c and c not in cands and (Path(c).exists() or shutil.which(c)):
            cands.append(c)
    if not cands:
        raise RuntimeError("no host C++ compiler found (set ASYMGEMM_CXX)")
    last = ""
    for cxx in cands:
        cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", str(TORCH_OPS_SRC),
               "-o", str(tmp), f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
        for inc in ce.include_paths() + [str(Path(cuda_home) / "include")]:
            cmd += ["-isystem", inc]
        for lib in ce.library_paths():
            cmd += ["-L", lib]
        cmd += ["-L", str(LIB_DIR), "-lasymgemm_b200", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch", "-Wl,-rpath,$ORIGIN"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            last = f"{cxx}: building the torch extension failed:\n{res.stdout}\n{res.stderr}"
            continue
        if b"libstdc++.so" not in _needed_libraries(tmp):
            last = f"{cxx} linked libstdc++ statically into the torch extension"
            continue
        break
    else:
        raise RuntimeError(last)
    os.replace(tmp, TORCH_OPS_PATH)
    return TORCH_OPS_PATH


def _needed_libraries(path: Path) -> bytes:
    """The DT_NEEDED lines of a shared library as readelf prints them. Without readelf the check cannot be made and the
    library is accepted as built."""
    readelf = shutil.which("readelf")
    if readelf is None:
        return b"libstdc++.so (unchecked: readelf not found)"
    res = subprocess.run([readelf, "-d", str(path)], capture_output=True)
    return b"\n".join(ln for ln in res.stdout.splitlines() if b"NEEDED" in ln)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a, link the shared library, then build the torch extension over it.
    Returns the path of the C library."""
    _build_c_library(force, verbose)
    build_torch_ops(force)
    return LIB_PATH


def _build_c_library(force: bool, verbose: bool) -> Path:
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
