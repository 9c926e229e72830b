"""Ahead-of-time build of libb200_gemm.so (sm_100a only) with nvcc.

Replaces the reference's in-process JIT (`flyc.compile` through kernels/common.py:7-39): there is no
run-time compilation here, the shared library is built once and kept in-tree next to this file.

    python -m flydsl_examples_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = PKG_DIR / "libb200_gemm.so"
STAMP_PATH = PKG_DIR / "libb200_gemm.so.stamp"

SOURCES = [CSRC / name for name in ("gemm_api.cu", "variants_single_k128.cu", "variants_single_k64.cu", "variants_pair.cu",
                                    "variants_loader.cu")]
HEADERS = [CSRC / "gemm_kernel.cuh", CSRC / "aux_kernels.cuh", CSRC / "variants.h", CSRC / "ptx.cuh", INCLUDE / "b200_gemm.h"]
OBJ_DIR = PKG_DIR / "_obj"  # object files of the translation units (not shipped, not tracked)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]
# Not used: --split-compile. With it the same sources came out with half as much code again per kernel (about 196 KB
# instead of 123 KB for the 256-wide pair kernel) and ran 15-20 % slower on every shape, and whether that happened
# flipped with small unrelated edits. Build time is kept down by compiling the translation units side by side.


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(cand).exists():
        raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")
    return cand


def _source_digest() -> str:
    h = hashlib.sha256()
    for f in SOURCES + HEADERS:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP_PATH.exists() and STAMP_PATH.read_text().strip() == _source_digest()


def _compile_one(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = OBJ_DIR / (src.stem + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", f"-I{CSRC}", "-c"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(obj), str(src)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if the sources changed since the last build; return its path. The translation units are
    compiled side by side (one nvcc process each), then linked into one shared object."""
    if not force and is_current():
        return LIB_PATH
    import fcntl

    OBJ_DIR.mkdir(exist_ok=True)
    # One builder at a time: the ranks of a multi-GPU job import this package at the same moment, and the first one
    # that finds the library stale builds it while the others wait here and then find it current.
    with open(OBJ_DIR / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current():
            return LIB_PATH
        return _build_locked(verbose)


def _build_locked(verbose: bool) -> Path:
    from concurrent.futures import ThreadPoolExecutor

    with ThreadPoolExecutor(max_workers=len(SOURCES)) as pool:
        results = list(pool.map(lambda src: _compile_one(src, verbose), SOURCES))
    if verbose:
        for _, log in results:
            sys.stderr.write(log)
    cmd = [_nvcc(), "-shared", "-Wno-deprecated-gpu-targets", "-o", str(LIB_PATH), *[str(obj) for obj, _ in results]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("link failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    STAMP_PATH.write_text(_source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
