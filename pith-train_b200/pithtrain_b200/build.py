"""Builds ``libpith_b200.so`` (the C-ABI library holding every sm_100a kernel) in-tree with nvcc.

Usage: ``python -m pithtrain_b200.build [--force] [--verbose]`` or ``build_library()``.
The library is written next to this file so that it travels with the source tree.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR.parent / "csrc"
INCLUDE_DIR = PKG_DIR.parent.parent / "include"
BUILD_DIR = CSRC_DIR / "build"
LIB_PATH = Path(os.environ.get("PITH_B200_LIB", PKG_DIR / "libpith_b200.so"))

SOURCES = ["host_common.cu", "elementwise.cu", "attn_fwd.cu", "attn_fwd_pair.cu", "attn_bwd.cu", "attn_bwd128.cu", "noalloc.cu", "peer.cu",
           "qk_norm_rope.cu", "mla_assemble.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the pith_b200 kernels cannot be built")
    return exe


def _sources() -> list[Path]:
    return [CSRC_DIR / s for s in SOURCES if (CSRC_DIR / s).exists()]


def _fingerprint() -> str:
    h = hashlib.sha256()
    files = sorted(list(CSRC_DIR.glob("*.cu")) + list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h"))
                   + list(INCLUDE_DIR.glob("*.h")))
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    stamp = BUILD_DIR / "fingerprint"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text() == _fingerprint()


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every kernel for sm_100a and links the shared library. Returns its path.

    Safe to call from several processes at once (one rank per GPU all call it): builders take a file lock, look
    again under the lock, and the finished library is moved into place in one step, so nobody loads a half-written
    file."""
    if not force and is_current():
        return LIB_PATH
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    with open(BUILD_DIR / "lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not force and is_current():  # another process built it while this one waited
                return LIB_PATH
            return _build_locked(verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(verbose: bool) -> Path:
    nvcc = _nvcc()
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(INCLUDE_DIR), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{r.stdout}{r.stderr}\n")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, _sources()))
    tmp = LIB_PATH.with_name(LIB_PATH.name + f".tmp{os.getpid()}")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link of libpith_b200.so failed")
    os.replace(tmp, LIB_PATH)
    (BUILD_DIR / "fingerprint").write_text(_fingerprint())
    return LIB_PATH


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
