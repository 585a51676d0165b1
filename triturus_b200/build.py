"""In-tree build of libtriturus_b200.so (the extern "C" launcher and the sm_100a kernels).

`python -m triturus_b200.build` compiles `csrc/api.cu` with nvcc for sm_100a only and leaves the shared
library next to this file, where `triturus_b200._native` loads it with ctypes.  nvcc cross-compiles, so no
GPU is needed to build.
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
LIB_PATH = PKG_DIR / "libtriturus_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(INCLUDE.glob("*.h"))


STAMP_PATH = LIB_PATH.with_suffix(".so.sources")  # digest of the sources the library was built from


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for src in _sources():
        h.update(src.name.encode())
        h.update(src.read_bytes())
    return h.hexdigest()


def is_stale() -> bool:
    """True when the library is missing or was built from other sources than the ones on disk.  The check is
    by content, not by time stamp: a copy of the tree to another machine must not look stale."""
    if not LIB_PATH.exists() or not STAMP_PATH.exists():
        return True
    return STAMP_PATH.read_text().strip() != _digest()


def find_nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc")
    if cand:
        return cand
    default = "/usr/local/cuda/bin/nvcc"
    return default if os.path.exists(default) else None


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is stale (or `force`); return its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libtriturus_b200.so (set NVCC or add nvcc to PATH)")
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    # one temporary file per process: ranks of one job that all find the library stale do not write into each
    # other's output, and os.replace makes whichever finishes last the library (they are identical)
    tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
    cmd += ["-o", str(tmp), *[str(p) for p in sorted(CSRC.glob("*.cu"))]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    STAMP_PATH.write_text(_digest() + "\n")
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
