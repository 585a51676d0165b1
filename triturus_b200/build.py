"""In-tree build of libtriturus_b200.so (the extern "C" launcher and the sm_100a kernels).

`python -m triturus_b200.build` compiles `csrc/api.cu` with nvcc for sm_100a only and leaves the shared
library next to this file, where `triturus_b200._native` loads it with ctypes.  nvcc cross-compiles, so no
GPU is needed to build.
"""

from __future__ import annotations

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


def is_stale() -> bool:
    """True when the library is missing or older than any of its sources."""
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    return any(src.stat().st_mtime > built for src in _sources())


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
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd += ["-o", str(tmp), *[str(p) for p in sorted(CSRC.glob("*.cu"))]]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, LIB_PATH)
    if verbose:
        sys.stderr.write(proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
