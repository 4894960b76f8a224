"""Builds the native library in-tree with nvcc for sm_100a.

``python -m flagdnn_b200.build`` compiles ``csrc/*.cu`` into
``flagdnn_b200/libflagdnn_b200.so``.  nvcc cross-compiles without a GPU, so
this runs on build machines that have none.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libflagdnn_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--threads", "4",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB_PATH.exists():
        return True
    built = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*")) + [PKG_DIR.parent / "include" / "flagdnn_b200.h"]
    return any(p.stat().st_mtime > built for p in deps if p.exists())


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and not _stale():
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", str(LIB_PATH)]
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(s) for s in sources()]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose or ptxas_info:
        sys.stderr.write(proc.stdout + proc.stderr)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(LIB_PATH)
