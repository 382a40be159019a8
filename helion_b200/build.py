"""Builds ``libhelion_b200.so`` (the sm_100a kernels behind the C ABI) in-tree with nvcc.

``python -m helion_b200.build`` compiles every ``csrc/*.cu`` for sm_100a and links
one shared library next to this file.  Objects are rebuilt only when their source
(or a header) is newer, so repeated calls are cheap.  No torch headers are
involved: the library depends on the CUDA runtime and driver only.
"""

from __future__ import annotations

import os
from pathlib import Path
import shutil
import subprocess
import sys

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
BUILD_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libhelion_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile and link the shared library; returns its path."""
    nvcc = _nvcc()
    BUILD_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_mtime = _newest_header_mtime()
    objects = []
    procs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_mtime)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
                print(" ".join(cmd), file=sys.stderr)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out, file=sys.stderr)
        if proc.returncode != 0:
            failed.append((src, out))
    if failed:
        msg = "\n".join(f"--- {src.name} ---\n{out}" for src, out in failed)
        raise RuntimeError(f"nvcc failed:\n{msg}")
    relink = force or bool(procs) or not LIB_PATH.exists()
    if relink:
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objects)]
        res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print(path)
