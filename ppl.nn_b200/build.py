"""Build recipe for the CUDA library (sm_100a only) and the C++ host layer.

``build()`` runs nvcc on every source under csrc/ (and host/) and writes
``lib/libppl_nn_b200.so`` next to this file.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
HOST = HERE / "host"
LIB_DIR = HERE / "lib"
LIB = LIB_DIR / "libppl_nn_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-shared",
    # no fast-math: the quantiser relies on IEEE division and rounding to be bit-reproducible
]


def sources() -> list[Path]:
    srcs = sorted(CSRC.glob("*.cu")) + sorted(HOST.glob("*.cc"))
    return srcs


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def needs_build() -> bool:
    if not LIB.exists():
        return True
    newest = max(p.stat().st_mtime for p in list(CSRC.iterdir()) + list(HOST.rglob("*")) + [HERE.parent / "include" / "ppl_nn_b200.h"] if p.is_file())
    return newest > LIB.stat().st_mtime


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(HERE.parent / "include"), "-I", str(HOST), "-x", "cu"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    tmp = LIB.with_suffix(".so.tmp")
    cmd += ["-o", str(tmp)] + [str(s) for s in sources()]
    subprocess.run(cmd, check=True)
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    import sys
    print(build(force=True, verbose="-v" in sys.argv))
