"""Build the sm_100a kernel library in-tree with nvcc.

The library is a plain C-ABI shared object (``libjb_kernels.so``) next to this file, loaded
with :mod:`ctypes`.  It is compiled for ``sm_100a`` only; nvcc cross-compiles on a machine
without a GPU.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_PATH = HERE / "libjb_kernels.so"
_STAMP = HERE / "libjb_kernels.stamp"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-shared",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def source_hash() -> str:
    """Hash of every file under ``csrc`` (rebuild trigger)."""
    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*")):
        if p.suffix in (".cu", ".cuh", ".h"):
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_fresh() -> bool:
    return LIB_PATH.exists() and _STAMP.exists() and _STAMP.read_text().strip() == source_hash()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile ``csrc/jb_kernels.cu`` into ``libjb_kernels.so`` if the sources changed."""
    if not force and is_fresh():
        return LIB_PATH
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found; cannot build jigsaw_b200 kernels")
    tmp = LIB_PATH.with_suffix(".so.tmp%d" % os.getpid())
    cmd = [nvcc, *NVCC_FLAGS, "-o", str(tmp), str(CSRC / "jb_kernels.cu")]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        print(proc.stderr)
    os.replace(tmp, LIB_PATH)
    _STAMP.write_text(source_hash())
    return LIB_PATH


if __name__ == "__main__":
    import sys

    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
