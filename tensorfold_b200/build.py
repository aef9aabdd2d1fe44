"""Ahead-of-time build of the sm_100a kernel library (no JIT at import).

``python -m tensorfold_b200.build`` compiles every ``csrc/*.cu`` with nvcc into
``tensorfold_b200/libtensorfold_b200.so`` next to this file. The library is plain C ABI
(``include/tensorfold_b200.h``); Python reaches it through ctypes, so no torch headers are involved
and the build needs only nvcc.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "libtensorfold_b200.so"
OBJ = HERE / "build"
STAMP = OBJ / "sources.sha256"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--fmad=false",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found: the kernel library cannot be built")
    return found


def source_hash() -> str:
    """Hash of every kernel source and header: a saved state is only valid for the same kernels."""

    h = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "tensorfold_b200.h"]):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    digest = source_hash()
    if not force and LIB.exists() and STAMP.exists() and STAMP.read_text().strip() == digest:
        return LIB
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(CSRC.glob("*.cu"))

    def compile_one(src: Path) -> Path:
        obj = OBJ / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode:
            sys.stderr.write(res.stdout + res.stderr)
        if res.returncode:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources))
    res = subprocess.run([nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-gencode",
                          "arch=compute_100a,code=sm_100a"], capture_output=True, text=True)
    if res.returncode:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    STAMP.write_text(digest + "\n")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
