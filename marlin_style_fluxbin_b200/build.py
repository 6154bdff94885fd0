"""Ahead-of-time build of the CUDA library (``libfluxbin_b200.so``) with nvcc for sm_100a.

The library is built in-tree, next to this file, so that it travels with the source tree.
``python -m marlin_style_fluxbin_b200.build`` rebuilds it; ``build()`` is incremental.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libfluxbin_b200.so"
STAMP = PACKAGE / "csrc" / ".build_stamp"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
# Per-file extras.  The GEMV kernels keep separate multiply and add, as the reference
# builds its kernels (--fmad=false), so that products are rounded where it rounds them.
EXTRA = {"fb_w3_gemv.cu": ["--fmad=false"], "fb_bb_gemv.cu": ["--fmad=false"]}


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _fingerprint() -> str:
    digest = hashlib.sha256()
    for path in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PACKAGE.parent / "include" / "fluxbin_b200.h", Path(__file__)]):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library."""
    fingerprint = _fingerprint()
    if not force and LIBRARY.exists() and STAMP.exists() and STAMP.read_text() == fingerprint:
        return LIBRARY
    nvcc = _nvcc()
    objects = []
    logs = []
    for source in sources():
        obj = source.with_suffix(".o")
        cmd = [nvcc, *ARCH, *COMMON, *EXTRA.get(source.name, []), "-c", str(source), "-o", str(obj)]
        done = subprocess.run(cmd, capture_output=True, text=True)
        logs.append(f"$ {' '.join(cmd)}\n{done.stdout}{done.stderr}")
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed on {source.name}:\n{done.stdout}{done.stderr}")
        objects.append(obj)
    cmd = [nvcc, *ARCH, "-shared", "-o", str(LIBRARY), *map(str, objects)]
    done = subprocess.run(cmd, capture_output=True, text=True)
    if done.returncode != 0:
        raise RuntimeError(f"link failed:\n{done.stdout}{done.stderr}")
    (CSRC / "ptxas_report.txt").write_text("\n".join(logs))
    STAMP.write_text(fingerprint)
    if verbose:
        print("\n".join(logs))
    return LIBRARY


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print(LIBRARY)
