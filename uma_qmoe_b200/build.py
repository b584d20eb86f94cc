"""Build ``libumaq_b200.so`` in-tree with nvcc for sm_100a.

    python -m uma_qmoe_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library links the CUDA runtime
statically and resolves driver entry points at run time, so it also loads (for
symbol checks) on a machine without a driver.
"""

from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
INCLUDE = PACKAGE.parent / "include"
LIBRARY = PACKAGE / "libumaq_b200.so"
STAMP = PACKAGE / "libumaq_b200.so.sha256"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_sha256() -> str:
    """Digest over name + NUL + bytes of every native source and header, the same
    construction the reference uses for its kernel identity
    (``src/uma_qmoe/native_backend.py:32-38``)."""
    digest = hashlib.sha256()
    for path in sorted([*CSRC.glob("*.cu"), *CSRC.glob("*.cuh"), *INCLUDE.glob("*.h")]):
        digest.update(path.name.encode("utf-8"))
        digest.update(b"\0")
        digest.update(path.read_bytes())
    return digest.hexdigest()


def nvcc_path() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; libumaq_b200.so cannot be built")
    return found


def build(force: bool = False, verbose: bool = False) -> Path:
    want = source_sha256()
    if not force and LIBRARY.exists() and STAMP.exists() and STAMP.read_text().strip() == want:
        return LIBRARY
    cmd = [nvcc_path(), *NVCC_FLAGS, "-I", str(INCLUDE), "-o", str(LIBRARY), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=str(CSRC))
    if verbose or proc.returncode:
        print(" ".join(cmd))
        print(proc.stdout)
        print(proc.stderr)
    if proc.returncode:
        raise RuntimeError(f"nvcc failed with exit code {proc.returncode}")
    STAMP.write_text(want + "\n")
    (PACKAGE / "libumaq_b200.ptxas.log").write_text(proc.stderr)
    return LIBRARY


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
