"""Build libb200sparse.so (sm_100a only) next to this file.

``python -m flagsparse_b200._build`` compiles every ``csrc/*.cu`` with nvcc and links one shared
library.  Objects are rebuilt only when a source or header is newer.  nvcc cross-compiles without
a GPU, so this also runs on a CPU-only machine.

Two more libraries come from the same sources:

* ``libb200sparse_checked.so`` (``build(checked=True)``, ``--checked``): compiled with
  ``-DB2S_CHECKED``; every column index and row pointer a kernel reads from the matrix is
  range-checked before it is used as an address, and a violation sets ``B2S_ERR_BOUNDS`` in the
  device status word instead of touching memory.  Slower; stands in for a memory checker when
  raw C-ABI callers pass matrices nobody validated.  ``B200SPARSE_CHECKED=1`` makes
  ``flagsparse_b200._lib`` load it.
* ``libb2sprobe.so`` (``build_probe()``, ``--probe``): the gather-rate probe ``bench.py`` times;
  not part of the product library.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
BUILD_DIR = PKG_DIR / "csrc" / "build"
LIB_PATH = PKG_DIR / "libb200sparse.so"
CHECKED_LIB_PATH = PKG_DIR / "libb200sparse_checked.so"
PROBE_LIB_PATH = PKG_DIR / "libb2sprobe.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: libb200sparse.so cannot be built")


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), checked: bool = False) -> Path:
    nvcc = _nvcc()
    build_dir = BUILD_DIR / "checked" if checked else BUILD_DIR
    lib_path = CHECKED_LIB_PATH if checked else LIB_PATH
    if checked:
        extra_flags = (*extra_flags, "-DB2S_CHECKED")
    build_dir.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "b200sparse.h"]

    def compile_one(src: Path) -> Path:
        obj = build_dir / (src.stem + ".o")
        if force or _newer(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-c", str(src), "-o", str(obj)]
            if verbose:
                print(" ".join(cmd), flush=True)
            res = subprocess.run(cmd, capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
            if verbose and res.stderr:
                print(res.stderr, flush=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))

    if force or _newer(lib_path, objects):
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(lib_path), *map(str, objects)]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


def build_probe(force: bool = False) -> Path:
    """libb2sprobe.so from csrc/probe/b2s_probe.cu (measurement aid of bench.py)."""
    src = CSRC / "probe" / "b2s_probe.cu"
    if force or _newer(PROBE_LIB_PATH, [src]):
        cmd = [_nvcc(), *NVCC_FLAGS, "-shared", str(src), "-o", str(PROBE_LIB_PATH)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    return PROBE_LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True,
                 extra_flags=("-Xptxas", "-v") if "--ptxas" in sys.argv else (),
                 checked="--checked" in sys.argv)
    print(path)
    if "--probe" in sys.argv:
        print(build_probe(force="--force" in sys.argv))
