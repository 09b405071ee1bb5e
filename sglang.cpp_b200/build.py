"""Builds the C-ABI kernel library ``lib/libb200_token_loop.so`` with nvcc for sm_100a.

The library is built in-tree so that the compiled file travels with the source
tree; nothing is installed into site-packages.  Each ``.cu`` file is compiled to
an object (in parallel) and the objects are linked into one shared library with
the CUDA runtime linked statically, so loading it needs neither libcudart nor
libcuda on the loader path (the driver API entry point that TMA descriptors
need is looked up at run time).
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = LIB_DIR / "libb200_token_loop.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the kernel library cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp(src: Path, extra: list[str]) -> str:
    h = hashlib.sha256()
    h.update(src.read_bytes())
    for dep in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [PKG_DIR.parent / "include" / "b200_token_loop.h"]:
        h.update(dep.read_bytes())
    h.update(" ".join(extra).encode())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool, ptxas_v: bool) -> Path:
    obj = OBJ_DIR / (src.stem + ".o")
    stamp_file = OBJ_DIR / (src.stem + ".stamp")
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_v else [])
    stamp = _stamp(src, flags)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = [_nvcc(), *flags, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    if ptxas_v:
        (OBJ_DIR / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    stamp_file.write_text(stamp)
    return obj


def build(verbose: bool = False, ptxas_v: bool = False, force: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link the shared library."""
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    if force:
        for f in OBJ_DIR.glob("*.stamp"):
            f.unlink()
    srcs = _sources()
    workers = min(len(srcs), os.cpu_count() or 4)
    with concurrent.futures.ThreadPoolExecutor(max_workers=workers) as ex:
        objs = list(ex.map(lambda s: _compile_one(s, verbose, ptxas_v), srcs))
    newest = max(o.stat().st_mtime for o in objs)
    if not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < newest:
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static",
               "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, ptxas_v="--ptxas" in sys.argv, force="-f" in sys.argv)
    print(path)
