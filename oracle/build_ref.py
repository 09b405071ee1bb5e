"""Builds ``oracle/_ref/libsglang_ref_cpu.so`` from the reference's own sources — TEST INFRASTRUCTURE ONLY.

Only the part of the reference's path that is CPU-capable and self-contained is compiled: the MoE
layer (src/moe/moe.cc).  The dense forward cannot be: its layers are CUDA-only and depend on
FlashInfer v0.2.0.post1, which the reference fetches at configure time and which is not on this
machine.  Sources are compiled from the reference tree where they lie; nothing is copied.
Needs the reference tree (REFERENCE_DIR, default: a `reference` directory beside this repository); without it the function
returns None and the golden fixtures committed under tests/golden/ stand in.
"""
from __future__ import annotations

import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "libsglang_ref_cpu.so"


def build(reference_dir: str | None = None, verbose: bool = False):
    ref = Path(reference_dir or os.environ.get("REFERENCE_DIR", str(HERE.parent.parent / "reference")))
    src = ref / "src" / "moe" / "moe.cc"
    if not src.exists():
        return None
    import torch
    from torch.utils import cpp_extension

    OUT.parent.mkdir(exist_ok=True)
    shim = HERE / "ref_shim.cc"
    if OUT.exists() and OUT.stat().st_mtime >= max(src.stat().st_mtime, shim.stat().st_mtime):
        return OUT
    tlib = Path(torch.__file__).parent / "lib"
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [f"-I{ref / 'include'}"]
    cmd = ["g++", "-std=c++20", "-O2", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *inc, str(src), str(shim), "-o", str(OUT), f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10",
           f"-Wl,-rpath,{tlib}"]
    if verbose:
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building the reference MoE layer failed:\n{res.stderr[-4000:]}")
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
