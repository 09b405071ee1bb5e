"""Builds ``oracle/_ref/libsglang_ref_cpu.so`` from the reference's own sources — TEST INFRASTRUCTURE ONLY.

Only the parts of the reference's path that are CPU-capable and self-contained are compiled: the
MoE layer (src/moe/moe.cc) and the integer side that defines table rows, KV slots and prefix-match
lengths (Req, RadixTreeNode / RadixPrefixCache, TableManager / CacheManager / PrefillManager,
DecodeManager).  The dense forward cannot be: its layers are CUDA-only and depend on
FlashInfer v0.2.0.post1, which the reference fetches at configure time and which is not on this
machine.  Sources are compiled from the reference tree where they lie; nothing is copied.
Needs the reference tree (REFERENCE_DIR, default: a `reference` directory beside this repository); without it the function
returns None and the golden fixtures committed under tests/golden/ stand in.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
OUT = OUT_DIR / "libsglang_ref_cpu.so"
# Paths inside the reference's src/ directory.
REF_SOURCES = [
    "moe/moe.cc",
    "core/req.cc", "core/batch.cc", "core/sampling_params.cc",
    "kernels/radix.cc",
    "kvcache/radix_tree.cc", "kvcache/cache_manager.cc",
    "scheduler/decode.cc", "scheduler/prefill.cc",
]
SHIMS = ["ref_shim.cc", "ref_sched_shim.cc"]


def _compile(src: Path, obj: Path, flags: list[str], verbose: bool) -> Path:
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, Path(__file__).stat().st_mtime):
        return obj
    cmd = ["g++", *flags, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {src} failed:\n{res.stderr[-4000:]}")
    return obj


def build(reference_dir: str | None = None, verbose: bool = False):
    ref = Path(reference_dir or os.environ.get("REFERENCE_DIR", str(HERE.parent.parent / "reference")))
    srcs = [ref / "src" / rel for rel in REF_SOURCES]
    if not all(src.exists() for src in srcs):
        return None
    import torch
    from torch.utils import cpp_extension

    OUT_DIR.mkdir(exist_ok=True)
    units = [(src, OUT_DIR / ("ref_" + src.stem + ".o")) for src in srcs]
    units += [(HERE / name, OUT_DIR / (Path(name).stem + ".o")) for name in SHIMS]
    tlib = Path(torch.__file__).parent / "lib"
    flags = ["-std=c++20", "-O1", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             *[f"-I{p}" for p in cpp_extension.include_paths()], f"-I{ref / 'include'}"]
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(units), os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda u: _compile(u[0], u[1], flags, verbose), units))
    if OUT.exists() and OUT.stat().st_mtime >= max(o.stat().st_mtime for o in objs):
        return OUT
    cmd = ["g++", "-shared", "-o", str(OUT), *map(str, objs), f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-lc10",
           f"-Wl,-rpath,{tlib}"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"linking the reference's CPU-capable sources failed:\n{res.stderr[-4000:]}")
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
