"""Builds the link-time drop-in probe: the reference's own Engine with this directory's adapters.

The four translation units of the reference that call FlashInfer (src/layers/normalization.cu,
src/layers/rotary_embedding.cu, src/engine/sampling.cu, src/attention/flashinfer_backend.cu) are
left out; normalization_b200.cc, rotary_embedding_b200.cc, sampling_b200.cc and attn_backend_b200.cc
define the same C++ symbols on top of libb200_token_loop.so.  Every other source of the reference's
engine (core, utils, distributed, kernels, kvcache, layers, models, moe, engine) is compiled
UNCHANGED from the reference tree where it lies — nothing is copied — and linked with the adapters
and engine_probe.cc into ``adapters/build/engine_probe``.  The link leaves no undefined symbol, which
is the proof that the adapters cover what the reference's Engine needs from those four units.

Needs the reference tree (REFERENCE_DIR, default: a `reference` directory beside this repository)
and the LibTorch inside the torch wheel; returns None without the tree.  The binary is a test
artefact (tests/test_adapters_gpu.py runs it on a GPU); the kernel library itself never needs it.
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
OUT_DIR = HERE / "build"
PROBE = OUT_DIR / "engine_probe"
ADAPTERS = ["normalization_b200.cc", "rotary_embedding_b200.cc", "sampling_b200.cc", "attn_backend_b200.cc"]
# Paths inside the reference's src/ directory, compiled unchanged.
REF_CC = [
    "core/batch.cc", "core/context.cc", "core/req.cc", "core/sampling_params.cc",
    "utils/tensor_utils.cc", "distributed/distributed.cc", "kernels/radix.cc",
    "layers/linear.cc", "layers/embedding.cc", "layers/attention_layer.cc",
    "models/config.cc", "models/utils.cc", "models/llama.cc", "models/mistral.cc", "models/qwen.cc",
    "models/qwen3.cc", "models/qwen3_moe.cc", "models/weight_loader.cc",
    "moe/moe.cc", "engine/config.cc", "engine/engine.cc",
]
REF_CU = ["kernels/token_pool.cu", "kvcache/mha_kvcache.cu", "layers/activation.cu"]


def _site_packages() -> Path:
    import torch
    return Path(torch.__file__).resolve().parent.parent


def _run(cmd, what):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"{what} failed:\n{' '.join(map(str, cmd))}\n{res.stderr[-6000:]}")


def _stale(obj: Path, src: Path) -> bool:
    deps = [src, Path(__file__), HERE / "adapter_common.h", ROOT / "include" / "b200_token_loop.h"]
    return not obj.exists() or obj.stat().st_mtime < max(d.stat().st_mtime for d in deps)


def build(reference_dir: str | None = None, verbose: bool = False):
    ref = Path(reference_dir or os.environ.get("REFERENCE_DIR", str(ROOT.parent / "reference")))
    if not (ref / "src" / "engine" / "engine.cc").exists():
        return None
    import torch
    from torch.utils import cpp_extension

    sp = _site_packages()
    OUT_DIR.mkdir(exist_ok=True)
    abi = f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [
        f"-I{ref / 'include'}", f"-I{ROOT / 'include'}", f"-I{HERE}", "-I/usr/local/cuda/include",
        f"-I{sp / 'nvidia' / 'nccl' / 'include'}", f"-I{sp / 'include' / 'cudnn_frontend' / 'thirdparty'}",
        f"-I{sp / 'flashinfer' / 'data' / 'include'}",
    ]
    cxx = ["g++", "-std=c++20", "-O1", "-fPIC", abi, *inc]
    nvcc = ["/usr/local/cuda/bin/nvcc", "-std=c++20", "-O1", "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", abi, *inc]
    units = [(HERE / a, OUT_DIR / (Path(a).stem + ".o"), cxx) for a in ADAPTERS]
    units.append((HERE / "engine_probe.cc", OUT_DIR / "engine_probe.o", cxx))
    units += [(ref / "src" / s, OUT_DIR / ("ref_" + s.replace("/", "_").replace(".cc", ".o")), cxx) for s in REF_CC]
    units += [(ref / "src" / s, OUT_DIR / ("ref_" + s.replace("/", "_").replace(".cu", ".o")), nvcc) for s in REF_CU]

    def compile_one(u):
        src, obj, tool = u
        if _stale(obj, src):
            if verbose:
                print("compile", src, flush=True)
            _run([*tool, "-c", str(src), "-o", str(obj)], f"compiling {src}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        objs = list(ex.map(compile_one, units))
    if PROBE.exists() and PROBE.stat().st_mtime >= max(o.stat().st_mtime for o in objs):
        return PROBE
    tlib = sp / "torch" / "lib"
    nccl = sp / "nvidia" / "nccl" / "lib"
    klib = ROOT / "sglang.cpp_b200" / "lib"
    link = ["g++", "-o", str(PROBE), *map(str, objs), f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
            "-lc10_cuda", f"-L{nccl}", "-l:libnccl.so.2", "-L/usr/local/cuda/lib64", "-lcudart",
            f"-L{klib}", "-lb200_token_loop", "-lpthread", "-ldl",
            f"-Wl,-rpath,{tlib}", f"-Wl,-rpath,{nccl}", "-Wl,-rpath,/usr/local/cuda/lib64", "-Wl,-rpath,$ORIGIN/../../lib",
            "-Wl,--no-undefined", "-Wl,--no-as-needed"]
    if verbose:
        print(" ".join(link), flush=True)
    _run(link, "linking engine_probe")
    return PROBE


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv))
