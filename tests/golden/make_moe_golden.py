"""Generates tests/golden/moe_ref_fp32.json by running the reference's own MoELayer::forward.

Needs the reference tree: oracle/build_ref.py compiles its src/moe/moe.cc into
oracle/_ref/libsglang_ref_cpu.so, which this script calls through ctypes on seeded fp32 inputs.
Case "top2_renorm" uses the router logits of the reference's own test
(tests/moe/test_moe.cpp:69-99: 6 tokens, 3 experts, top-2, renormalised, hidden 4, intermediate 5).

    python tests/golden/make_moe_golden.py
"""
import ctypes
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import build_ref  # noqa: E402


def run_ref(lib, hidden, logits, gate_up, down, top_k, renorm, act):
    T, H = hidden.shape
    E, I = gate_up.shape[0], down.shape[2]
    out = np.zeros((T, H), dtype=np.float32)
    err = ctypes.create_string_buffer(512)
    f = lambda a: np.ascontiguousarray(a, dtype=np.float32).ctypes.data_as(ctypes.c_void_p)
    rc = lib.ref_moe_forward(f(hidden), f(logits), f(gate_up), f(down), T, E, top_k, H, I, int(renorm),
                             act.encode(), out.ctypes.data_as(ctypes.c_void_p), err, 512)
    if rc != 0:
        raise RuntimeError(err.value.decode())
    return out


def main():
    path = build_ref.build()
    if path is None:
        raise SystemExit("the reference tree is not available; cannot regenerate the fixture")
    lib = ctypes.CDLL(str(path))
    gen = torch.Generator().manual_seed(0)
    cases = []

    def add(name, T, E, top_k, H, I, renorm, act, logits=None):
        hidden = torch.randn(T, H, generator=gen).numpy()
        gate_up = torch.randn(E, 2 * I, H, generator=gen).numpy()
        down = torch.randn(E, H, I, generator=gen).numpy()
        if logits is None:
            logits = torch.randn(T, E, generator=gen).numpy()
        out = run_ref(lib, hidden, logits, gate_up, down, top_k, renorm, act)
        cases.append({"name": name, "top_k": top_k, "renormalize": renorm, "activation": act,
                      "hidden": hidden.tolist(), "router_logits": np.asarray(logits).tolist(),
                      "gate_up": gate_up.tolist(), "down": down.tolist(), "out": out.tolist()})

    ref_logits = np.array([[5.0, 1.0, -2.0], [0.1, 3.0, 2.0], [-1.0, 0.0, 4.0], [2.0, 2.5, 0.0],
                           [0.0, -0.5, 1.5], [3.0, 0.0, 3.5]], dtype=np.float32)
    add("top2_renorm", 6, 3, 2, 4, 5, True, "silu", ref_logits)
    add("top1_no_renorm", 5, 4, 1, 8, 6, False, "silu")
    add("top8_of_16_renorm", 12, 16, 8, 16, 8, True, "silu")
    add("top2_gelu", 7, 5, 2, 8, 4, True, "gelu")
    out = Path(__file__).resolve().parent / "moe_ref_fp32.json"
    out.write_text(json.dumps({"generator": "tests/golden/make_moe_golden.py", "cases": cases}))
    print(out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
