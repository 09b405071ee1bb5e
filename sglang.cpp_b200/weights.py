"""Checkpoint loading: safetensors shards -> the packed layouts the engine holds.

Restates the host side of the reference's loader (src/models/weight_loader.cc): the safetensors
header walk (:357-420), the name normalisation (:195-211), the merge of q/k/v into ``qkv_proj`` and
of gate/up into ``gate_up_proj`` (:27-41, 62-120) and the stacking of per-expert tensors into
``[E, ...]`` blocks (:43, 236-258).  Sharding for tensor / expert parallelism is done afterwards by
``tp.shard_layer`` when the engine uploads (``Engine.load_weights``).  Pure torch / numpy, no CUDA.

Not restated: the FP8 block-quantised checkpoints the reference dequantises at load (:213-234);
only BF16 / F16 / F32 tensors are accepted.
"""
from __future__ import annotations

import json
import re
import struct
from pathlib import Path

import numpy as np
import torch

_DTYPES = {"BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4)}
_EXPERT = re.compile(r"^(.*\.experts)\.(\d+)\.(.+)$")


def read_safetensors(path) -> dict:
    """name -> tensor for one ``.safetensors`` file (8-byte little-endian header length, a JSON
    header of dtype / shape / data_offsets, then the raw little-endian data).  The tensors are
    views of a read-only memory map."""
    path = Path(path)
    with open(path, "rb") as f:
        (hlen,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(hlen))
    data = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hlen)
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _DTYPES:
            raise ValueError(f"Unsupported safetensors dtype: {info['dtype']} ({name})")
        dtype, width = _DTYPES[info["dtype"]]
        lo, hi = info["data_offsets"]
        shape = tuple(info["shape"])
        n = int(np.prod(shape)) if shape else 1
        if hi - lo != n * width:
            raise ValueError(f"{name}: {hi - lo} bytes for shape {shape} of {info['dtype']}")
        buf = np.frombuffer(data[lo:hi], dtype=np.uint8)
        out[name] = torch.frombuffer(bytearray(buf.tobytes()), dtype=dtype).reshape(shape)
    return out


def write_safetensors(path, tensors: dict) -> None:
    """The inverse of read_safetensors (tests and tools; BF16 / F16 / F32 only)."""
    names = {v[0]: k for k, v in _DTYPES.items()}
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * (-len(h) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


def normalize_weight_name(name: str) -> str:
    """src/models/weight_loader.cc:195-200."""
    return name[len("language_model."):] if name.startswith("language_model.") else name


def pack_checkpoint(cfg, tensors: dict) -> dict:
    """Hugging Face parameter names -> {"embed", "lm_head", "final_norm", "layers": [...]} with
    qkv = cat(q, k, v), gate_up = cat(gate, up) and experts stacked, all cast to bf16 (the dtype
    the reference's ``model.to(device, dtype)`` ends with, weight_loader.cc:542)."""
    t = {normalize_weight_name(k): v for k, v in tensors.items()}
    bf = lambda x: x.to(torch.bfloat16).contiguous()

    def need(name):
        if name not in t:
            raise KeyError(f"checkpoint has no tensor {name}")
        return t[name]

    w = {"embed": bf(need("model.embed_tokens.weight")), "final_norm": bf(need("model.norm.weight")), "layers": []}
    w["lm_head"] = w["embed"] if cfg.tie_word_embeddings or "lm_head.weight" not in t else bf(t["lm_head.weight"])
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        L = {"qkv": bf(torch.cat([need(a + "q_proj.weight"), need(a + "k_proj.weight"), need(a + "v_proj.weight")], 0)),
             "o": bf(need(a + "o_proj.weight")),
             "input_norm": bf(need(p + "input_layernorm.weight")),
             "post_norm": bf(need(p + "post_attention_layernorm.weight"))}
        if cfg.attention_bias:
            L["qkv_bias"] = bf(torch.cat([need(a + "q_proj.bias"), need(a + "k_proj.bias"), need(a + "v_proj.bias")], 0))
        if cfg.qk_norm:
            L["q_norm"] = bf(need(a + "q_norm.weight"))
            L["k_norm"] = bf(need(a + "k_norm.weight"))
        m = p + "mlp."
        if cfg.num_experts > 0:
            L["router"] = bf(need(m + "gate.weight"))
            gu, dn = [], []
            for e in range(cfg.num_experts):
                x = f"{m}experts.{e}."
                gu.append(torch.cat([need(x + "gate_proj.weight"), need(x + "up_proj.weight")], 0))
                dn.append(need(x + "down_proj.weight"))
            L["experts_gate_up"] = bf(torch.stack(gu, 0))
            L["experts_down"] = bf(torch.stack(dn, 0))
        else:
            L["gate_up"] = bf(torch.cat([need(m + "gate_proj.weight"), need(m + "up_proj.weight")], 0))
            L["down"] = bf(need(m + "down_proj.weight"))
        w["layers"].append(L)
    _check_shapes(cfg, w)
    return w


def unpack_checkpoint(cfg, w: dict) -> dict:
    """Packed layouts -> Hugging Face parameter names (the inverse of pack_checkpoint)."""
    d = cfg.head_dim
    qd, kd = cfg.num_qo_heads * d, cfg.num_kv_heads * d
    out = {"model.embed_tokens.weight": w["embed"], "model.norm.weight": w["final_norm"]}
    if not cfg.tie_word_embeddings:
        out["lm_head.weight"] = w["lm_head"]
    for i, L in enumerate(w["layers"]):
        p = f"model.layers.{i}."
        a = p + "self_attn."
        out[a + "q_proj.weight"], out[a + "k_proj.weight"], out[a + "v_proj.weight"] = (
            L["qkv"][:qd], L["qkv"][qd:qd + kd], L["qkv"][qd + kd:])
        out[a + "o_proj.weight"] = L["o"]
        if "qkv_bias" in L:
            b = L["qkv_bias"]
            out[a + "q_proj.bias"], out[a + "k_proj.bias"], out[a + "v_proj.bias"] = b[:qd], b[qd:qd + kd], b[qd + kd:]
        if "q_norm" in L:
            out[a + "q_norm.weight"], out[a + "k_norm.weight"] = L["q_norm"], L["k_norm"]
        out[p + "input_layernorm.weight"] = L["input_norm"]
        out[p + "post_attention_layernorm.weight"] = L["post_norm"]
        m = p + "mlp."
        if "experts_gate_up" in L:
            ie = cfg.moe_intermediate_size
            out[m + "gate.weight"] = L["router"]
            for e in range(cfg.num_experts):
                x = f"{m}experts.{e}."
                out[x + "gate_proj.weight"] = L["experts_gate_up"][e, :ie]
                out[x + "up_proj.weight"] = L["experts_gate_up"][e, ie:]
                out[x + "down_proj.weight"] = L["experts_down"][e]
        else:
            I = cfg.intermediate_size
            out[m + "gate_proj.weight"], out[m + "up_proj.weight"] = L["gate_up"][:I], L["gate_up"][I:]
            out[m + "down_proj.weight"] = L["down"]
    return out


def load_checkpoint(cfg, directory) -> dict:
    """All ``*.safetensors`` shards of a directory, packed."""
    tensors = {}
    for f in sorted(Path(directory).glob("*.safetensors")):
        tensors.update(read_safetensors(f))
    if not tensors:
        raise FileNotFoundError(f"no .safetensors files under {directory}")
    return pack_checkpoint(cfg, tensors)


def _check_shapes(cfg, w: dict) -> None:
    d, H = cfg.head_dim, cfg.hidden_size
    qkv_out = (cfg.num_qo_heads + 2 * cfg.num_kv_heads) * d
    if tuple(w["embed"].shape) != (cfg.vocab_size, H):
        raise ValueError(f"embed_tokens has shape {tuple(w['embed'].shape)}, expected {(cfg.vocab_size, H)}")
    for i, L in enumerate(w["layers"]):
        want = {"qkv": (qkv_out, H), "o": (H, cfg.num_qo_heads * d)}
        if cfg.num_experts > 0:
            ie = cfg.moe_intermediate_size
            want.update(router=(cfg.num_experts, H), experts_gate_up=(cfg.num_experts, 2 * ie, H),
                        experts_down=(cfg.num_experts, H, ie))
        else:
            want.update(gate_up=(2 * cfg.intermediate_size, H), down=(H, cfg.intermediate_size))
        for k, shape in want.items():
            if tuple(L[k].shape) != shape:
                raise ValueError(f"layer {i} {k} has shape {tuple(L[k].shape)}, expected {shape}")
