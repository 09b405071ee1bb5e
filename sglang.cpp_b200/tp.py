"""Tensor-parallel sharding rules and the host side of the all-reduce set-up.

The shard rules restate the reference loader's (src/models/weight_loader.cc:284-353, 524-526):
q / k / v and gate / up are split by output rows (each half separately, then re-packed), o_proj and
down_proj by input columns, expert weights by the expert intermediate dimension; embeddings, lm_head
and norm weights are replicated (the models use nn::Embedding and LinearReplicated,
src/models/qwen3.cc:38-43,70-77).  Pure torch, no CUDA: the CPU tests run it under gloo.
"""
from __future__ import annotations

import copy

import torch


def divide_even(value: int, divisor: int, name: str) -> int:
    """src/distributed/distributed.cc:228-232."""
    if divisor <= 0 or value % divisor != 0:
        raise ValueError(f"{name} must be divisible by tp_size")
    return value // divisor


def shard_layer(cfg, L: dict, rank: int, size: int) -> dict:
    """One decoder layer's tensors for `rank` of `size`, in the packed layouts the engine loads."""
    d = cfg.head_dim
    hq = divide_even(cfg.num_qo_heads, size, "num_qo_heads")
    hkv = divide_even(cfg.num_kv_heads, size, "num_kv_heads")
    qd, kd = cfg.num_qo_heads * d, cfg.num_kv_heads * d

    def rows(t, n):
        return t[rank * n:(rank + 1) * n]

    out = {}
    w = L["qkv"]
    out["qkv"] = torch.cat([rows(w[:qd], hq * d), rows(w[qd:qd + kd], hkv * d), rows(w[qd + kd:], hkv * d)], 0)
    if "qkv_bias" in L:
        b = L["qkv_bias"]
        out["qkv_bias"] = torch.cat([rows(b[:qd], hq * d), rows(b[qd:qd + kd], hkv * d), rows(b[qd + kd:], hkv * d)], 0)
    out["o"] = L["o"][:, rank * hq * d:(rank + 1) * hq * d].contiguous()
    for k in ("input_norm", "post_norm", "q_norm", "k_norm", "router"):
        if k in L:
            out[k] = L[k]
    if "experts_gate_up" in L:
        ie = cfg.moe_intermediate_size
        il = divide_even(ie, size, "MoELayer intermediate size")
        gu = L["experts_gate_up"]
        out["experts_gate_up"] = torch.cat([gu[:, rank * il:(rank + 1) * il], gu[:, ie + rank * il:ie + (rank + 1) * il]], 1).contiguous()
        out["experts_down"] = L["experts_down"][:, :, rank * il:(rank + 1) * il].contiguous()
    else:
        I = cfg.intermediate_size
        il = divide_even(I, size, "LinearColParallelMerged output size")
        gu = L["gate_up"]
        out["gate_up"] = torch.cat([gu[rank * il:(rank + 1) * il], gu[I + rank * il:I + (rank + 1) * il]], 0)
        out["down"] = L["down"][:, rank * il:(rank + 1) * il].contiguous()
    return out


def shard_weights(cfg, w: dict, rank: int, size: int) -> dict:
    """All weights of one rank (embedding, lm_head and the final norm replicated)."""
    return {"embed": w["embed"], "lm_head": w["lm_head"], "final_norm": w["final_norm"],
            "layers": [shard_layer(cfg, L, rank, size) for L in w["layers"]]}


def local_config(cfg, size: int):
    """The per-rank view of a model config: heads and intermediate sizes divided by tp_size."""
    c = copy.copy(cfg)
    c.num_qo_heads = divide_even(cfg.num_qo_heads, size, "num_qo_heads")
    c.num_kv_heads = divide_even(cfg.num_kv_heads, size, "num_kv_heads")
    if cfg.num_experts > 0:
        c.moe_intermediate_size = divide_even(cfg.moe_intermediate_size, size, "MoELayer intermediate size")
    else:
        c.intermediate_size = divide_even(cfg.intermediate_size, size, "intermediate_size")
    return c


def exchange_handles(local_handle: bytes, rank: int, size: int, group=None) -> bytes:
    """Gather every rank's IPC handle in rank order over torch.distributed (any backend)."""
    import torch.distributed as dist

    gathered = [None] * size
    dist.all_gather_object(gathered, local_handle, group=group)
    return b"".join(gathered)
