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


def kv_heads_of_rank(num_kv_heads: int, rank: int, size: int) -> tuple[int, int]:
    """(first KV head, number of KV heads) of a rank.  With fewer KV heads than ranks each KV head
    is replicated on size / num_kv_heads consecutive ranks, which split the query heads of its
    group between them (the reference requires num_kv_heads % tp_size == 0 instead)."""
    if num_kv_heads >= size:
        n = divide_even(num_kv_heads, size, "num_kv_heads")
        return rank * n, n
    rep = divide_even(size, num_kv_heads, "tp_size (as a multiple of num_kv_heads)")
    return rank // rep, 1


def shard_layer(cfg, L: dict, rank: int, size: int, expert_parallel: bool = False) -> dict:
    """One decoder layer's tensors for `rank` of `size`, in the packed layouts the engine loads.
    expert_parallel: give the rank whole experts [rank * E / size, (rank + 1) * E / size) instead of
    a slice of every expert's intermediate dimension."""
    d = cfg.head_dim
    hq = divide_even(cfg.num_qo_heads, size, "num_qo_heads")
    kv0, hkv = kv_heads_of_rank(cfg.num_kv_heads, rank, size)
    qd, kd = cfg.num_qo_heads * d, cfg.num_kv_heads * d

    def rows(t, n):
        return t[rank * n:(rank + 1) * n]

    def kv_rows(t):
        return t[kv0 * d:(kv0 + hkv) * d]

    out = {}
    w = L["qkv"]
    out["qkv"] = torch.cat([rows(w[:qd], hq * d), kv_rows(w[qd:qd + kd]), kv_rows(w[qd + kd:])], 0)
    if "qkv_bias" in L:
        b = L["qkv_bias"]
        out["qkv_bias"] = torch.cat([rows(b[:qd], hq * d), kv_rows(b[qd:qd + kd]), kv_rows(b[qd + kd:])], 0)
    out["o"] = L["o"][:, rank * hq * d:(rank + 1) * hq * d].contiguous()
    for k in ("input_norm", "post_norm", "q_norm", "k_norm", "router"):
        if k in L:
            out[k] = L[k]
    if "experts_gate_up" in L and expert_parallel:
        el = divide_even(cfg.num_experts, size, "num_experts")
        out["experts_gate_up"] = L["experts_gate_up"][rank * el:(rank + 1) * el].contiguous()
        out["experts_down"] = L["experts_down"][rank * el:(rank + 1) * el].contiguous()
    elif "experts_gate_up" in L:
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


def shard_weights(cfg, w: dict, rank: int, size: int, expert_parallel: bool = False) -> dict:
    """All weights of one rank (embedding, lm_head and the final norm replicated)."""
    return {"embed": w["embed"], "lm_head": w["lm_head"], "final_norm": w["final_norm"],
            "layers": [shard_layer(cfg, L, rank, size, expert_parallel) for L in w["layers"]]}


def local_config(cfg, size: int, expert_parallel: bool = False):
    """The per-rank view of a model config: heads and intermediate sizes divided by tp_size (under
    expert parallelism the expert intermediate size stays whole; the rank's experts are a slice of
    the router's range, see shard_layer)."""
    c = copy.copy(cfg)
    c.num_qo_heads = divide_even(cfg.num_qo_heads, size, "num_qo_heads")
    c.num_kv_heads = kv_heads_of_rank(cfg.num_kv_heads, 0, size)[1]
    if cfg.num_experts > 0 and expert_parallel:
        pass
    elif cfg.num_experts > 0:
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
