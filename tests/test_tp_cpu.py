"""Tensor-parallel host logic on two gloo ranks (no GPU): the shard rules give, after the
all-reduces the reference performs, the unsharded model's logits."""
import socket

import torch
import torch.multiprocessing as mp

from tests import tp_workers


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_sharded_oracle_equals_unsharded_on_two_gloo_ranks(tmp_path):
    out = tmp_path / "tp_cpu.pt"
    mp.spawn(tp_workers.cpu_oracle_worker, args=(2, _free_port(), str(out)), nprocs=2, join=True)
    r = torch.load(out)
    assert torch.allclose(r["got"], r["want"], atol=2e-5, rtol=1e-5)


def test_shard_shapes_follow_the_reference_rules(pkg):
    """tests/layers/test_linear.cpp:101-123 (TP shard shapes) on the packed layouts."""
    from oracle import token_loop_oracle as O
    from sglang_cpp_b200 import tp

    cfg = O.ModelConfig(1, 256, 8, 4, 128, 512, 64, tie_word_embeddings=False)
    w = O.init_weights(cfg, seed=1)
    for size in (1, 2, 4):
        for rank in range(size):
            L = tp.shard_layer(cfg, w["layers"][0], rank, size)
            assert L["qkv"].shape == ((8 + 2 * 4) * 128 // size, 256)
            assert L["o"].shape == (256, 8 * 128 // size)
            assert L["gate_up"].shape == (2 * 512 // size, 256)
            assert L["down"].shape == (256, 512 // size)
    # the shards tile the full matrices
    full = w["layers"][0]["down"]
    assert torch.equal(torch.cat([tp.shard_layer(cfg, w["layers"][0], r, 4)["down"] for r in range(4)], 1), full)
    import pytest
    with pytest.raises(ValueError):
        tp.shard_layer(cfg, w["layers"][0], 0, 3)   # 8 q heads are not divisible by 3
